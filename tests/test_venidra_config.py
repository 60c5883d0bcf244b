"""Venidra without a GPU: config.json reading and defaults, the specification it becomes, tensor names and shapes, cache
requests (one row of latents a token, pages of a chunk or a window given back), and the plain implementation's own
consistency."""
import copy
import math

import numpy as np
import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_venidra as plain
from dryft_challenge_htn_2026_b200.cache import Cache, KVRequest
from dryft_challenge_htn_2026_b200.config.specs import (GatedMLPSpec, LatentAttentionSpec, MaskedAttentionSpec, RMSNormSpec,
                                                        RotaryPairsSpec, RotaryPartSpec, SandwichLayerSpec, UnitRMSNormSpec)
from dryft_challenge_htn_2026_b200.engine.model import CausalLM

ATT = {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.3, "v_mix": True,
                                      "rot": {"dims": 4, "base": 1000.0}, "mask": {"size": 20}},
       "mlp": {"kind": "dense", "ff": 48}}
LAT = {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 12, "q_rank": 10, "kv_rank": 14, "scale": 0.25,
                                             "rot": {"base": 300.0, "dims": 4}, "mask": {"size": 9}},
       "mlp": None}
BASE = dict(architecture="Venidra", vocab=90, width=32, norm={"eps": 2e-6}, embedding={"scale": 1.5}, logit_scale=0.7,
            logit_softcap=12.0, layers=[copy.deepcopy(l) for l in (LAT, ATT, dict(ATT, mlp=None), LAT, ATT)])


def test_config_round_trip_and_registry():
    cfg = dk.config_from_dict(BASE)
    assert type(cfg).__name__ == "VenidraConfig" and "Venidra" in dk.architectures()
    assert dk.config_from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"][1]["mixer"]["mask"] == {"size": 20} and cfg.to_dict()["layers"][0]["mlp"] is None


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="conv"), "not implemented"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), "multiple"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "not implemented"),
    (lambda d: d["layers"][0]["mixer"].pop("rot"), "rot"),
    (lambda d: d["layers"][4]["mixer"].update(vdim=16), "one shape"),
    (lambda d: d.update(logit_softcap=-1.0), "negative"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(layers=[]), "non-empty"),
])
def test_config_errors(change, message):
    d = copy.deepcopy(BASE)
    change(d)
    with pytest.raises(dk.ConfigError, match=message):
        dk.config_from_dict(d)


def test_spec_carries_every_constant():
    spec = dk.config_from_dict(BASE).to_spec()
    assert (spec.embed_scale, spec.logit_scale, spec.logit_cap, spec.tie_embeddings) == (1.5, 0.7, 12.0, True)
    assert spec.final_norm == RMSNormSpec(32, 2e-6, tensor="") and len(spec.layers) == len(spec.schedule) == 5
    l0, l1, l2, l3, l4 = spec.layers
    assert all(isinstance(l, SandwichLayerSpec) for l in spec.layers)
    m = l1.mixer
    assert isinstance(m, MaskedAttentionSpec) and (m.num_heads, m.num_kv_heads, m.head_dim, m.v_head_dim) == (6, 2, 16, 8)
    assert (m.chunk, m.window, m.scale, m.norm_after_rotation, m.value_mix) == (20, None, 0.3, True, "source")
    assert m.position == RotaryPartSpec(4, 1000.0) and m.qk_norm == UnitRMSNormSpec(16, 2e-6)
    assert l2.mixer.value_mix == "blend" and l4.mixer.value_mix == "blend"
    assert l1.feed_forward == GatedMLPSpec(32, 48, "gelu_tanh", names=("gate", "up", "down"))
    assert l2.feed_forward is None and l2.norm_post is None and l2.norm_ff_out is None and l2.norm_mix_out is not None
    m = l0.mixer
    assert isinstance(m, LatentAttentionSpec) and (m.num_heads, m.head_dim, m.rot_dim, m.v_head_dim, m.q_rank, m.kv_rank) == (3, 8, 4, 12, 10, 14)
    assert (m.window, m.chunk, m.scale, m.norm_eps, m.position) == (9, None, 0.25, 2e-6, RotaryPairsSpec(4, 300.0))


def test_what_a_config_leaves_out():
    d = copy.deepcopy(BASE)
    d["layers"] = [copy.deepcopy(ATT), copy.deepcopy(LAT)]
    for k in ("kv_heads", "vdim", "rot", "mask", "v_mix"):
        d["layers"][0]["mixer"].pop(k)
    d["layers"][1]["mixer"].pop("mask")
    d["layers"][1]["mixer"]["rot"].pop("dims")
    for k in ("embedding", "logit_scale", "logit_softcap"):
        d.pop(k)
    spec = dk.config_from_dict(d).to_spec()
    m = spec.layers[0].mixer
    assert (m.num_kv_heads, m.v_head_dim, m.position, m.chunk, m.value_mix) == (6, 16, None, None, None)
    assert spec.layers[1].mixer.window is None and spec.layers[1].mixer.position == RotaryPairsSpec(4, 300.0)
    assert (spec.embed_scale, spec.logit_scale, spec.logit_cap) == (1.0, 1.0, None)
    # a blending weight that comes with a layer that does not blend is nobody's
    assert spec.unused_tensors == ("l0.mix.vmix",)


def test_tensor_names_and_shapes():
    decls = CausalLM(dk.config_from_dict(BASE).to_spec(), torch.float32, "cpu").param_decls(True)
    shapes = {k: tuple(v.shape) for k, v in decls.items()}
    want = {"embed": (90, 32), "final.norm": (32,), "l0.norm1": (32,), "l0.norm1b": (32,), "l0.mix.dq": (10, 32), "l0.mix.dq.norm": (10,),
            "l0.mix.uq": (36, 10), "l0.mix.dkv": (18, 32), "l0.mix.dkv.norm": (14,), "l0.mix.uk": (24, 14), "l0.mix.uv": (36, 14),
            "l0.mix.o": (32, 36), "l1.norm1": (32,), "l1.norm1b": (32,), "l1.norm2": (32,), "l1.norm2b": (32,), "l1.mix.q": (96, 32),
            "l1.mix.k": (32, 32), "l1.mix.v": (16, 32), "l1.mix.vmix": (), "l1.mix.o": (32, 48), "l1.mlp.gate": (48, 32),
            "l1.mlp.up": (48, 32), "l1.mlp.down": (32, 48), "l2.mix.vmix": (), "l4.mix.vmix": ()}
    for k, v in want.items():
        assert shapes[k] == v, (k, shapes.get(k))
    assert "head" not in shapes and "l0.norm2" not in shapes and "l2.norm2b" not in shapes and "l2.mlp.up" not in shapes
    assert decls["l0.mix.dq.norm"].keep_float32 and decls["l1.norm1b"].keep_float32 and decls["l1.mix.vmix"].keep_float32


def test_a_token_holds_one_row_of_latents_and_pages_behind_the_mask_go_back():
    model = CausalLM(dk.config_from_dict(BASE).to_spec(), torch.float32, "cpu")
    reqs = model.entry_requests()
    # key row [latent | rotated part]; the value row is its start, so the cache keeps no values of its own
    assert reqs[0] == reqs[3] == [KVRequest(1, 18, 9, torch.float32, 14, None, 0, True)]
    assert reqs[1] == reqs[2] == reqs[4] == [KVRequest(2, 16, None, torch.float32, 8, 20)]
    held = Cache(reqs, 64 * 8, 2, "cpu")
    per_token = [g.bytes() // (len(g.entries) * held.num_pages * 64) for g in held.groups]
    assert sorted(per_token) == [4 * 18, 4 * 2 * (16 + 8)], per_token                     # 18 numbers a token and latent layer
    assert all(held.views(e)[0].v is None for e in (0, 3)) and held.views(1)[0].v is not None
    cache = Cache(reqs, 64 * 8, 2, "cpu", allocate=False)
    s = cache.begin()
    cache.reserve(s, 200)
    cache.commit(s, 200)
    for g in cache.groups:      # a window of 9 or a chunk of 20 behind position 199: only the last page is still held
        assert [p >= 0 for p in g.pages[s][:4]] == [False, False, False, True], g.pages[s][:4]
    cache.end(s)
    assert all(f == cache.num_pages for f in cache.pages_free())


def test_plain_masks_and_rotations():
    m = plain.chunk_mask(10, 4)
    assert m[5].tolist() == [False] * 4 + [True, True] + [False] * 4 and m[4].tolist() == [False] * 4 + [True] + [False] * 5
    m = plain.window_mask(10, 3)
    assert m[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4 and m[1].tolist() == [True, True] + [False] * 8
    a = plain.angles(3, 4, 100.0)
    assert a.shape == (3, 2) and abs(float(a[2, 1]) - 2 * 100.0 ** -0.5) < 1e-6
    x = torch.arange(12, dtype=torch.float64).view(1, 1, 12).repeat(3, 1, 1)
    h, p = plain.rotate_halves(x, a), plain.rotate_pairs(x, a)
    assert torch.equal(h[0], x[0]) and torch.equal(p[0], x[0]) and torch.equal(h[..., 4:], x[..., 4:])      # position 0; the rest passes
    c, s = math.cos(float(a[2, 0])), math.sin(float(a[2, 0]))
    assert abs(float(h[2, 0, 0]) - (0 * c - 2 * s)) < 1e-12 and abs(float(h[2, 0, 2]) - (2 * c + 0 * s)) < 1e-12     # (0, 2) pair up
    assert abs(float(p[2, 0, 0]) - (0 * c - 1 * s)) < 1e-12 and abs(float(p[2, 0, 1]) - (1 * c + 0 * s)) < 1e-12     # (0, 1) pair up
    assert abs(float(plain.rms(torch.tensor([[3.0, 4.0]], dtype=torch.float64), 0.5)[0, 0]) - 3 / math.sqrt(12.5 + 0.5)) < 1e-12


def test_plain_model_sees_what_the_masks_allow():
    """The logits at a position do not change when a token behind every mask changes, and do when one inside does."""
    cfg = dict(BASE, layers=[LAT, ATT])
    t = {k: v.double() for k, v in dk.weights.random_init.random_tensors(dk.config_from_dict(cfg), 1, torch.float32, 0.3).items()}
    tokens = list(range(1, 61))
    base = plain.forward(cfg, t, tokens)
    far = list(tokens)
    far[3] = 77                 # position 59: the chunk starts at 40, the window of 9 (seen through one more layer) reaches 51 at most
    assert float((plain.forward(cfg, t, far)[59] - base[59]).abs().max()) < 1e-12
    near = list(tokens)
    near[52] = 77
    assert float((plain.forward(cfg, t, near)[59] - base[59]).abs().max()) > 1e-6


def test_plans_of_the_kernel_for_rows_that_are_key_and_value():
    """Which sizes the kernel takes, how many queries a block of 64 (query, head) rows holds, how a single token's keys
    are dealt out, and the vectorised list of query tiles (most keys first, ties in sequence order)."""
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.parts.attention import QueryTiles
    assert api.shared_rows_takes(576, 512) and api.shared_rows_takes(336, 320) and api.shared_rows_takes(32, 32)
    assert not api.shared_rows_takes(80, 48) and not api.shared_rows_takes(648, 512) and not api.shared_rows_takes(320, 336)
    assert [api.shared_rows_tile_queries(g) for g in (1, 3, 32, 64, 70, 128)] == [64, 21, 2, 1, 1, 1]
    sms = api.sm_count()
    assert api.shared_rows_splits(sms, 32, 1, 40, 1024, None) == 1                         # a block an SM already
    assert api.shared_rows_splits(1, 32, 1, 40, None, 64) == 2                             # a chunk of two half pages (and the ragged one)
    assert api.shared_rows_splits(1, 32, 1, 400, None, None) == api.SHARED_ROWS_MAX_SPLITS
    assert api.shared_rows_splits(1, 128, 1, 400, None, None) == min(api.SHARED_ROWS_MAX_SPLITS, sms // 2)   # two blocks of heads a token
    tiles = QueryTiles(21).build(np.array([50, 1, 30]), np.array([0, 70, 40]), False)
    assert tiles.dtype == np.int32
    assert tiles.tolist() == [[1, 0], [2, 21], [2, 0], [0, 42], [0, 21], [0, 0]]           # last keys 71, 70, 61, 50, 42, 21
    assert QueryTiles(21).build(np.array([1, 1]), np.array([5, 6]), True).shape == (0, 2)
