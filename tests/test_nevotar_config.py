"""Nevotar without a GPU: config keys and their errors, the specification that comes out of a config (shared weights as
schedule entries, tensor names and shapes, cache requests), and the plain implementation's mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_nevotar as plain
from dryft_challenge_htn_2026_b200.cache import Cache, KVRequest, StateRequest
from dryft_challenge_htn_2026_b200.config.specs import (DiffAttentionSpec, GroupRMSNormSpec, LowerBoundRecurrenceSpec, MaskedAttentionSpec,
                                                        ParallelMixerSpec, RoutedMLPSpec, StateSpaceSpec)
from dryft_challenge_htn_2026_b200.engine.model import CausalLM

MOE = {"kind": "moe", "expert": {"ff": 24, "limit": 2.0}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 16, "limit": 1.5}}
ATT = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16, "scale": 0.3, "diff": 0.7,
                                      "q_temp": {"coef": 0.3, "every": 5}}, "mlp": MOE}
HG = {"type": "hgrn2", "mixer": {"heads": 2, "dim": 12, "vdim": 20}, "mlp": None}
PAR = {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.25, "rot": {"dims": 8, "base": 1000.0},
                                              "mask": {"size": 70}},
                                     "right": {"heads": 4, "vdim": 8, "state": 12, "groups": 2, "conv": 3, "norm_groups": 2},
                                     "left_scale": 0.5, "right_scale": 2.0}, "mlp": MOE}
CFG = {"architecture": "Nevotar", "vocab": 120, "width": 40, "norm": {"eps": 1e-5, "groups": 4},
       "layers": [ATT, HG, PAR, dict(copy.deepcopy(ATT), weights_of=0), {"type": "parallel", "weights_of": 2}]}


def test_config_round_trip_and_what_may_be_left_out():
    cfg = dk.config_from_dict(copy.deepcopy(CFG))
    assert isinstance(cfg, dk.NevotarConfig)
    d = cfg.to_dict()
    assert d["layers"][4]["mixer"] == PAR["mixer"] and d["layers"][4]["weights_of"] == 2     # what was left out is layer 2's
    assert dk.config_from_dict(d) == cfg
    small = {"architecture": "Nevotar", "vocab": 50, "width": 16, "norm": {"eps": 1e-6},
             "layers": [{"type": "attention", "mixer": {"heads": 2, "dim": 8, "scale": 0.3, "diff": 0.5}, "mlp": None},
                        {"type": "parallel", "mixer": {"left": {"heads": 2, "dim": 8, "scale": 0.3},
                                                       "right": {"heads": 2, "vdim": 4, "state": 8, "conv": 2}}, "mlp": None}]}
    spec = dk.config_from_dict(small).to_spec()
    a, p = spec.layers[0].mixer, spec.layers[1].mixer
    assert (a.num_kv_heads, a.v_head_dim, a.q_temp) == (2, 8, None) and spec.layers[0].norm_in.groups == 1
    left, right = p.branches[0][1], p.branches[1][1]
    assert (left.window, left.position, left.talk, left.bias) == (None, None, True, True) and (right.groups, right.norm_groups) == (1, 1)
    assert p.branches[0][2] == 1.0 and p.branches[1][2] == 1.0


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "'diff' is missing"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "must be positive"),
    (lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=18), "even and at most dim"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(groups=3), "do not divide"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not implemented"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "chooses 7 of 6"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "'limit' is missing"),
    (lambda c: c["layers"][3].update(weights_of=3), "must name another layer"),
    (lambda c: c["layers"][3].update(weights_of=1), "described differently"),
    (lambda c: c["norm"].update(groups=3), "does not divide the width"),
    (lambda c: c.pop("vocab"), "'vocab' is missing"),
])
def test_config_errors(change, text):
    c = copy.deepcopy(CFG)
    change(c)
    with pytest.raises(dk.ConfigError, match=text):
        dk.config_from_dict(c).to_spec()


def test_specification_schedule_tensors_and_cache_requests():
    spec = dk.config_from_dict(copy.deepcopy(CFG)).to_spec()
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (0, 3), (2, 4)] and len(spec.layers) == 3
    assert spec.tie_embeddings and isinstance(spec.final_norm, GroupRMSNormSpec) and spec.final_norm.groups == 4
    a, h, p = (l.mixer for l in spec.layers)
    assert isinstance(a, DiffAttentionSpec) and a.q_temp == (0.3, 5) and isinstance(h, LowerBoundRecurrenceSpec)
    assert isinstance(p, ParallelMixerSpec) and isinstance(p.branches[0][1], MaskedAttentionSpec) and isinstance(p.branches[1][1], StateSpaceSpec)
    ff = spec.layers[0].feed_forward
    assert isinstance(ff, RoutedMLPSpec) and (ff.activation, ff.renorm, ff.correction, ff.weight_on_input, ff.shared_gate) == \
        ("clamped", False, False, True, False) and (ff.limit, ff.shared_limit) == (2.0, 1.5) and spec.layers[1].feed_forward is None
    model = CausalLM(spec, dtype=torch.float32, device="cpu")
    shapes = {n: d.shape for n, d in model.param_decls(True).items()}
    assert shapes["embed"] == (120, 40) and shapes["final.norm"] == (40,) and "head" not in shapes
    assert shapes["l0.mix.q"] == (4 * 2 * 8, 40) and shapes["l0.mix.k"] == (2 * 2 * 8, 40) and shapes["l0.mix.v"] == (2 * 16, 40)
    assert shapes["l0.mix.q.b"] == (64,) and shapes["l0.mix.lq1"] == (8,) and shapes["l0.mix.o"] == (40, 64)
    assert shapes["l1.mix.f"] == (24, 40) and shapes["l1.mix.lower"] == (24,) and shapes["l1.mix.norm"] == (20,) and "l1.norm2" not in shapes
    assert shapes["l2.mix.left.talk"] == (4, 4) and shapes["l2.mix.left.q.norm"] == (16,) and shapes["l2.mix.left.k.b"] == (32,)
    assert shapes["l2.mix.right.in"] == (2 * 32 + 2 * 24 + 4, 40) and shapes["l2.mix.right.conv"] == (32 + 48, 3)
    assert shapes["l2.mix.right.norm"] == (32,) and shapes["l2.mix.right.D"] == (4,) and shapes["l2.mlp.shared.up"] == (16, 40)
    assert "l0.mlp.correction" not in shapes and "l0.mlp.shared.sg" not in shapes and not any(n.startswith(("l3.", "l4.")) for n in shapes)
    req = model.entry_requests()
    # two maps side by side in one key row; a state per recurrent head; the window's keys, the state and the convolution's memory
    assert req[0] == [KVRequest(2, 16, None, torch.float32, 16)] and req[3] == req[0]
    assert req[1] == [StateRequest((2, 12, 20), torch.float32)]
    assert req[2] == [KVRequest(2, 16, 70, torch.float32, 8), StateRequest((4, 12, 8), torch.float32), StateRequest((2, 80), torch.float32)]
    cache = Cache(req, 64 * 8, 4, "cpu", allocate=False)
    slot = cache.begin()
    cache.reserve(slot, 300)
    cache.commit(slot, 300)
    windowed = [g for g in cache.groups if isinstance(g.request, KVRequest) and g.request.window == 70][0]
    full = [g for g in cache.groups if isinstance(g.request, KVRequest) and g.request.window is None][0]
    assert windowed.pages[slot][:3] == [-1, -1, -1] and windowed.pages[slot][3] >= 0 and all(p >= 0 for p in full.pages[slot])


def test_plain_mechanisms_against_closed_forms():
    F = torch.float64
    # a norm in one group is the plain RMS norm; in as many groups as coordinates every coordinate is x / sqrt(x^2 + eps)
    x = torch.tensor([[3.0, -4.0, 1.0, 2.0]], dtype=F)
    w = torch.tensor([1.0, 2.0, 0.5, 1.0], dtype=F)
    assert torch.allclose(plain.group_norm(x, w, 0.0, 1), x / math.sqrt(30 / 4) * w)
    assert torch.allclose(plain.group_norm(x, w, 0.0, 2), torch.tensor([[3 / math.sqrt(12.5), -8 / math.sqrt(12.5), 0.5 / math.sqrt(2.5), 2 / math.sqrt(2.5)]], dtype=F))
    assert torch.allclose(plain.group_norm(x, w, 1.0, 4), x / torch.sqrt(x * x + 1.0) * w)
    # the temperature steps when (p + 1) / every passes a whole number
    t = plain.query_temperature(torch.tensor([0, 3, 4, 8, 9, 14]), 0.5, 5)
    assert torch.allclose(t, 1 + 0.5 * torch.log(torch.tensor([1.0, 1.0, 2.0, 2.0, 3.0, 4.0], dtype=F)))
    # with a constant gate f the recurrence is a geometric sum: S_t = (1 - f) sum_j f^(t - j) v_j
    T, D, V = 6, 1, 2
    p = {"q": torch.zeros(1, 1, dtype=F), "v": torch.eye(2, dtype=F)[:, :1].repeat(1, 1), "f": torch.zeros(1, 1, dtype=F),
         "f.b": torch.zeros(1, dtype=F), "lower": torch.tensor([0.5], dtype=F), "norm": torch.ones(2, dtype=F), "o": torch.eye(2, dtype=F)}
    h = torch.ones(T, 1, dtype=F)
    _, S = plain.hgrn2(h, p, {"heads": 1, "dim": D, "vdim": V}, 1e-6)
    f = 0.5 + 0.5 * 0.5
    assert torch.allclose(S[0, 0, 0], torch.tensor((1 - f) * sum(f ** (T - 1 - j) for j in range(T)), dtype=F))
    # the window: position i sees exactly the window's size of positions, itself included
    see = plain.causal(10, 3)
    assert see.sum(-1).tolist() == [1, 2, 3, 3, 3, 3, 3, 3, 3, 3] and bool(see[5, 3]) and not bool(see[5, 2]) and not bool(see[5, 6])
    # the convolution's last column is the current token's; what came before a step continues it exactly
    u = torch.arange(1.0, 7.0, dtype=F).reshape(6, 1)
    wc = torch.tensor([[100.0, 10.0, 1.0]], dtype=F)
    y, _ = plain.conv_taps(u, wc, torch.zeros(1, dtype=F))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0, 456.0]
    y1, before = plain.conv_taps(u[:4], wc, torch.zeros(1, dtype=F))
    y2, _ = plain.conv_taps(u[4:], wc, torch.zeros(1, dtype=F), before)
    assert torch.equal(torch.cat([y1, y2]), y)
    # a clamped expert: the gate is cut from above only, the other factor on both sides, and one is added to it
    one = torch.ones(1, 1, dtype=F)
    big = plain.clamped_expert(torch.tensor([[10.0]], dtype=F), one, one, one, 2.0)
    assert torch.allclose(big, torch.tensor([[2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0]], dtype=F))
    low = plain.clamped_expert(torch.tensor([[-10.0]], dtype=F), one, one, one, 2.0)
    assert torch.allclose(low, torch.tensor([[-10.0 / (1 + math.exp(17.02)) * (-1.0)]], dtype=F))
    # the router's weights are the scores themselves
    idx, wt = plain.route(torch.tensor([[1.0, 0.0]], dtype=F), torch.tensor([[0.0, 0.0], [2.0, 0.0], [1.0, 0.0]], dtype=F), 2)
    assert idx.tolist() == [[1, 2]] and torch.allclose(wt, torch.sigmoid(torch.tensor([[2.0, 1.0]], dtype=F)))


def test_plain_recurrences_do_not_depend_on_how_a_sequence_is_cut():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64) * 0.5
    W, H, V, N, G, taps = 12, 2, 4, 6, 1, 3
    p = {"in": r(2 * H * V + 2 * G * N + H, W), "conv": r(H * V + 2 * G * N, taps), "conv.b": r(H * V + 2 * G * N), "dt_bias": r(H),
         "A_log": r(H), "D": r(H), "norm": 1 + r(H * V), "o": r(W, H * V)}
    m = {"heads": H, "vdim": V, "state": N, "groups": G, "norm_groups": 2}
    x = r(9, W)
    whole, _ = plain.ssd(x, p, m, 1e-5)
    a, st = plain.ssd(x[:4], p, m, 1e-5)
    b, st = plain.ssd(x[4:5], p, m, 1e-5, st)
    c, _ = plain.ssd(x[5:], p, m, 1e-5, st)
    assert torch.allclose(torch.cat([a, b, c]), whole, atol=1e-12)
