"""The Venidra decoder in the library against the plain implementation (``plain_venidra``): every mechanism alone,
then whole models of several small shapes through the step function, the cache, the decode state and the entry
points. The shapes differ in every size and option: a latent-attention layer first and an attention layer first,
the first blending layer at any index, layers that do not blend, a single blending layer, key/value groups of 1 to
3 and as many key/value heads as query heads, key and value heads of different sizes, rotations over the whole
head, a part of it and none, chunks and windows of one position, smaller and larger than a page and longer than
the sequence, latents wider and narrower than the heads, layers without feed-forward, models without embedding
scale, logit scale or cap, head sizes the tensor-core kernels take and ones they do not."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_venidra as plain
from dryft_challenge_htn_2026_b200.cache import Cache
from dryft_challenge_htn_2026_b200.config.specs import (GatedMLPSpec, LatentAttentionSpec, MaskedAttentionSpec, RMSNormSpec,
                                                        RotaryPairsSpec, RotaryPartSpec, UnitRMSNormSpec)
from dryft_challenge_htn_2026_b200.csrc import api
from dryft_challenge_htn_2026_b200.engine import DecodeLoop, Runner, load_model
from dryft_challenge_htn_2026_b200.engine.batch import build_context
from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
from dryft_challenge_htn_2026_b200.parts.norm import NormedDelta
from helpers import ROOT, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]
DENSE = lambda ff: {"kind": "dense", "ff": ff}


def attn(heads, kv, dim, vdim, scale, rot, mask, v_mix, mlp):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, mask, mlp):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if mask is not None:
        m["mask"] = {"size": mask}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


SHAPES = {
    # a latent layer first (window smaller than a page); the first blending layer is layer 1; a layer that does not blend,
    # with the whole head rotated, value heads wider than key heads and no feed-forward; a blending layer of another head
    # count without rotation; a last latent layer with a window of 7 and no feed-forward
    "A": dict(architecture="Venidra", vocab=200, width=64, norm={"eps": 1e-5}, embedding={"scale": 2.0}, logit_scale=0.5,
              logit_softcap=20.0,
              layers=[latent(4, 16, 16, 32, 24, 32, 0.2, 10000.0, 40, DENSE(96)),
                      attn(4, 2, 32, 16, 0.3, (16, 10000.0), 24, True, DENSE(80)),
                      attn(2, 1, 16, 48, 0.25, (16, 500.0), 64, False, None),
                      attn(6, 2, 16, 16, 0.4, None, 100, True, DENSE(128)),
                      latent(2, 32, 8, 16, 16, 48, 0.15, 300.0, 7, None)]),
    # sizes that no tensor-core kernel takes (heads of 20 / 10, latents of 24 + 6, 12 + 6 a query head, a feed-forward of
    # 52); no embedding scale, logit scale or cap; a single blending layer (nobody reads its values); a chunk of 5
    "B": dict(architecture="Venidra", vocab=136, width=48, norm={"eps": 3e-6},
              layers=[attn(3, 1, 20, 10, 0.22, (10, 100.0), 5, True, DENSE(52)),
                      latent(3, 12, 6, 20, 10, 24, 0.3, 50.0, 33, DENSE(40))]),
    # head sizes 64 and 128 (what the tcgen05 kernel is built for), a cached latent row of 128 with values of 112, as many
    # key/value heads as query heads, a chunk of one position and a window of one position (every token sees itself
    # alone), a window longer than any sequence here, a chunk of exactly one page; three blending layers
    "C": dict(architecture="Venidra", vocab=320, width=128, norm={"eps": 1e-6}, embedding={"scale": 0.5}, logit_scale=3.0,
              logit_softcap=8.0,
              layers=[attn(2, 2, 64, 64, 0.125, (32, 250000.0), 64, True, DENSE(192)),
                      attn(1, 1, 128, 128, 0.09, (64, 5000.0), 300, False, None),
                      latent(2, 64, 16, 48, 40, 112, 0.1, 10000.0, 1000, DENSE(96)),
                      attn(2, 2, 128, 64, 0.09, (128, 10000.0), 1, True, None),
                      latent(3, 16, 32, 16, 64, 16, 0.2, 1000000.0, 1, DENSE(64)),
                      attn(4, 2, 32, 64, 0.2, (8, 100.0), 150, True, DENSE(160))]),
    # no mask at all on either mixer, groups of 3, the blending layers far apart with latent layers between them
    "D": dict(architecture="Venidra", vocab=264, width=96, norm={"eps": 1e-5}, embedding={"scale": 4.0}, logit_softcap=50.0,
              layers=[attn(6, 2, 16, 32, 0.3, (4, 20.0), None, False, DENSE(64)),
                      attn(3, 1, 48, 16, 0.15, (24, 1000.0), 70, True, None),
                      latent(4, 32, 16, 64, 48, 64, 0.12, 500000.0, None, DENSE(128)),
                      latent(1, 48, 32, 80, 8, 96, 0.1, 100.0, 129, None),
                      attn(1, 1, 32, 16, 0.2, None, 2, True, DENSE(72))]),
}


def make_model(tmp_path, name, seed=0):
    cfg = dk.config_from_dict(SHAPES[name])
    folder = str(tmp_path / f"venidra{name}_{seed}")
    dk.write_random_model(cfg, folder, seed=seed, dtype=torch.float32, matrix_std=0.08)
    return folder, cfg


def tol(dtype, ref):
    return (2e-4 if dtype in (torch.float32, "float32") else 6e-2) * max(1.0, float(ref.abs().max()))


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


def close(got, ref, dtype, what="", slack=0.5):
    err = float((got.double().cpu() - ref.double()).abs().max())
    assert err <= tol(dtype, ref) * slack, f"{what}: max error {err} > {tol(dtype, ref) * slack}"


def dev(x, dtype):
    return x.to(dtype).to(DEV)


def summed(x, dtype):
    return x.sum(dtype) if isinstance(x, api.Partial) else x


# ------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W", [48, 200, 1024])
def test_norm_of_a_sublayers_output_the_sum_and_the_next_norm(dtype, W):
    """x <- x + rms(y) * w_b; a = rms(x) * w_n, in one kernel; then the same for a few rows only, leaving x alone."""
    n = 13
    x0, y = rnd(n, W, seed=1, scale=3.0).float(), rnd(n, W, seed=2, scale=0.2).to(dtype)
    wb, wn = (1 + 0.2 * rnd(W, seed=3)).float(), (1 + 0.2 * rnd(W, seed=4)).float()
    rt = Runtime(DEV, dtype)
    nb, nn = build_part(RMSNormSpec(W, 1e-5, tensor=""), rt), build_part(RMSNormSpec(W, 3e-6, tensor=""), rt)
    nb.bind({"": wb.to(DEV)}), nn.bind({"": wn.to(DEV)})
    x = x0.to(DEV)
    a = nn.add_forward(x, NormedDelta(y.to(DEV), nb), torch.empty(n, W, dtype=dtype, device=DEV))
    x_ref = x0.double() + plain.rms(y.double(), 1e-5) * wb.double()
    assert float((x.cpu().double() - x_ref).abs().max()) < 3e-6 * float(x_ref.abs().max())     # the stream stays 32-bit
    close(a, plain.rms(x_ref, 3e-6) * wn.double(), dtype, "norm after the sum")
    rows = torch.tensor([12, 0, 5], dtype=torch.int32, device=DEV)
    before = x.clone()
    a = nn.add_forward(x, NormedDelta(y.to(DEV), nb), torch.empty(3, W, dtype=dtype, device=DEV), rows)
    x2 = before.cpu().double() + plain.rms(y.double(), 1e-5) * wb.double()
    close(a, (plain.rms(x2, 3e-6) * wn.double())[[12, 0, 5]], dtype, "wanted rows")
    assert torch.equal(x, before)
    close(NormedDelta(y.to(DEV), nb).to_float32(), plain.rms(y.double(), 1e-5) * wb.double(), dtype, "the delta alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,Fw", [(64, 104), (48, 52), (128, 384)])
def test_feed_forward_gated_by_the_tanh_form_of_gelu(dtype, W, Fw):
    part = build_part(GatedMLPSpec(W, Fw, "gelu_tanh", names=("gate", "up", "down")), Runtime(DEV, dtype))
    w = {"gate": rnd(Fw, W, seed=4, scale=0.4).to(dtype), "up": rnd(Fw, W, seed=5, scale=0.3).to(dtype),
         "down": rnd(W, Fw, seed=6, scale=0.2).to(dtype)}
    part.bind({k: v.to(DEV) for k, v in w.items()})
    wd = {k: v.double() for k, v in w.items()}
    for rows in (1, 5, 33, 70, 200):          # the row counts that pick the library's different products
        a = rnd(rows, W, seed=7, scale=1.5).to(dtype)
        close(summed(part.forward(None, a.to(DEV)), dtype), plain.feed_forward(a.double(), wd, ""), dtype,
              f"feed-forward, {rows} rows", slack=1.0)


def test_angle_tables_at_near_and_far_positions():
    for spec, base in ((RotaryPartSpec(16, 1000000.0), 1000000.0), (RotaryPairsSpec(6, 50.0), 50.0)):
        part = build_part(spec, Runtime(DEV, torch.float32))
        cos, sin = part.tables(300000)
        for p in (0, 1, 63, 64, 4097, 299999):
            a = plain.angles(1, spec.dim, base, pos0=p)[0]
            assert float((cos[p].cpu().double() - a.cos()).abs().max()) < 1e-6
            assert float((sin[p].cpu().double() - a.sin()).abs().max()) < 1e-6


def qkv_rows_case(dtype, H, G, D, Dv, rot, base, positions, blend):
    """The kernel between the projection and the cache: rotation of the heads' first ``rot`` coordinates by halves, then
    q and k heads divided by their root mean square, values blended with another layer's."""
    T = len(positions)
    q, k, v = rnd(T, H, D, seed=1, scale=2.0).to(dtype), rnd(T, G, D, seed=2, scale=0.5).to(dtype), rnd(T, G, Dv, seed=3).to(dtype)
    v_src = rnd(T, G, Dv, seed=4).to(dtype)
    lam = 0.3
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).to(DEV)
    out = torch.empty_like(proj)
    cos = sin = None
    if rot:
        cos, sin = build_part(RotaryPartSpec(rot, base), Runtime(DEV, dtype)).tables(max(positions) + 1)
    pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(T, dtype=torch.int32, device=DEV)
    api.conv_norm_rope(proj, out, None, None, 1, None, None, 1e-5, cos, sin, rot, pos, zeros, pos, zeros, H, G, D, Dv,
                       norm_mode=api.NORM_AFTER_ROTATION, v_mix=torch.tensor([lam], dtype=torch.float32, device=DEV) if blend else None,
                       v_src=v_src.reshape(T, -1).to(DEV) if blend else None)
    qd, kd = q.double(), k.double()
    if rot:
        a = torch.stack([plain.angles(1, rot, base, pos0=p)[0] for p in positions])
        qd, kd = plain.rotate_halves(qd, a), plain.rotate_halves(kd, a)
    vd = (1 - lam) * v.double() + lam * v_src.double() if blend else v.double()
    ref = torch.cat([plain.rms(qd, 1e-5).reshape(T, -1), plain.rms(kd, 1e-5).reshape(T, -1), vd.reshape(T, -1)], 1)
    close(out, ref, dtype, "rotated, normed, blended rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv,rot,base,blend", [(4, 2, 32, 16, 16, 10000.0, True), (2, 1, 16, 48, 16, 500.0, False),
                                                     (6, 2, 16, 16, 0, 1.0, True), (3, 1, 20, 10, 10, 100.0, True),
                                                     (1, 1, 128, 128, 128, 1000000.0, False), (5, 5, 24, 8, 2, 7.0, True)])
def test_rotation_by_halves_unit_rms_and_blended_values(dtype, H, G, D, Dv, rot, base, blend):
    qkv_rows_case(dtype, H, G, D, Dv, rot, base, [0, 1, 2, 63, 64, 65, 1000, 4097, 250000], blend)


def test_unit_rms_comes_after_the_rotation_not_before():
    """With a part of the head rotated the two orders agree (a rotation keeps the length); the test pins the epsilon's
    place and that no weight is applied: tiny heads, where eps decides the result."""
    T, H, D = 3, 2, 8
    q = (rnd(T, H, D, seed=1) * 1e-4).float()
    proj = torch.cat([q.reshape(T, -1), q.reshape(T, -1)[:, :D], q.reshape(T, -1)[:, :D]], 1).to(DEV)
    out = torch.empty_like(proj)
    cos, sin = build_part(RotaryPartSpec(4, 100.0), Runtime(DEV, torch.float32)).tables(8)
    pos = torch.tensor([0, 3, 7], dtype=torch.int32, device=DEV)
    z = torch.zeros(T, dtype=torch.int32, device=DEV)
    api.conv_norm_rope(proj, out, None, None, 1, None, None, 1e-5, cos, sin, 4, pos, z, pos, z, H, 1, D, D,
                       norm_mode=api.NORM_AFTER_ROTATION)
    a = torch.stack([plain.angles(1, 4, 100.0, pos0=p)[0] for p in (0, 3, 7)])
    ref = plain.rms(plain.rotate_halves(q.double(), a), 1e-5).reshape(T, -1)
    assert float((out[:, :H * D].cpu().double() - ref).abs().max()) < 1e-6
    assert float(ref.abs().max()) < 0.2          # eps dominates: without it the entries would be of order 1


def attention_case(dtype, H, G, D, V, chunk, window, lens_steps, plant=None, seed=0, values_in_keys=False):
    """The attention part's ``mix`` with nothing between projection and cache (cache write and whichever attention kernel
    the part picks) over one sequence cut into steps, a second sequence beside it, against the plain softmax over the
    whole sequence. ``plant`` = (query position, key position, strength): that key is given the query's direction, so
    that its score stands out, and a value of 5. ``values_in_keys``: every value row is the start of its key row (what an
    attention through latents caches), which the part may use to read the key rows alone."""
    T = sum(lens_steps)
    q, k, v = rnd(T, H, D, seed=seed), rnd(T, G, D, seed=seed + 1), rnd(T, G, V, seed=seed + 2)
    if plant:
        qi, kj, strength = plant
        k[kj] = strength * q[qi, 0] / q[qi, 0].norm()
        v[kj] = 5.0
    if values_in_keys:
        v = k[..., :V].clone()
    q, k, v = (x.to(dtype).double() for x in (q, k, v))
    scale = 0.9 * D ** -0.5
    mask = plain.chunk_mask(T, chunk or T) & plain.window_mask(T, window or T)
    ref = plain.masked_softmax_attention(q, k, v, mask, scale)
    spec = MaskedAttentionSpec(hidden_size=8, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=V, scale=scale, chunk=chunk,
                               window=window, values_in_keys=values_in_keys)
    part = build_part(spec, Runtime(DEV, dtype))
    if values_in_keys and dtype == torch.bfloat16 and max(D, V) > 256:
        assert part.shared_rows        # the kernel under test is the one that runs
    cache = Cache([part.cache_requests()], 64 * 40, 4, DEV)
    other, slot = cache.begin(), cache.begin()
    t0, got = 0, []
    for n in lens_steps:
        m = 1 if n == 1 else 3
        ctx = build_context(cache, [(other, [0] * m, []), (slot, [0] * n, [])], DEV, plans=part.step_plans())
        wide = torch.zeros(m + n, part.n_in + 8, dtype=dtype, device=DEV)
        wide[m:, :part.n_in] = dev(torch.cat([q[t0:t0 + n].reshape(n, -1), k[t0:t0 + n].reshape(n, -1),
                                              v[t0:t0 + n].reshape(n, -1)], 1), dtype)
        out = torch.empty(m + n, H * V + 8, dtype=dtype, device=DEV)
        part.mix(ctx, cache.views(0), wide[:, :part.n_in], out[:, :H * V], 1.0)
        got.append(out[m:, :H * V].double().cpu())
        cache.commit(other, m), cache.commit(slot, n)
        t0 += n
    return torch.cat(got, 0), ref


# (4, 2, 32, 16): float32-arithmetic kernel in both types; (8, 1, 80, 64) and (3, 3, 16, 48): mma.sync kernels in bfloat16 (the
# first is a cached row of latents with every head on it); (2, 1, 64, 64) and (2, 2, 128, 128): tcgen05 prompts, split single
# tokens; (2, 1, 320, 288): heads beyond 256
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,chunk,window", [(4, 2, 32, 16, 24, None), (8, 1, 80, 64, None, 40), (3, 3, 16, 48, 64, None),
                                                  (2, 1, 64, 64, 100, None), (2, 2, 128, 128, None, 70), (6, 2, 16, 16, 1, None),
                                                  (3, 1, 20, 10, None, 1), (2, 1, 320, 288, None, 33), (4, 4, 64, 64, 7, None),
                                                  (5, 1, 48, 32, None, None)])
def test_attention_under_a_chunk_mask_or_a_window(dtype, H, G, D, V, chunk, window):
    got, ref = attention_case(dtype, H, G, D, V, chunk, window, [131, 2, 1, 1, 40, 1, 1, 1, 90])
    close(got, ref, dtype, "attention")


# value rows that are the start of the key rows, wider than 256: groups of 3 (21 queries a block), of 70 (two blocks of heads
# a query), of 1 (64 queries a block) and of 32; a chunk, windows smaller and larger than a page, no mask (single tokens' keys
# dealt out to several blocks)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,chunk,window", [(6, 2, 320, 288, None, 33), (70, 1, 272, 32, 50, None), (3, 3, 288, 288, None, None),
                                                  (32, 1, 576, 512, None, 100),
                                                  # narrower rows: the kernels that otherwise read a store of values (mma.sync
                                                  # prompts and single tokens, float32 arithmetic) take them from the key rows
                                                  (8, 1, 80, 64, None, 40), (4, 2, 32, 16, 24, None), (3, 1, 20, 10, None, 7),
                                                  (2, 2, 64, 64, 100, None)])
def test_attention_over_rows_that_are_key_and_value(dtype, H, G, D, V, chunk, window):
    got, ref = attention_case(dtype, H, G, D, V, chunk, window, [131, 2, 1, 1, 40, 1, 1, 1, 90], values_in_keys=True)
    close(got, ref, dtype, "attention over shared rows")


@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("edge", ["first of the chunk", "last of the chunk before", "last inside the window", "first outside the window",
                                  "far key among hundreds", "page border", "half page border"])
def test_a_planted_row_shows_inside_and_is_hidden_outside(where, edge):
    """The same edges on the kernel for rows that are key and value at once (bfloat16, rows of 288 with values of 256): the
    head's output is the planted row's start when it is seen."""
    qi, D, V = 300, 288, 256
    chunk, window, kj, seen = {"first of the chunk": (70, None, 280, True), "last of the chunk before": (70, None, 279, False),
                               "last inside the window": (None, 70, 231, True), "first outside the window": (None, 70, 230, False),
                               "far key among hundreds": (None, None, 1, True), "page border": (None, 70, 256, True),
                               "half page border": (None, 13, 288, True)}[edge]
    lens = [qi + 20] if where == "prompt" else [qi - 10] + [1] * 30
    got, ref = attention_case(torch.bfloat16, 4, 1, D, V, chunk, window, lens, plant=(qi, kj, 25.0), seed=3, values_in_keys=True)
    close(got, ref, torch.bfloat16, edge)
    planted = 25.0 * rnd(sum(lens), 4, D, seed=3)[qi, 0] / rnd(sum(lens), 4, D, seed=3)[qi, 0].norm()
    off = float((got[qi, :V] - planted[:V].to(torch.bfloat16).double()).abs().max())
    assert (off < 0.5) == seen, (edge, off)


@pytest.mark.parametrize("dtype,D,V", [(torch.float32, 32, 32), (torch.bfloat16, 32, 16), (torch.bfloat16, 64, 64), (torch.bfloat16, 80, 64)])
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("edge", ["first of the chunk", "last of the chunk before", "last inside the window", "first outside the window",
                                  "far key among hundreds", "page border"])
def test_a_planted_key_shows_inside_and_is_hidden_outside(dtype, D, V, where, edge):
    """A chunk of 70 positions counted from position 0 (the query at 300 is in the chunk that starts at 280), a window of 70
    (the query sees 231..300), and no mask for the far key."""
    qi = 300
    chunk, window, kj, seen = {"first of the chunk": (70, None, 280, True), "last of the chunk before": (70, None, 279, False),
                               "last inside the window": (None, 70, 231, True), "first outside the window": (None, 70, 230, False),
                               "far key among hundreds": (None, None, 1, True), "page border": (None, 70, 256, True)}[edge]
    lens = [qi + 20] if where == "prompt" else [qi - 10] + [1] * 30
    got, ref = attention_case(dtype, 4, 1, D, V, chunk, window, lens, plant=(qi, kj, 25.0), seed=3)
    close(got, ref, dtype, edge)
    head0 = got[qi, :V]
    assert (float(head0.min()) > 4.0) == seen, (edge, float(head0.min()), float(head0.max()))


def test_chunks_count_from_the_sequences_start_not_from_the_portions():
    """A prompt cut at 50 and 103 under chunks of 32: the portion that starts at 50 sees back to 32, not to 50 and not to 18."""
    got, ref = attention_case(torch.float32, 2, 1, 16, 16, 32, None, [50, 53, 2, 1, 1, 30], seed=9)
    close(got, ref, torch.float32, "chunks over portions")


def latent_case(dtype, H, D, R, V, q_rank, kv_rank, window, lens_steps, base=10000.0, W=40, seed=0):
    """The whole latent-attention mixer over one sequence cut into steps, a second sequence beside it, against the plain
    mixer over the whole sequence."""
    spec = LatentAttentionSpec(hidden_size=W, num_heads=H, head_dim=D, rot_dim=R, v_head_dim=V, q_rank=q_rank, kv_rank=kv_rank,
                               scale=(D + R) ** -0.5, norm_eps=1e-5, position=RotaryPairsSpec(R, base), window=window)
    part = build_part(spec, Runtime(DEV, dtype))
    p = {"dq": rnd(q_rank, W, seed=seed, scale=0.3), "dq.norm": 1 + rnd(q_rank, seed=seed + 1, scale=0.2),
         "uq": rnd(H * (D + R), q_rank, seed=seed + 2, scale=0.3), "dkv": rnd(kv_rank + R, W, seed=seed + 3, scale=0.3),
         "dkv.norm": 1 + rnd(kv_rank, seed=seed + 4, scale=0.2), "uk": rnd(H * D, kv_rank, seed=seed + 5, scale=0.3),
         "uv": rnd(H * V, kv_rank, seed=seed + 6, scale=0.3), "o": rnd(W, H * V, seed=seed + 7, scale=0.2)}
    p = {k: v.to(dtype).double() for k, v in p.items()}
    part.bind({k: dev(v, torch.float32 if k.endswith("norm") else dtype) for k, v in p.items()})
    T = sum(lens_steps)
    h = rnd(T, W, seed=seed + 8).to(dtype).double()
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "q_rank": q_rank, "kv_rank": kv_rank, "scale": spec.scale,
         "rot": {"base": base, "dims": R}}
    if window:
        m["mask"] = {"size": window}
    ref = plain.latent_attention(h, p, "", m, 1e-5)
    cache = Cache([part.cache_requests()], 64 * 16, 4, DEV)
    other, slot = cache.begin(), cache.begin()
    part.prepare(T + 8)
    t0, got = 0, []
    for n in lens_steps:
        k = 1 if n == 1 else 2
        ctx = build_context(cache, [(other, [0] * k, []), (slot, [0] * n, [])], DEV, plans=part.step_plans())
        a = torch.zeros(k + n, W, dtype=dtype, device=DEV)
        a[k:] = dev(h[t0:t0 + n], dtype)
        got.append(summed(part.forward(ctx, cache.views(0), a), dtype)[k:].double().cpu())
        cache.commit(other, k), cache.commit(slot, n)
        t0 += n
    return torch.cat(got, 0), ref


# latents wider and narrower than the heads, a rotated part as wide as the plain one and wider, one head, sizes no
# tensor-core kernel takes (24 + 6), a cached row of 128 and ones of 320 and 336 (5 and 66 heads on them), windows of 1, 7, 64,
# 200 and none
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,R,V,q_rank,kv_rank,window", [(4, 16, 16, 32, 24, 32, 40), (2, 32, 8, 16, 16, 48, 7), (3, 12, 6, 20, 10, 24, 33),
                                                           (2, 64, 16, 48, 40, 112, 200), (3, 16, 32, 16, 64, 16, 1), (1, 48, 32, 80, 8, 96, None),
                                                           (8, 32, 16, 80, 96, 64, 64), (2, 24, 64, 40, 32, 256, 50),
                                                           (5, 16, 32, 24, 16, 288, 50), (66, 8, 16, 8, 12, 320, None)])
def test_latent_attention_in_prompts_portions_and_single_tokens(dtype, H, D, R, V, q_rank, kv_rank, window):
    got, ref = latent_case(dtype, H, D, R, V, q_rank, kv_rank, window, [70, 2, 1, 1, 33, 1, 1, 1, 60, 1])
    close(got, ref, dtype, "latent attention", slack=1.0)


def test_latent_attention_far_positions_and_another_base():
    """Rotation by pairs at positions past a page and with a small base: a rotation by halves, or angles of a wrong index,
    would differ in every score."""
    got, ref = latent_case(torch.float32, 2, 8, 8, 8, 8, 16, None, [150, 1, 1], base=20.0, seed=4)
    close(got, ref, torch.float32, "rotation by pairs")


# ------------------------------------------------------------------------------------ whole models
def plain_logits(folder, tokens):
    cfg, t = plain.read_model(folder)
    return plain.forward(cfg, t, tokens)


class Errors:
    """Every position must hold: the design has no discrete choice that rounding could flip."""

    def __init__(self, dtype):
        self.dtype, self.n, self.bad = dtype, 0, []

    def add(self, err, bound, what):
        self.n += 1
        if err > bound:
            self.bad.append((what, err))

    def verdict(self):
        assert not self.bad, f"{len(self.bad)} of {self.n} positions off: {self.bad[:5]}"


def test_the_stream_after_every_layer(tmp_path):
    folder, cfg = make_model(tmp_path, "A", seed=2)
    pcfg, t = plain.read_model(folder)
    tokens = random_tokens(cfg.vocab, 90, 11)
    layers = []
    plain.forward(pcfg, t, tokens, layers_out=layers)
    runner = Runner(load_model(folder, torch.float32), 64 * 4, 2)
    taps = []
    slot = runner.begin()
    runner.step([(slot, tokens, [])], tap=lambda k, h: taps.append(h.cpu().double()))
    runner.end(slot)
    assert len(taps) == len(layers) == len(cfg.layers)
    for k, (got, ref) in enumerate(zip(taps, layers)):
        assert float((got - ref).abs().max()) < 2e-4 * max(1.0, float(ref.abs().max())), f"after layer {k}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_portions_batches_and_reused_slots(tmp_path, name, dtype):
    folder, cfg = make_model(tmp_path, name)
    model = load_model(folder, dtype)
    runner = Runner(model, 64 * 24, 6)
    lens = [1, 23, 131, 200]
    seqs = [random_tokens(cfg.vocab, n, 40 + i) for i, n in enumerate(lens)]
    ref = [plain_logits(folder, s) for s in seqs]
    errs = Errors(dtype)

    def check(out, pairs, what):
        out = out.cpu().double()
        for row, (i, p) in enumerate(pairs):
            errs.add(float((out[row] - ref[i][p]).abs().max()), tol(dtype, ref[i]), f"{name} {what}: sequence {i} position {p}")

    for round_ in range(2):        # the second round runs on the slots and pages the first gave back
        for i, s in enumerate(seqs):
            slot = runner.begin()
            want = sorted({0, len(s) // 2, len(s) - 1})
            check(runner.step([(slot, s, want)]), [(i, p) for p in want], "alone")
            runner.end(slot)
        # a ragged batch of prompts cut short, then one token each, shorter ones ending earlier
        cut = [1, 17, 100, 130]
        slots = [runner.begin() for _ in seqs]
        check(runner.step([(sl, s[:c], [c - 1]) for sl, s, c in zip(slots, seqs, cut)]), [(i, c - 1) for i, c in enumerate(cut)],
              "batch of prompts")
        live = [i for i in range(4) if cut[i] < lens[i]]
        k = 0
        while live and k < 40:
            out = runner.step([(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live])
            check(out, [(i, cut[i] + k) for i in live], f"decode step {k}")
            k += 1
            for i in [i for i in live if cut[i] + k >= lens[i]]:
                runner.end(slots[i])
                slots[i] = None
            live = [i for i in live if cut[i] + k < lens[i]]
        for sl in slots:
            if sl is not None:
                runner.end(sl)
        # portions of several sizes, down to two tokens and one
        s, i = seqs[3], 3
        slot = runner.begin()
        at = 0
        for n in [64, 2, 31, 1, 2, 70, 30]:
            check(runner.step([(slot, s[at:at + n], [0, n - 1])]), [(i, at), (i, at + n - 1)], f"portion of {n} at {at}")
            at += n
        runner.end(slot)
    errs.verdict()
    assert runner.cache.slots.n_live == 0 and all(f == runner.cache.num_pages for f in runner.cache.pages_free())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_long_decoding_through_the_decode_state_and_its_graph(tmp_path, name, dtype):
    folder, cfg = make_model(tmp_path, name, seed=3)
    model = load_model(folder, dtype)
    seqs = [random_tokens(cfg.vocab, n, 60 + i) for i, n in enumerate([190, 120])]
    ref = [plain_logits(folder, s) for s in seqs]
    for use_graph in (False, True):
        errs = Errors(dtype)
        runner = Runner(model, 64 * 12, 4)
        loop = DecodeLoop(runner, use_graph=use_graph)
        slots = [runner.begin() for _ in seqs]
        cut = [30, 5]
        runner.step([(sl, s[:c], []) for sl, s, c in zip(slots, seqs, cut)])
        for k in range(115):                 # windows and chunks of 2 to 129 positions pass over decoded tokens, pages fill
            out = loop.forced_step([(sl, [s[c + k]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu().double()
            for i in range(2):
                errs.add(float((out[i] - ref[i][cut[i] + k]).abs().max()), tol(dtype, ref[i]), f"graph={use_graph} step {k} sequence {i}")
        errs.verdict()
        for sl in slots:
            runner.end(sl)
    api.gemm_tc_check()


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    folder, cfg = make_model(tmp_path, name, seed=5)
    pcfg, t = plain.read_model(folder)
    prompts = [random_tokens(cfg.vocab, n, 80 + i) for i, n in enumerate([3, 40, 77])]
    n_new = 30
    for dtype in DTYPES:
        eng = dk.Engine(folder, dtype=dtype)
        steps = list(eng.generate(prompts, n_new))
        again = list(dk.Engine(folder, dtype=dtype, use_graph=False, max_prefill_tokens=16).generate(prompts, n_new))
        for i, p in enumerate(prompts):
            emitted = [s[i] for s in steps]
            logits = plain.forward(pcfg, t, p + emitted[:-1])[len(p) - 1:]
            gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
            assert gap <= (1e-4 if dtype == torch.float32 else 0.12 * max(1.0, float(logits.abs().max()))), (name, dtype, i, gap)
            if dtype == torch.float32:               # prompts cut into portions of 16, plain launches: the same tokens
                assert emitted == [s[i] for s in again]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_ragged_schedule(tmp_path, dtype):
    folder, cfg = make_model(tmp_path, "B", seed=7)
    seqs = {"a": random_tokens(cfg.vocab, 140, 1), "b": random_tokens(cfg.vocab, 9, 2), "c": random_tokens(cfg.vocab, 66, 3)}
    ref = {k: plain_logits(folder, s) for k, s in seqs.items()}
    start = {"a": 130, "b": 1, "c": 60}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": seqs["a"][:130], "want": [0, 63, 64, 129]},
                                     {"id": "b", "tokens": seqs["b"][:1], "want": [0]},
                                     {"id": "c", "tokens": seqs["c"][:60], "want": []}], "end": []}]
    for k in range(10):
        ent = [{"id": i, "tokens": [seqs[i][start[i] + k]], "want": [0] if (i != "c" or k % 2) else []}
               for i in ("a", "b", "c") if start[i] + k < len(seqs[i])]
        steps.append({"step": k + 1, "entries": ent, "end": [e["id"] for e in ent if start[e["id"]] + k + 1 == len(seqs[e["id"]])]})
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", "512"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    at = {"a": 0, "b": 0, "c": 0}
    errs = Errors(dtype)
    for s in steps:
        rows = []
        for e in s["entries"]:
            rows += [(e["id"], at[e["id"]] + w) for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        if rows:
            got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(len(rows), cfg.vocab))
            for r, (i, p) in enumerate(rows):
                errs.add(float((got[r].double() - ref[i][p]).abs().max()), tol(dtype, ref[i]), (s["step"], i, p))
    errs.verdict()


def test_a_blending_weight_nobody_reads_is_let_pass(tmp_path):
    """An attention layer that does not blend may still come with a blending weight in the file; any other stray tensor is an error."""
    from safetensors.torch import load_file, save_file

    from dryft_challenge_htn_2026_b200.weights.loader import WeightError
    folder, cfg = make_model(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["l2.mix.vmix"] = torch.tensor(0.5)
    save_file(t, path)
    load_model(folder, torch.float32)
    t["l0.mix.vmix"] = torch.tensor(0.5)
    save_file(t, path)
    with pytest.raises(WeightError):
        load_model(folder, torch.float32)


def test_command_line_generates_with_a_venidra_model(tmp_path):
    """Random weights from a config.json of this design through the command line, the tokens it prints against the
    plain implementation's greedy tokens."""
    from dryft_challenge_htn_2026_b200.cli import random_prompts

    cfg = dk.config_from_dict(SHAPES["D"])
    cfg.save(str(tmp_path))
    model_dir = str(tmp_path / "model")
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "dryft_challenge_htn_2026_b200.cli", "--random-weights", str(tmp_path / "config.json"),
                        "--save-model", model_dir, "--seed", "3", "--dtype", "float32", "--shapes", "2,30,6", "--samples", "1",
                        "--print-tokens"], capture_output=True, text=True, env=env, cwd=str(ROOT), timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens 2,30,6 seq ")]
    assert len(lines) == 2
    pcfg, t = plain.read_model(model_dir)
    prompts = random_prompts(2, 30, 1, cfg.vocab, False)
    for i, line in enumerate(lines):
        emitted = [int(x) for x in line.split(":")[1].split()]
        logits = plain.forward(pcfg, t, prompts[i] + emitted[:-1])[len(prompts[i]) - 1:]
        gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
        assert gap <= 1e-4, (i, gap)
