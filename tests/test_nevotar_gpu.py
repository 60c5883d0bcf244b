"""The Nevotar decoder in the library against the plain implementation (``plain_nevotar``): every mechanism alone,
then whole models of several small shapes through the step function, the cache, the decode state and the entry
points. The shapes differ in every size and option: norms in 1 to 4 groups, key/value groups of 1 to 4, key and value
heads of different sizes, a query temperature that steps every few positions and none, rotations over the whole head,
a part of it and none, windows smaller and larger than a page and none, state-space groups of 1 to 3, convolutions of
1 to 4 taps, 1 to 3 chosen experts with and without a shared expert, a layer without feed-forward, layers that run on
another layer's weights, head sizes the tensor-core kernels take and ones they do not."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_nevotar as plain
from dryft_challenge_htn_2026_b200.cache import Cache
from dryft_challenge_htn_2026_b200.config.specs import (DiffAttentionSpec, GroupRMSNormSpec, LowerBoundRecurrenceSpec,
                                                        MaskedAttentionSpec, RMSNormSpec, RotaryPartSpec, RoutedMLPSpec,
                                                        StateSpaceSpec)
from dryft_challenge_htn_2026_b200.csrc import api
from dryft_challenge_htn_2026_b200.engine import DecodeLoop, Runner, load_model
from dryft_challenge_htn_2026_b200.engine.batch import build_context
from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
from helpers import ROOT, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


def att(heads, kv, dim, vdim, scale, diff, q_temp, mlp, **more):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return dict({"type": "attention", "mixer": m, "mlp": mlp}, **more)


def hg(heads, dim, vdim, mlp, **more):
    return dict({"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}, **more)


def par(left, right, left_scale, right_scale, mlp, **more):
    H, G, D, V, scale, rot, mask = left
    l = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
    if rot is not None:
        l["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        l["mask"] = {"size": mask}
    r = dict(zip(("heads", "vdim", "state", "groups", "conv", "norm_groups"), right))
    return dict({"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale},
                 "mlp": mlp}, **more)


def moe(experts, ff, limit, top, shared):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


_A0 = att(4, 2, 16, 16, 0.25, 0.7, (0.3, 5), moe(8, 40, 2.0, 2, (48, 1.5)))
_A2 = par((4, 2, 32, 16, 0.18, (16, 10000.0), 24), (4, 16, 16, 2, 4, 2), 0.5, 1.25, moe(8, 40, 2.0, 2, (48, 1.5)))
SHAPES = {
    # norms in 4 groups, key/value groups of 2, a temperature that steps every 5 positions, a rotation over half the
    # head, a window smaller than a page, two layers that run on other layers' weights, a last layer without feed-forward
    "A": dict(architecture="Nevotar", vocab=200, width=64, norm={"eps": 1e-5, "groups": 4},
              layers=[_A0, hg(2, 16, 24, moe(4, 24, 1.0, 1, None)), _A2, dict(_A0, weights_of=0), dict(_A2, weights_of=2),
                      hg(1, 32, 8, None)]),
    # a recurrence first, one group for the norm, as many key/value heads as query heads, no temperature, no rotation, a
    # window of exactly one page, one state-space group, 2 taps, 3 of 6 experts without a shared one
    "B": dict(architecture="Nevotar", vocab=264, width=96, norm={"eps": 3e-6, "groups": 1},
              layers=[hg(3, 16, 32, moe(6, 24, 3.0, 3, None)),
                      par((3, 3, 16, 48, 0.3, None, 64), (3, 32, 16, 1, 2, 1), 1.0, 1.0, moe(6, 24, 3.0, 3, None)),
                      att(3, 3, 16, 32, 0.2, 0.5, None, moe(4, 32, 0.75, 1, (16, 4.0)))]),
    # head sizes the tensor-core kernels are built for (two maps of 32 and of 64 side by side), a window that spans pages
    # and none, wide states, a norm in 2 groups
    "C": dict(architecture="Nevotar", vocab=320, width=128, norm={"eps": 1e-6, "groups": 2},
              layers=[att(2, 1, 32, 64, 0.17, 0.55, (0.5, 40), moe(8, 64, 2.5, 2, (64, 2.0))),
                      par((8, 4, 64, 32, 0.125, (64, 250000.0), 100), (4, 64, 128, 2, 4, 1), 0.75, 0.8, moe(8, 64, 2.5, 2, (64, 2.0))),
                      att(2, 2, 64, 128, 0.11, 0.4, (1.0, 72), None),
                      par((2, 1, 128, 128, 0.09, (32, 10000.0), None), (2, 32, 64, 1, 3, 2), 1.5, 0.5, moe(4, 32, 1.0, 2, None))]),
    # sizes that no tensor-core kernel takes: heads of 10 / 20 / 24, values of 10 (no multiple of 4), an expert size of
    # 20, three state-space groups, a norm of the width in 3 groups and of the inner size in 5, a convolution of one tap
    "D": dict(architecture="Nevotar", vocab=136, width=48, norm={"eps": 1e-5, "groups": 3},
              layers=[att(3, 1, 10, 20, 0.3, 0.8, (2.0, 3), moe(3, 20, 1.5, 2, (20, 0.5))),
                      hg(1, 24, 10, moe(3, 20, 1.5, 2, (20, 0.5))),
                      par((3, 1, 20, 10, 0.22, (10, 100.0), 33), (3, 10, 24, 3, 3, 5), 0.9, 1.1, None),
                      par((2, 2, 12, 12, 0.3, None, 5), (2, 6, 40, 1, 1, 1), 1.0, 1.0, moe(5, 12, 1.0, 3, None))]),
}


def make_model(tmp_path, name, seed=0):
    cfg = dk.config_from_dict(SHAPES[name])
    folder = str(tmp_path / f"nevotar{name}_{seed}")
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


def bound_part(spec, dtype, seed=0, scale=0.3, **given):
    """A part with random tensors bound (or the ``given`` ones): -> (part, tensors as float64 after the rounding the
    part's type does to them)."""
    part = build_part(spec, Runtime(DEV, dtype))
    p = {}
    for i, d in enumerate(part.param_decls()):
        if d.name in given:
            x = given[d.name].double()
        else:
            x = rnd(*d.shape, seed=seed + 7 * i + 1)
            if d.init == "near_identity":
                x = torch.eye(d.shape[-1], dtype=torch.float64) + 0.3 * x
            else:
                x = {"norm": 1 + 0.2 * x, "fraction": torch.sigmoid(x), "taps": 0.6 * x, "unit": x, "around_zero": 0.2 * x,
                     "wide": x}.get(d.init, scale * x)
        p[d.name] = x.to(torch.float32 if d.keep_float32 else dtype).double()
    part.bind({d.name: dev(p[d.name], torch.float32 if d.keep_float32 else dtype) for d in part.param_decls()})
    return part, p


def run_cut(part, rows, lens, dtype, width_out, call=None):
    """The part over one sequence of input rows cut into steps of ``lens``, a second sequence of other rows beside it in
    every step (three tokens, or one when the step is a single token): -> the outputs of the first sequence's rows."""
    cache = Cache([part.cache_requests()], 64 * 40, 4, DEV)
    other, slot = cache.begin(), cache.begin()
    part.prepare(sum(lens) + 8)
    noise = rnd(4, rows.shape[1], seed=99)
    got, t0 = [], 0
    for n in lens:
        m = 1 if n == 1 else 3
        ctx = build_context(cache, [(other, [0] * m, []), (slot, [0] * n, [])], DEV, plans=part.step_plans())
        ctx.carry = {}
        a = torch.cat([dev(noise[:m], dtype), dev(rows[t0:t0 + n], dtype)], 0).contiguous()
        out = call(ctx, cache.views(0), a) if call else part.forward(ctx, cache.views(0), a)
        if isinstance(out, api.Partial):
            out = out.ws.sum(0)
        got.append(out[m:, :width_out].double().cpu())
        cache.commit(other, m), cache.commit(slot, n)
        t0 += n
    return torch.cat(got, 0), cache, slot


CUTS = [131, 2, 1, 1, 40, 1, 1, 1, 90]


# ------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,groups", [(5, 48, 3), (70, 256, 1), (3, 1000, 8), (9, 64, 64), (130, 96, 2), (4, 2560, 5)])
def test_norm_in_groups_with_the_residual_sum_and_at_chosen_rows(dtype, rows, width, groups):
    part, p = bound_part(GroupRMSNormSpec(width, 1e-5, groups), dtype)
    h0, d = rnd(rows, width, seed=1, scale=3.0).float().double(), rnd(rows, width, seed=2).to(dtype).double()
    h = dev(h0, torch.float32)
    out = torch.empty(rows, width, dtype=dtype, device=DEV)
    part.add_forward(h, dev(d, dtype), out)
    close(h, h0 + d, torch.float32, "sum")
    close(out, plain.group_norm(h0 + d, p[""], 1e-5, groups), dtype, "norm", slack=0.25)
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, width, dtype=dtype, device=DEV)
    part.add_forward(h, None, out2, rows=pick)                 # gathered: h stays as it is
    close(out2, plain.group_norm((h0 + d)[[rows - 1, 0]], p[""], 1e-5, groups), dtype, "gathered", slack=0.25)
    close(h, h0 + d, torch.float32, "untouched")
    ws = torch.stack([dev(d * 0.25, torch.float32), dev(d * 0.75, torch.float32)]).contiguous()
    h = dev(h0, torch.float32)
    part.add_forward(h, api.Partial(ws), out)                  # split-K partial sums are added while they are read
    close(out, plain.group_norm(h0 + d, p[""], 1e-5, groups), dtype, "partial sums", slack=0.25)


def test_a_tiny_row_shows_eps_inside_the_root_of_each_group():
    part, p = bound_part(GroupRMSNormSpec(8, 1e-2, 2), torch.float32)
    h0 = torch.tensor([[1e-2, -1e-2, 2e-2, 1e-2, 3.0, -1.0, 2.0, 0.5]], dtype=torch.float64)
    out = torch.empty(1, 8, dtype=torch.float32, device=DEV)
    part.add_forward(dev(h0, torch.float32), None, out)
    close(out, plain.group_norm(h0, p[""], 1e-2, 2), torch.float32, "eps")
    assert float(out[0, :4].abs().max()) < 0.5          # the small group is held down by eps, not blown up to unit size


DIFF_SHAPES = [(4, 2, 16, 16, (0.3, 5)), (3, 3, 16, 32, None), (2, 1, 32, 64, (0.5, 40)), (3, 1, 10, 20, (2.0, 3)), (2, 2, 64, 128, (1.0, 72)),
               (1, 1, 24, 8, (0.7, 1))]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,qt", DIFF_SHAPES)
def test_differential_attention_in_prompts_portions_and_single_tokens(dtype, H, G, D, V, qt):
    W = 40
    spec = DiffAttentionSpec(hidden_size=W, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=V, scale=D ** -0.5, diff=0.65,
                             norm_eps=1e-5, q_temp=qt)
    part, p = bound_part(spec, dtype, seed=3)
    x = rnd(sum(CUTS), W, seed=4).to(dtype).double()
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": D ** -0.5, "diff": 0.65}
    if qt:
        m["q_temp"] = {"coef": qt[0], "every": qt[1]}
    ref = plain.diff_attention(x, p, m, 1e-5)
    got, _, _ = run_cut(part, x, CUTS, dtype, W)
    # a1 - lambda a2 of two nearly equal maps, then a division by the head's root mean square: what bfloat16 rounding
    # leaves in q, k and the maps comes out about 1 / (1 - lambda) times larger than after a single softmax
    close(got, ref, dtype, "differential attention", slack=0.5 if dtype == torch.float32 else 1.5)


def diff_planted(dtype, D, V, lens, qi, kj):
    """Rows [q | k | v] straight into ``mix`` (no biases): key kj's first map is given the direction of query qi's first
    map of head 0 and a value of fives."""
    H, G, T = 4, 2, sum(lens)
    q, k, v = rnd(T, H, 2, D, seed=1), rnd(T, G, 2, D, seed=2), rnd(T, G, V, seed=3)
    k[kj, 0, 0] = 25.0 * q[qi, 0, 0] / q[qi, 0, 0].norm()
    v[kj] = 5.0
    q, k, v = (t.to(dtype).double() for t in (q, k, v))
    spec = DiffAttentionSpec(hidden_size=8, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=V, scale=D ** -0.5, diff=0.3,
                             norm_eps=1e-5, q_temp=(0.2, 50))
    zeros = {n: torch.zeros(s) for n, s in (("q.b", H * 2 * D), ("k.b", G * 2 * D), ("v.b", G * V))}
    part, p = bound_part(spec, dtype, **zeros)
    ref = plain.diff_core(q, k, v, D ** -0.5, plain.diff_lambda(p, 0.3), 0.3, 1e-5, {"coef": 0.2, "every": 50}).reshape(T, H * V)
    rows = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1)

    def call(ctx, views, a):
        mid = torch.empty(a.shape[0], H * V + 8, dtype=dtype, device=DEV)
        part.mix(ctx, views, a, mid[:, :H * V], 1.0)
        return mid
    got, _, _ = run_cut(part, rows, lens, dtype, H * V, call)
    return got, ref


@pytest.mark.parametrize("dtype,D,V", [(torch.float32, 16, 16), (torch.bfloat16, 16, 16), (torch.bfloat16, 32, 64), (torch.bfloat16, 24, 48)])
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("edge", ["the first token", "far key among hundreds", "page border", "the query's own position", "a later key"])
def test_a_planted_key_shows_in_the_first_map_and_a_later_one_does_not(dtype, D, V, where, edge):
    """Maps of 16 run on the float32-arithmetic kernel in float32 and the mma.sync kernels in bfloat16, maps of 32 with
    values of 64 on the tcgen05 prompt kernel and the split single-token kernel, 24 / 48 on the mma.sync ones."""
    qi = 300
    kj, seen = {"the first token": (0, True), "far key among hundreds": (7, True), "page border": (256, True),
                "the query's own position": (qi, True), "a later key": (qi + 1, False)}[edge]
    lens = [qi + 20] if where == "prompt" else [qi - 10] + [1] * 30
    got, ref = diff_planted(dtype, D, V, lens, qi, kj)
    close(got, ref, dtype, edge)
    head0 = got[qi, :V]       # after the head's unit norm a seen key leaves all coordinates alike and positive
    assert (float(head0.min()) > 0.35) == seen, (edge, float(head0.min()), float(head0.max()))


def talk_spec(H, G, D, V, window, rot, W=8):
    return MaskedAttentionSpec(hidden_size=W, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=V, scale=D ** -0.5, window=window,
                               qk_norm=RMSNormSpec(D, 1e-5), position=RotaryPartSpec(*rot) if rot else None, bias=True, talk=True)


TALK_SHAPES = [(4, 2, 32, 16, 24, (16, 10000.0)), (3, 3, 16, 48, 64, None), (8, 4, 64, 32, 100, (64, 250000.0)), (3, 1, 20, 10, 33, (10, 100.0)),
               (2, 1, 128, 128, None, (32, 10000.0)), (2, 2, 12, 12, 1, None), (16, 2, 48, 96, 70, (48, 1e6)), (20, 4, 32, 16, 50, None)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,window,rot", TALK_SHAPES)
def test_attention_with_mixed_head_scores_in_prompts_portions_and_single_tokens(dtype, H, G, D, V, window, rot):
    W = 40
    part, p = bound_part(talk_spec(H, G, D, V, window, rot, W), dtype, seed=5)
    x = rnd(sum(CUTS), W, seed=6).to(dtype).double()
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": D ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    ref = plain.talking_window_attention(x, p, m, 1e-5)
    got, _, _ = run_cut(part, x, CUTS, dtype, W)
    close(got, ref, dtype, "attention with mixed scores")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("edge", ["last inside the window", "first outside the window", "page border", "far key without a window",
                                  "the first token without a window"])
def test_a_planted_key_shows_inside_the_window_and_is_hidden_outside(dtype, where, edge):
    H, G, D, V, qi, size = 4, 2, 64, 32, 300, 70
    kj, seen, window = {"last inside the window": (qi - size + 1, True, size), "first outside the window": (qi - size, False, size),
                        "page border": (256, True, size), "far key without a window": (9, True, None),
                        "the first token without a window": (0, True, None)}[edge]
    lens = [qi + 20] if where == "prompt" else [qi - 10] + [1] * 30
    T = sum(lens)
    q, k, v = rnd(T, H, D, seed=1), rnd(T, G, D, seed=2), rnd(T, G, V, seed=3)
    k[kj, 0] = q[qi, 0]                  # the norm makes both unit size: the scale below makes the score stand out
    v[kj] = 5.0
    q, k, v = (t.to(dtype).double() for t in (q, k, v))
    spec = MaskedAttentionSpec(hidden_size=8, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=V, scale=1.0, window=window,
                               qk_norm=RMSNormSpec(D, 1e-6), bias=True, talk=True)
    zeros = {n: torch.zeros(s) for n, s in (("q.b", H * D), ("k.b", G * D), ("v.b", G * V))}
    ones = {"q.norm": torch.ones(D), "k.norm": torch.ones(D), "talk": torch.eye(H, dtype=torch.float64) + 0.1 * rnd(H, H, seed=4)}
    part, p = bound_part(spec, dtype, **zeros, **ones)
    ref = plain.talking_core(plain.rms(q, 1e-6), plain.rms(k, 1e-6), v, p["talk"], 1.0, window).reshape(T, H * V)
    rows = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1)

    def call(ctx, views, a):
        mid = torch.empty(a.shape[0], H * V + 8, dtype=dtype, device=DEV)
        part.mix(ctx, views, a, mid[:, :H * V], 1.0)
        return mid
    got, cache, slot = run_cut(part, rows, lens, dtype, H * V, call)
    close(got, ref, dtype, edge)
    assert (float(got[qi, :V].min()) > 4.0) == seen, (edge, float(got[qi, :V].min()))
    if window:       # pages wholly before the window were given back
        assert cache.groups[0].pages[slot][0] == -1


REC_SHAPES = [(2, 16, 24), (4, 32, 64), (1, 48, 10), (3, 100, 32), (2, 256, 8), (1, 24, 130)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V", REC_SHAPES)
def test_lower_bound_recurrence_in_prompts_portions_and_single_tokens(dtype, H, D, V):
    W = 40
    part, p = bound_part(LowerBoundRecurrenceSpec(hidden_size=W, num_heads=H, head_dim=D, v_head_dim=V, norm_eps=1e-5), dtype, seed=7)
    x = rnd(sum(CUTS), W, seed=8).to(dtype).double()
    ref, _ = plain.hgrn2(x, p, {"heads": H, "dim": D, "vdim": V}, 1e-5)
    got, _, _ = run_cut(part, x, CUTS, dtype, W)
    close(got, ref, dtype, "recurrence")


@pytest.mark.parametrize("dtype", DTYPES)
def test_lower_bound_recurrence_keeps_far_tokens_when_the_bound_is_near_one(dtype):
    """With l = 0.999 the state forgets a thousandth a token at most: what the first tokens wrote is still there 900 tokens on."""
    H, D, V, W = 2, 32, 16, 24
    lower = torch.full((H * D,), 0.999)
    part, p = bound_part(LowerBoundRecurrenceSpec(hidden_size=W, num_heads=H, head_dim=D, v_head_dim=V, norm_eps=1e-5), dtype, seed=9,
                         lower=lower)
    x = rnd(930, W, seed=10).to(dtype).double()
    ref, _ = plain.hgrn2(x, p, {"heads": H, "dim": D, "vdim": V}, 1e-5)
    other, _ = plain.hgrn2(torch.cat([rnd(100, W, seed=11), x[100:]]), p, {"heads": H, "dim": D, "vdim": V}, 1e-5)
    assert float((ref[920:] - other[920:]).abs().max()) > 2 * tol(dtype, ref)        # the first hundred tokens matter at the end
    got, _, _ = run_cut(part, x, [500, 1, 1, 2, 400, 1, 25], dtype, W)
    close(got, ref, dtype, "slow decay")


SSD_SHAPES = [(4, 16, 16, 2, 4, 2), (3, 32, 16, 1, 2, 1), (4, 64, 128, 2, 4, 1), (3, 10, 24, 3, 3, 5), (2, 6, 40, 1, 1, 1), (1, 8, 100, 1, 9, 2)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V,N,G,taps,ng", SSD_SHAPES)
def test_state_space_mixer_in_prompts_portions_and_single_tokens(dtype, H, V, N, G, taps, ng):
    W = 40
    spec = StateSpaceSpec(hidden_size=W, num_heads=H, v_head_dim=V, state_dim=N, groups=G, conv_taps=taps, norm_groups=ng, norm_eps=1e-5)
    part, p = bound_part(spec, dtype, seed=11, scale=0.15)
    x = rnd(sum(CUTS), W, seed=12).to(dtype).double()
    ref, _ = plain.ssd(x, p, {"heads": H, "vdim": V, "state": N, "groups": G, "norm_groups": ng}, 1e-5)
    got, _, _ = run_cut(part, x, CUTS, dtype, W)
    close(got, ref, dtype, "state space")


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_space_mixer_keeps_far_tokens_when_steps_are_small(dtype):
    """A strongly negative dt_bias makes every step small, so the decay stays near one over 900 tokens (the norm behind
    the state brings the small writes back to size)."""
    H, V, N, W = 2, 16, 32, 24
    spec = StateSpaceSpec(hidden_size=W, num_heads=H, v_head_dim=V, state_dim=N, groups=1, conv_taps=3, norm_groups=1, norm_eps=1e-5)
    part, p = bound_part(spec, dtype, seed=13, scale=0.15, dt_bias=torch.full((H,), -8.0), A_log=torch.zeros(H),
                         D=torch.zeros(H))       # no skip: the output is what the state gives
    x = rnd(930, W, seed=14).to(dtype).double()
    m = {"heads": H, "vdim": V, "state": N, "groups": 1, "norm_groups": 1}
    ref, _ = plain.ssd(x, p, m, 1e-5)
    other, _ = plain.ssd(torch.cat([rnd(100, W, seed=15), x[100:]]), p, m, 1e-5)
    assert float((ref[920:] - other[920:]).abs().max()) > 2 * tol(dtype, ref)        # the first hundred tokens matter at the end
    got, _, _ = run_cut(part, x, [500, 1, 1, 2, 400, 1, 25], dtype, W)
    close(got, ref, dtype, "small steps")


def test_states_are_zeroed_when_a_slot_is_taken_again():
    H, D, V, W = 2, 16, 8, 24
    part, p = bound_part(LowerBoundRecurrenceSpec(hidden_size=W, num_heads=H, head_dim=D, v_head_dim=V, norm_eps=1e-5), torch.float32)
    cache = Cache([part.cache_requests()], 64 * 8, 2, DEV)
    x = rnd(20, W, seed=1).float().double()
    ref, _ = plain.hgrn2(x, p, {"heads": H, "dim": D, "vdim": V}, 1e-5)
    for _ in range(3):
        slot = cache.begin()
        ctx = build_context(cache, [(slot, [0] * 20, [])], DEV)
        close(part.forward(ctx, cache.views(0), dev(x, torch.float32)), ref, torch.float32, "a slot used again")
        cache.commit(slot, 20)
        cache.end(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,ff,limit,top,shared,W,T", [(8, 40, 2.0, 2, (48, 1.5), 64, 7), (6, 24, 3.0, 3, None, 96, 50), (3, 20, 1.5, 2, (20, 0.5), 48, 3),
                                                       (8, 64, 0.4, 2, (64, 2.0), 128, 200), (4, 32, 1.0, 1, (16, 4.0), 96, 40), (5, 12, 1.0, 5, None, 40, 33)])
def test_experts_weighted_on_their_input_with_the_clamped_gate(dtype, E, ff, limit, top, shared, W, T):
    """Few tokens run a warp per output, many tokens in bfloat16 tiles on the tensor cores. Inputs large enough that the
    clamps bite on both sides."""
    spec = RoutedMLPSpec(hidden_size=W, expert_ff=ff, num_experts=E, top=top, shared_ff=shared[0] if shared else None,
                         activation="clamped", correction=False, renorm=False, weight_on_input=True, shared_gate=False, limit=limit,
                         shared_limit=shared[1] if shared else None)
    # a router whose scores stay away from 1: float32 sigmoids that saturate would tie
    part, p = bound_part(spec, dtype, seed=15, scale=0.25, router=rnd(E, W, seed=17, scale=0.08))
    x = rnd(T, W, seed=16, scale=1.5).to(dtype).double()
    mlp = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": E, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    ref = plain.moe(x, p, mlp)
    got = part.forward(type("Ctx", (), {"scratch": staticmethod(lambda key, make: make())})(), dev(x, dtype))
    idx, wt = plain.route(x, p["router"], top)
    assert float(wt.sum(-1).min()) < 0.9 * top            # the weights are the scores themselves, not their share of a sum
    err = (got.double().cpu() - ref).abs().max(-1).values
    bad = int((err > tol(dtype, ref) * 0.5).sum())
    assert bad <= (0 if dtype == torch.float32 else T // 10), f"{bad} of {T} tokens off, worst {float(err.max())}"


# ------------------------------------------------------------------------------------ whole models
def plain_logits(folder, tokens):
    cfg, t = plain.read_model(folder)
    return plain.forward(tokens, t, cfg)


class Errors:
    """float32 must hold everywhere. In bfloat16 a router's choice flips where two scores lie within what rounding has
    left in the stream by then (the plain implementation routes on float64 activations), and a position that has taken
    another expert stays off in every later layer: with several routed layers a good part of the positions may be off;
    a fault in a kernel would put nearly all of them off."""

    def __init__(self, dtype):
        self.dtype, self.n, self.bad = dtype, 0, []

    def add(self, err, bound, what):
        self.n += 1
        if err > bound:
            self.bad.append((what, err))

    def verdict(self):
        allowed = 0 if self.dtype in (torch.float32, "float32") else self.n // 3
        assert len(self.bad) <= allowed, f"{len(self.bad)} of {self.n} positions off: {self.bad[:5]}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_stream_after_every_layer_run(tmp_path, name, dtype):
    folder, cfg = make_model(tmp_path, name, seed=1)
    tokens = random_tokens(cfg.vocab, 75, 3)
    pcfg, t = plain.read_model(folder)
    ref = []
    plain.forward(tokens, t, pcfg, ref)
    runner = Runner(load_model(folder, dtype), 64 * 4, 2)
    got = []
    slot = runner.begin()
    runner.step([(slot, tokens, [])], tap=lambda k, h: got.append(h.double().cpu()))
    assert len(got) == len(ref) == len(SHAPES[name]["layers"])
    errs = Errors(dtype)
    for k, (g, r) in enumerate(zip(got, ref)):
        for pos in range(len(tokens)):
            errs.add(float((g[pos] - r[pos]).abs().max()), tol(dtype, r), f"{name} layer run {k} position {pos}")
    errs.verdict()


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

    for round_ in range(2):        # the second round runs on the slots, pages and states the first gave back
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
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_through_the_decode_state_and_its_graph(tmp_path, name, dtype):
    folder, cfg = make_model(tmp_path, name, seed=3)
    model = load_model(folder, dtype)
    seqs = [random_tokens(cfg.vocab, n, 60 + i) for i, n in enumerate([150, 90])]
    ref = [plain_logits(folder, s) for s in seqs]
    for use_graph in (False, True):
        errs = Errors(dtype)
        runner = Runner(model, 64 * 12, 4)
        loop = DecodeLoop(runner, use_graph=use_graph)
        slots = [runner.begin() for _ in seqs]
        cut = [30, 5]
        runner.step([(sl, s[:c], []) for sl, s, c in zip(slots, seqs, cut)])
        for k in range(85):                          # windows pass over decoded tokens, the temperature steps, pages fill
            out = loop.forced_step([(sl, [s[c + k]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu().double()
            for i in range(2):
                errs.add(float((out[i] - ref[i][cut[i] + k]).abs().max()), tol(dtype, ref[i]), f"graph={use_graph} step {k} sequence {i}")
        errs.verdict()
        for sl in slots:
            runner.end(sl)
    api.gemm_tc_check()


def random_config(rng):
    """A configuration drawn at random: any order of layers, shared weights, sizes that no kernel was built for."""
    width = rng.choice([40, 48, 60, 100, 128, 160])
    groups = rng.choice([g for g in (1, 2, 4, 5, 8) if width % g == 0])

    def mlp():
        if rng.random() < 0.15:
            return None
        E = rng.choice([2, 3, 4, 8, 16])
        return moe(E, rng.choice([8, 20, 32, 64]), rng.choice([0.5, 2.0, 7.0]), rng.randint(1, min(E, 4)),
                   (rng.choice([8, 24, 32]), rng.choice([1.0, 7.0])) if rng.random() < 0.7 else None)

    def heads():
        G = rng.choice([1, 2, 3, 4])
        return G * rng.choice([1, 2, 3, 4]), G

    def one():
        kind = rng.choice(["attention", "hgrn2", "parallel"])
        if kind == "attention":
            H, G = heads()
            D = rng.choice([8, 12, 16, 24, 32, 64])
            return att(H, G, D, rng.choice([8, 16, 20, 32, 64, 128]), D ** -0.5 * rng.choice([0.5, 1.0, 2.0]), rng.choice([0.2, 0.5, 0.8]),
                       (rng.choice([0.1, 0.5, 1.0]), rng.choice([1, 3, 16, 100])) if rng.random() < 0.8 else None, mlp())
        if kind == "hgrn2":
            return hg(rng.choice([1, 2, 3, 4, 6]), rng.choice([8, 16, 24, 32, 64, 128]), rng.choice([6, 8, 16, 32, 40]), mlp())
        H, G = heads()
        D = rng.choice([8, 16, 20, 32, 64, 128])
        rot = (rng.choice([d for d in (2, 4, 8, 16, 32, 64, 128) if d <= D]), rng.choice([100.0, 1e4, 1e6])) if rng.random() < 0.8 else None
        g = rng.choice([1, 2, 3, 4])
        rh, rv = g * rng.choice([1, 2, 3]), rng.choice([4, 8, 12, 16, 32, 64])
        right = (rh, rv, rng.choice([8, 16, 24, 32, 64, 128]), g, rng.choice([1, 2, 3, 4]), rng.choice([n for n in (1, 2, 3, 4, 6) if (rh * rv) % n == 0]))
        return par((H, G, D, rng.choice([8, 12, 16, 32, 64]), D ** -0.5, rot, rng.choice([None, 1, 2, 7, 31, 32, 33, 64, 65, 100, 128])),
                   right, rng.choice([0.5, 1.0]), rng.choice([0.8, 1.5]), mlp())

    layers = []
    for _ in range(rng.randint(2, 5)):
        if layers and rng.random() < 0.3:
            j = rng.choice([k for k, l in enumerate(layers) if "weights_of" not in l])
            layers.append(dict(json.loads(json.dumps(layers[j])), weights_of=j))
        else:
            layers.append(one())
    return dict(architecture="Nevotar", vocab=rng.choice([50, 136, 333]), width=width, norm={"eps": rng.choice([1e-6, 1e-5]), "groups": groups},
                layers=layers)


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_through_batches_the_decode_state_and_portions(tmp_path, seed):
    import random

    from safetensors.torch import load_file, save_file

    cfg = dk.config_from_dict(random_config(random.Random(1000 + seed)))
    folder = str(tmp_path / "model")
    dk.write_random_model(cfg, folder, seed=seed, dtype=torch.float32, matrix_std=0.08)
    # the random-weights mode spreads routers wide: scores that reach 1 in float32 would tie, which float64 does not
    path = os.path.join(folder, "model.safetensors")
    save_file({k: (v * 0.15 if k.endswith(".router") else v).contiguous() for k, v in load_file(path).items()}, path)
    lens = [1, 37, 150, 230]
    seqs = [random_tokens(cfg.vocab, n, 10 * seed + i) for i, n in enumerate(lens)]
    ref = [plain_logits(folder, s) for s in seqs]
    for dtype in DTYPES:
        runner = Runner(load_model(folder, dtype), 64 * 24, 6)
        errs = Errors(dtype)

        def check(out, pairs, what):
            out = out.cpu().double()
            for row, (i, p) in enumerate(pairs):
                errs.add(float((out[row] - ref[i][p]).abs().max()), tol(dtype, ref[i]), f"seed {seed} {what}: sequence {i} position {p}")

        for use_graph in (False, True):
            cut = [1, 20, 100, 140]
            slots = [runner.begin() for _ in seqs]
            check(runner.step([(sl, s[:c], [c - 1]) for sl, s, c in zip(slots, seqs, cut)]), [(i, c - 1) for i, c in enumerate(cut)], "prompts")
            loop = DecodeLoop(runner, use_graph=use_graph)
            live, k = [i for i in range(4) if cut[i] < lens[i]], 0
            while live and k < 40:
                check(loop.forced_step([(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live]), [(i, cut[i] + k) for i in live], f"token {k}")
                k += 1
                for i in [i for i in live if cut[i] + k >= lens[i]]:
                    runner.end(slots[i])
                    slots[i] = None
                live = [i for i in live if cut[i] + k < lens[i]]
            for sl in slots:
                if sl is not None:
                    runner.end(sl)
        slot, at = runner.begin(), 0
        for n in [64, 2, 31, 1, 2, 70, 30]:
            check(runner.step([(slot, seqs[3][at:at + n], [0, n - 1])]), [(3, at), (3, at + n - 1)], f"portion of {n} at {at}")
            at += n
        runner.end(slot)
        errs.verdict()


@pytest.mark.parametrize("name", ["A", "D"])
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
            logits = plain.forward(p + emitted[:-1], t, pcfg)[len(p) - 1:]
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


def test_command_line_generates_with_a_nevotar_model(tmp_path):
    """Random weights from a config.json of this design through the command line, the tokens it prints against the
    plain implementation's greedy tokens."""
    from dryft_challenge_htn_2026_b200.cli import random_prompts

    cfg = dk.config_from_dict(SHAPES["A"])
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
        logits = plain.forward(prompts[i] + emitted[:-1], t, pcfg)[len(prompts[i]) - 1:]
        gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
        assert gap <= 1e-4, (i, gap)
