"""Differential attention: two softmax maps per head over the same values, o = unit_rms(a1 - lambda a2) * (1 - diff).

A key/value head's two key maps lie side by side in one cached row of 2 * head_dim numbers. The kernel between the
projection and the cache (biases, the query temperature, the cache write) also makes two query heads of each query
head, [map 1 | zeros] and [zeros | map 2]: against the two-map key row each scores exactly its own map, so the
attention itself is the library's masked attention with 2 * heads query heads of size 2 * head_dim (its tensor-core
kernels for prompts and single tokens, its float32-arithmetic kernel otherwise), on a cache entry of the ordinary
layout. A last kernel takes a1 - lambda a2 per head, divides by the head's root mean square and scales. lambda is one
number per layer, worked out in float64 when the tensors are bound. Runs as a branch of a ``ParallelMixer`` too.
"""
import math

import torch

from ..config.specs import DiffAttentionSpec, MaskedAttentionSpec
from ..csrc import api
from .attention_masked import MaskedAttention
from .base import ParamDecl, Part, register_part
from .linear import linear


class DiffAttention(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads are not a multiple of {s.num_kv_heads} key/value heads")
        if s.q_temp is not None and not int(s.q_temp[1]) >= 1:
            raise ValueError(f"a query temperature every {s.q_temp[1]} positions")
        if 2 * s.head_dim > 256 or s.v_head_dim > 256:
            raise ValueError(f"differential attention takes key heads up to 128 and value heads up to 256, not {s.head_dim} / {s.v_head_dim}")
        # the attention over the two-map rows: every query head twice, key rows of both maps
        self.core = MaskedAttention(MaskedAttentionSpec(
            hidden_size=s.hidden_size, num_heads=2 * s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=2 * s.head_dim,
            v_head_dim=s.v_head_dim, scale=s.scale, window=s.window), rt)
        self.n_q, self.n_k = s.num_heads * 2 * s.head_dim, s.num_kv_heads * 2 * s.head_dim
        self.n_v, self.n_mid = s.num_kv_heads * s.v_head_dim, s.num_heads * s.v_head_dim
        self.n_in = self.n_q + self.n_k + self.n_v
        self.lam = None

    def param_decls(self):
        s = self.spec
        d = [ParamDecl("q", (self.n_q, s.hidden_size)), ParamDecl("k", (self.n_k, s.hidden_size)),
             ParamDecl("v", (self.n_v, s.hidden_size)), ParamDecl("o", (s.hidden_size, self.n_mid)),
             ParamDecl("q.b", (self.n_q,), init="around_zero", keep_float32=True),
             ParamDecl("k.b", (self.n_k,), init="around_zero", keep_float32=True),
             ParamDecl("v.b", (self.n_v,), init="around_zero", keep_float32=True)]
        d += [ParamDecl(n, (s.head_dim,), init="around_zero", keep_float32=True) for n in ("lq1", "lk1", "lq2", "lk2")]
        return d

    def bind(self, tensors):
        self.w_in = torch.cat([tensors.pop("q"), tensors.pop("k"), tensors.pop("v")], 0).contiguous()
        self.w_o = tensors.pop("o").contiguous()
        self.bias = torch.cat([tensors.pop(n).to(torch.float32).reshape(-1) for n in ("q.b", "k.b", "v.b")]).contiguous()
        l = {n: tensors.pop(n).to(torch.float64).cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((l["lq1"] * l["lk1"]).sum())) - math.exp(float((l["lq2"] * l["lk2"]).sum())) + self.spec.diff

    def step_weights(self):
        return [self.w_in, self.w_o]

    def step_plans(self):
        return self.core.step_plans()

    def cache_requests(self):
        return self.core.cache_requests()

    def mix(self, ctx, views, proj, mid, scale, writes=True):
        s, kv = self.spec, views[0]
        T = ctx.n_tok
        # [q as 2 * heads heads of 2 * head_dim | k | v], the biases in, q times its temperature, k and v cached
        rows = torch.empty((T, 2 * self.n_q + self.n_k + self.n_v), dtype=self.rt.dtype, device=self.rt.device)
        pos0 = ctx.row_pos if ctx.is_decode else ctx.seq_pos0
        api.conv_norm_rope(proj[:, :self.n_in], rows, None, None, 1, None, None, 0.0, None, None, 0, ctx.row_pos, ctx.row_seq,
                           pos0, ctx.seq_slot, s.num_heads, s.num_kv_heads, 2 * s.head_dim, s.v_head_dim,
                           kv.k if writes else None, kv.v if writes else None, ctx.tables[kv.group] if writes else None,
                           bias=self.bias, q_temp=s.q_temp, q_split=2)
        q = rows[:, :2 * self.n_q]
        k = rows[:, 2 * self.n_q:2 * self.n_q + self.n_k]
        v = rows[:, 2 * self.n_q + self.n_k:]
        maps = torch.empty((T, 2 * self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.core.attend(ctx, kv, q, k, v, None, maps, 1.0, writes=False)
        api.diff_combine(maps, self.lam, s.norm_eps, (1.0 - s.diff) * scale, mid, s.num_heads, s.v_head_dim)

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.mix(ctx, views, proj, mid, 1.0, writes)
        return linear(mid, self.w_o, allow_partial=True)


register_part(DiffAttentionSpec, DiffAttention)
