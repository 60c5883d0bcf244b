"""Mixers that carry a float32 state [key size, value size] per head from token to token, both on one recurrence kernel
(S <- diag(a) S + k v^T, o = S^T q, all operands float32):

* ``LowerBoundRecurrence`` (HGRN2): the forget gate f = l + (1 - l) sigmoid(W_f x + b) is the decay and 1 - f the key;
  q = silu(W_q x); each head's output through an RMS norm with a weight shared by the heads.
* ``StateSpace`` (Mamba-2): x, B, C through a short causal convolution with bias and SiLU (its last taps - 1 inputs are a
  per-sequence state beside the recurrent one), dt = softplus(. + bias), decay exp(-exp(A_log) dt) per head, key dt B,
  query C, a skip D x; the output times silu(z), an RMS norm in parts, the output projection.

forward = one fused input projection -> a kernel that makes the recurrence's float32 operands -> the recurrence over
the state in the cache's state storage -> the output's norm kernel -> the output projection. Both run as branches of a
``ParallelMixer`` (``mix``). The same kernels serve prompts, portions and single tokens.
"""
import torch

from ..cache.requests import StateRequest
from ..config.specs import LowerBoundRecurrenceSpec, StateSpaceSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part
from .linear import linear


def _sequences(ctx):
    """(cu_q, seq_pos0, n_seq) as the recurrence kernels want them: one token a row in a decode step (padding rows carry
    position -1), else the step's sequences."""
    if ctx.is_decode:
        return None, ctx.row_pos, ctx.n_tok
    return ctx.cu_q, ctx.seq_pos0, ctx.n_seq


class LowerBoundRecurrence(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.head_dim > 256:
            raise ValueError(f"the recurrence takes key sizes up to 256, not {s.head_dim}")
        self.n_qk, self.n_mid = s.num_heads * s.head_dim, s.num_heads * s.v_head_dim
        self.n_in = 2 * self.n_qk + self.n_mid

    def param_decls(self):
        s = self.spec
        return [ParamDecl("q", (self.n_qk, s.hidden_size)), ParamDecl("f", (self.n_qk, s.hidden_size)),
                ParamDecl("f.b", (self.n_qk,), init="unit", keep_float32=True),
                ParamDecl("lower", (self.n_qk,), init="fraction", keep_float32=True),
                ParamDecl("v", (self.n_mid, s.hidden_size)), ParamDecl("norm", (s.v_head_dim,), init="norm", keep_float32=True),
                ParamDecl("o", (s.hidden_size, self.n_mid))]

    def bind(self, tensors):
        self.w_in = torch.cat([tensors.pop("q"), tensors.pop("f"), tensors.pop("v")], 0).contiguous()
        self.w_o = tensors.pop("o").contiguous()
        self.f_bias = tensors.pop("f.b").to(torch.float32).contiguous()
        self.lower = tensors.pop("lower").to(torch.float32).contiguous()
        self.norm_weight = tensors.pop("norm").to(torch.float32).contiguous()

    def step_weights(self):
        return [self.w_in, self.w_o]

    def cache_requests(self):
        s = self.spec
        return [StateRequest((s.num_heads, s.head_dim, s.v_head_dim), torch.float32)]

    def mix(self, ctx, views, proj, mid, scale, writes=True):
        s, dev = self.spec, self.rt.device
        if not writes:
            raise ValueError("a recurrent layer cannot read another layer's state")
        T = ctx.n_tok
        q, k, v, a = api.recurrence_operands(T, self.n_qk, self.n_mid, dev)
        api.hgrn2_prepare(proj[:, :self.n_in], self.f_bias, self.lower, q, k, a, v)
        o = torch.empty((T, self.n_mid), dtype=torch.float32, device=dev)
        cu_q, pos0, n_seq = _sequences(ctx)
        api.recurrence(q, k, a, v, o, views[0].state, cu_q, pos0, ctx.seq_slot, n_seq, s.num_heads, s.head_dim, s.v_head_dim)
        api.norm_gate(o, self.norm_weight, s.norm_eps, None, scale, mid, group=s.v_head_dim)

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.mix(ctx, views, proj, mid, 1.0, writes)
        return linear(mid, self.w_o, allow_partial=True)


register_part(LowerBoundRecurrenceSpec, LowerBoundRecurrence)


class StateSpace(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_heads % s.groups or s.state_dim > 256 or not 1 <= s.conv_taps <= api.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"{s.num_heads} heads in {s.groups} groups, states of {s.state_dim} (up to 256), {s.conv_taps} taps "
                             f"(up to {api.SHORT_CONV_MAX_TAPS})")
        self.inner = s.num_heads * s.v_head_dim
        if s.norm_groups < 1 or self.inner % s.norm_groups:
            raise ValueError(f"a norm in {s.norm_groups} parts of {self.inner} coordinates")
        self.n_bc = s.groups * s.state_dim
        self.n_conv = self.inner + 2 * self.n_bc            # the channels that pass the convolution: x, B, C
        self.n_in = 2 * self.inner + 2 * self.n_bc + s.num_heads
        self.n_mid = self.inner

    def param_decls(self):
        s = self.spec
        return [ParamDecl("in", (self.n_in, s.hidden_size)), ParamDecl("conv", (self.n_conv, s.conv_taps), init="taps"),
                ParamDecl("conv.b", (self.n_conv,), init="around_zero", keep_float32=True),
                ParamDecl("dt_bias", (s.num_heads,), init="unit", keep_float32=True),
                ParamDecl("A_log", (s.num_heads,), init="unit", keep_float32=True),
                ParamDecl("D", (s.num_heads,), init="norm", keep_float32=True),
                ParamDecl("norm", (self.inner,), init="norm", keep_float32=True), ParamDecl("o", (s.hidden_size, self.inner))]

    def bind(self, tensors):
        self.w_in = tensors.pop("in").contiguous()
        self.w_o = tensors.pop("o").contiguous()
        self.w_conv = tensors.pop("conv").contiguous()
        self.conv_bias = tensors.pop("conv.b").to(torch.float32).contiguous()
        self.dt_bias = tensors.pop("dt_bias").to(torch.float32).contiguous()
        self.a_log = tensors.pop("A_log").to(torch.float32).contiguous()
        self.skip = tensors.pop("D").to(torch.float32).contiguous()
        self.norm_weight = tensors.pop("norm").to(torch.float32).contiguous()

    def step_weights(self):
        return [self.w_in, self.w_o]

    def cache_requests(self):
        s = self.spec
        r = [StateRequest((s.num_heads, s.state_dim, s.v_head_dim), torch.float32)]
        if s.conv_taps > 1:     # the convolution's memory: the last taps - 1 projected rows [x | B | C] of a sequence
            r.append(StateRequest((s.conv_taps - 1, self.n_conv), self.rt.dtype))
        return r

    def mix(self, ctx, views, proj, mid, scale, writes=True):
        s, dev = self.spec, self.rt.device
        if not writes:
            raise ValueError("a recurrent layer cannot read another layer's state")
        T, inner, nbc = ctx.n_tok, self.inner, self.n_bc
        z = proj[:, :inner]
        xbc = proj[:, inner:inner + self.n_conv]
        dt = proj[:, inner + self.n_conv:self.n_in]
        conv_state = views[1].state if s.conv_taps > 1 else None
        # the recurrence's operands head by head: q = C and k = dt B of the head's group, the head's decay on every channel
        q, k, x, a = api.recurrence_operands(T, s.num_heads * s.state_dim, inner, dev)
        cu_q, pos0, n_seq = _sequences(ctx)
        api.ssd_prepare(xbc, dt, conv_state, self.w_conv, self.conv_bias, s.conv_taps, self.dt_bias, self.a_log, ctx.row_pos,
                        ctx.row_seq, pos0, ctx.seq_slot, s.groups, q, k, a, x)
        if s.conv_taps > 1:
            api.conv_state_update(xbc, conv_state, s.conv_taps, cu_q, pos0, ctx.seq_slot, n_seq)
        y = torch.empty((T, inner), dtype=torch.float32, device=dev)
        api.recurrence(q, k, a, x, y, views[0].state, cu_q, pos0, ctx.seq_slot, n_seq, s.num_heads, s.state_dim, s.v_head_dim)
        api.gate_group_norm(y, x, self.skip, z, self.norm_weight, s.norm_eps, s.norm_groups, scale, mid)

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.mix(ctx, views, proj, mid, 1.0, writes)
        return linear(mid, self.w_o, allow_partial=True)


register_part(StateSpaceSpec, StateSpace)
