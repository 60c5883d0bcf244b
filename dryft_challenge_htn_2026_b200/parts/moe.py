"""Mixture of experts: a router in float32, routed gated feed-forwards, an optional shared expert with a gate.

forward = router kernel (sigmoid scores, choice by score + correction among the best groups, weights from the
scores alone; also the shared expert's gate) -> the chosen experts' gate/up products with the activation ->
their down products, weighted and summed per token, plus gate * shared expert. Steps of many tokens in bfloat16
sort the (token, expert) pairs by expert on the device and run tiles of one expert on the tensor cores; single
tokens, float32 and odd sizes run a warp per output, each pair reading its expert's rows once. The experts' matrices are
stacked [experts, rows, inner] when they are bound, so that a kernel finds an expert's rows by its number.
"""
import torch

from ..config.specs import RoutedMLPSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part
from .linear import SILU, linear

_ACTS = {"silu": api.ACT_SILU, "gelu_tanh": api.ACT_GELU_TANH, "clamped": api.ACT_CLAMPED}


class RoutedMLP(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.activation not in _ACTS:
            raise ValueError(f"activation {s.activation!r} is not implemented ({sorted(_ACTS)})")
        if s.num_experts > api.MOE_MAX_EXPERTS or s.num_experts % s.groups or not 1 <= s.keep_groups <= s.groups or \
                not 1 <= s.top <= min(s.num_experts, 32):
            raise ValueError(f"{s.num_experts} experts in {s.groups} groups, {s.keep_groups} kept, {s.top} chosen")
        if s.top > s.keep_groups * (s.num_experts // s.groups):
            raise ValueError(f"{s.top} experts cannot be chosen from {s.keep_groups} groups of {s.num_experts // s.groups}")
        if s.shared_ff is not None and s.activation not in ("silu", "clamped"):
            raise ValueError("the shared expert runs with SiLU or the clamped gate only")
        if s.activation == "clamped" and (s.limit is None or not s.limit > 0 or
                                          (s.shared_ff is not None and (s.shared_limit is None or not s.shared_limit > 0))):
            raise ValueError(f"the clamped gate wants positive limits, not {s.limit} / {s.shared_limit}")

    def param_decls(self):
        s = self.spec
        d = []
        for e in range(s.num_experts):
            d += [ParamDecl(f"e{e}.gate", (s.expert_ff, s.hidden_size)), ParamDecl(f"e{e}.up", (s.expert_ff, s.hidden_size)),
                  ParamDecl(f"e{e}.down", (s.hidden_size, s.expert_ff))]
        d.append(ParamDecl("router", (s.num_experts, s.hidden_size), init="wide", keep_float32=True))
        if s.correction:
            d.append(ParamDecl("correction", (s.num_experts,), init="around_zero", keep_float32=True))
        if s.shared_ff is not None:
            d += [ParamDecl("shared.gate", (s.shared_ff, s.hidden_size)), ParamDecl("shared.up", (s.shared_ff, s.hidden_size)),
                  ParamDecl("shared.down", (s.hidden_size, s.shared_ff))]
            if s.shared_gate:
                d.append(ParamDecl("shared.sg", (1, s.hidden_size), init="wide", keep_float32=True))
        return d

    def bind(self, tensors):
        s = self.spec
        self.w_gate_up = torch.stack([torch.cat([tensors.pop(f"e{e}.gate"), tensors.pop(f"e{e}.up")], 0)
                                      for e in range(s.num_experts)], 0).contiguous()          # [E, 2 ff, W]
        self.w_down = torch.stack([tensors.pop(f"e{e}.down") for e in range(s.num_experts)], 0).contiguous()   # [E, W, ff]
        self.w_router = tensors.pop("router").to(torch.float32).contiguous()
        self.correction = tensors.pop("correction").to(torch.float32).contiguous() if s.correction else None
        self.w_shared_gu = self.w_shared_down = self.w_shared_gate = None
        if s.shared_ff is not None:
            self.w_shared_gu = torch.cat([tensors.pop("shared.gate"), tensors.pop("shared.up")], 0).contiguous()
            self.w_shared_down = tensors.pop("shared.down").contiguous()
            if s.shared_gate:
                self.w_shared_gate = tensors.pop("shared.sg").to(torch.float32).reshape(-1).contiguous()

    def step_weights(self):
        """What a single-token step streams: the router, the shared expert, and ``top`` experts of the stack."""
        s = self.spec
        w = [self.w_router, self.w_gate_up[:s.top], self.w_down[:s.top]]
        if s.shared_ff is not None:
            w += [self.w_shared_gu, self.w_shared_down]
        return w

    def forward(self, ctx, a):
        s, dev = self.spec, self.rt.device
        T = a.shape[0]
        idx = torch.empty((T, s.top), dtype=torch.int32, device=dev)
        wt = torch.empty((T, s.top), dtype=torch.float32, device=dev)
        sgate = torch.empty((T,), dtype=torch.float32, device=dev) if self.w_shared_gate is not None else None
        api.moe_route(a, self.w_router, self.correction, self.w_shared_gate, s.top, s.groups, s.keep_groups, s.route_scale,
                      idx, wt, sgate, renorm=s.renorm)
        shared = None
        if s.shared_ff is not None and s.activation == "clamped":      # the clamped gate in the product's epilogue
            shared = linear(linear(a, self.w_shared_gu, SILU, act=api.gate_clamped(s.shared_limit)), self.w_shared_down)
        elif s.shared_ff is not None:
            shared = linear(linear(a, self.w_shared_gu, SILU), self.w_shared_down)
        out = torch.empty((T, s.hidden_size), dtype=self.rt.dtype, device=dev)
        # the pair's weight stands on the expert's input (times both sums before the activation) or on its output
        w_in, w_out = (wt, None) if s.weight_on_input else (None, wt)
        limit = s.limit or 0.0
        if api.moe_tiles_take(a, s.expert_ff):
            # many tokens: the pairs sorted by expert, tiles of one expert on the tensor cores
            api.moe_experts_tiles(a, self.w_gate_up, self.w_down, idx, w_out, shared, sgate, out, _ACTS[s.activation],
                                  ctx.scratch if ctx is not None else None, in_wt=w_in, limit=limit)
            return out
        # few tokens (a pair reads its expert's matrices once), float32, or sizes the tiles do not take
        mid = torch.empty((T * s.top, s.expert_ff), dtype=self.rt.dtype, device=dev)
        api.moe_up_rows(a, self.w_gate_up, idx, mid, _ACTS[s.activation], in_wt=w_in, limit=limit)
        api.moe_down_rows(mid, self.w_down, idx, w_out, shared, sgate, out)
        return out


register_part(RoutedMLPSpec, RoutedMLP)
