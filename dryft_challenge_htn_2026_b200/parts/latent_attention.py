"""Softmax attention whose queries, keys and values come through low-rank latents, over a cache that holds the
key/value latent and one rotated key part per token.

forward = one fused down projection [dq; dkv] -> (norm of the query latent; norm of the key/value latent and the
rotation of the shared key part, both straight into the cache; one kernel) -> query up projection -> per head the
plain key's up projection moved to the query's side, q_h <- [W_uk_h^T q_plain | q_rot rotated], so that a score is
q_h . [c | k_rot] against the cached row itself -> attention with all heads on the one cached head (the masked
attention's kernels: float32-arithmetic, mma.sync prompts, single tokens; rows wider than 256 on the kernel for rows that
are key and value at once), whose values are the latents -> per head
W_uv times the latent output -> output projection. Nothing per head is ever cached or recomputed for old tokens, so
a step costs the same however a prompt is cut.
"""
import torch

from ..cache.requests import KVRequest
from ..config.specs import LatentAttentionSpec, MaskedAttentionSpec
from ..csrc import api
from .attention_masked import MaskedAttention
from .base import ParamDecl, Part, build_part, register_part
from .linear import linear

# steps of more rows than this take the per-head products of a bfloat16 model through the library's batched matrix
# product (tensor cores); float32 takes the row kernels. (At 32 heads of 128 over latents of 512 the row kernels took
# 127 and 57 us for 8 tokens, the batched product 10.)
HEAD_PRODUCT_ROWS = 0


class LatentAttention(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        self.position = build_part(s.position, rt) if s.position is not None else None
        if self.position is not None and not getattr(self.position, "pairs", False):
            raise TypeError(f"{type(self.position).__name__}: the shared key part is rotated by neighbouring pairs")
        if self.position is not None and self.position.spec.dim > s.rot_dim:
            raise ValueError(f"a rotation over {self.position.spec.dim} coordinates of a rotated part of {s.rot_dim}")
        self.lat = s.kv_rank + s.rot_dim                     # what a token holds in the cache: the key row
        self.n_q = s.num_heads * (s.head_dim + s.rot_dim)
        self.n_down = s.q_rank + s.kv_rank + s.rot_dim
        self.n_mid = s.num_heads * s.v_head_dim
        # the attention itself: every query head on the one cached head, keys [c | k_rot], values c
        self.core = MaskedAttention(MaskedAttentionSpec(
            hidden_size=s.hidden_size, num_heads=s.num_heads, num_kv_heads=1, head_dim=self.lat, v_head_dim=s.kv_rank,
            scale=s.scale, chunk=s.chunk, window=s.window, values_in_keys=True), rt)
        self.max_positions = 0

    def param_decls(self):
        s = self.spec
        return [ParamDecl("dq", (s.q_rank, s.hidden_size)), ParamDecl("dq.norm", (s.q_rank,), init="norm", keep_float32=True),
                ParamDecl("uq", (self.n_q, s.q_rank)), ParamDecl("dkv", (s.kv_rank + s.rot_dim, s.hidden_size)),
                ParamDecl("dkv.norm", (s.kv_rank,), init="norm", keep_float32=True),
                ParamDecl("uk", (s.num_heads * s.head_dim, s.kv_rank)), ParamDecl("uv", (s.num_heads * s.v_head_dim, s.kv_rank)),
                ParamDecl("o", (s.hidden_size, self.n_mid))]

    def bind(self, tensors):
        self.w_down = torch.cat([tensors.pop("dq"), tensors.pop("dkv")], 0).contiguous()
        self.q_norm_w = tensors.pop("dq.norm").to(torch.float32).contiguous()
        self.kv_norm_w = tensors.pop("dkv.norm").to(torch.float32).contiguous()
        self.w_uq = tensors.pop("uq").contiguous()
        self.w_uk = tensors.pop("uk").contiguous()
        self.w_uv = tensors.pop("uv").contiguous()
        self.w_o = tensors.pop("o").contiguous()

    def step_weights(self):
        return [self.w_down, self.w_uq, self.w_uk, self.w_uv, self.w_o]

    def step_plans(self):
        return self.core.step_plans()

    def cache_requests(self):
        s = self.spec
        return [KVRequest(1, self.lat, s.window, self.rt.dtype, s.kv_rank, s.chunk, values_in_keys=True)]

    def prepare(self, max_positions):
        self.max_positions = max_positions
        if self.position is not None:
            self.position.tables(max_positions)

    def _tables(self, ctx):
        if self.position is None:
            return None, None, 0
        cos, sin = self.position.tables(max(self.max_positions, ctx.max_position + 1))
        return cos, sin, self.position.spec.dim

    def queries(self, ctx, q):
        """q of the up projection -> the rows the attention runs on: head by head [W_uk_h^T q_plain | q_rot rotated]."""
        s, T = self.spec, q.shape[0]
        H, D, R, L = s.num_heads, s.head_dim, s.rot_dim, s.kv_rank
        cos, sin, rot = self._tables(ctx)
        out = torch.empty((T, H * self.lat), dtype=self.rt.dtype, device=self.rt.device)
        batched = self.rt.dtype == torch.bfloat16 and T > HEAD_PRODUCT_ROWS
        if batched:      # [H, T, D] x [H, D, L] -> the plain parts of out, seen as [H, T, L]
            torch.bmm(q.view(T, H, D + R)[:, :, :D].transpose(0, 1), self.w_uk.view(H, D, L),
                      out=out.view(T, H, self.lat)[:, :, :L].transpose(0, 1))
        api.latent_query(q, self.w_uk, out, cos, sin, rot, ctx.row_pos, H, D, R, L, plain=not batched)
        return out

    def values(self, o_lat):
        """The attention's output over latents -> head by head W_uv_h times it."""
        s, T = self.spec, o_lat.shape[0]
        H, L, Dv = s.num_heads, s.kv_rank, s.v_head_dim
        out = torch.empty((T, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        if self.rt.dtype == torch.bfloat16 and T > HEAD_PRODUCT_ROWS:
            torch.bmm(o_lat.view(T, H, L).transpose(0, 1), self.w_uv.view(H, Dv, L).transpose(1, 2),
                      out=out.view(T, H, Dv).transpose(0, 1))
        else:
            api.latent_value(o_lat, self.w_uv, out, H, L, Dv)
        return out

    def forward(self, ctx, views, a, writes=True):
        s, kv = self.spec, views[0]
        dtype, dev = self.rt.dtype, self.rt.device
        down = linear(a, self.w_down)
        cq = torch.empty((ctx.n_tok, s.q_rank), dtype=dtype, device=dev)
        cos, sin, rot = self._tables(ctx)
        api.latent_norm_rope_write(down, cq, self.q_norm_w, self.kv_norm_w, s.norm_eps, cos, sin, rot, ctx.row_pos,
                                   ctx.row_seq, s.q_rank, s.kv_rank, s.rot_dim, kv.k if writes else None,
                                   kv.v if writes else None, ctx.tables[kv.group] if writes else None)
        q = self.queries(ctx, linear(cq, self.w_uq))
        o_lat = torch.empty((ctx.n_tok, s.num_heads * s.kv_rank), dtype=dtype, device=dev)
        self.core.attend(ctx, kv, q, None, None, None, o_lat, 1.0, writes=False)
        return linear(self.values(o_lat), self.w_o, allow_partial=True)


register_part(LatentAttentionSpec, LatentAttention)
