"""Grouped-query softmax attention without rotation over the paged cache, with a chunk mask or a
window, a logarithmic distance bias, a sink in the softmax's denominator and an output gate, each
switched on by its specification; key and value heads may differ in size.

forward = one fused projection [q; k; v; gate] -> (where the specification asks: a short causal convolution
over time on q, k and v with a per-sequence state, a norm per q and k head, a rotation of the heads' first
coordinates; one kernel) -> k and v into the cache -> attention over the cache with the gate in its epilogue
-> output projection. Further options of the scores: a cap, first tokens that the window keeps, a sink fixed
at zero. Kernels: bfloat16 prompts with equal head sizes of 64
or 128 on tcgen05 tensor cores, other head sizes in steps of 16 on mma.sync, single tokens by a kernel of
their own, and float32 (or any other size) on the float32-arithmetic kernel that serves every phase. The part also runs as a branch of a
``ParallelMixer``, which does the projections of all its branches in one product each: ``mix`` takes
the projected rows and leaves scale * (gated heads) where the caller wants them.
"""
import torch

from ..cache.requests import KVRequest, StateRequest
from ..config.specs import MaskedAttentionSpec, UnitRMSNormSpec
from ..csrc import api
from .attention import QueryTiles
from .base import ParamDecl, Part, build_part, register_part
from .linear import linear


class MaskedAttention(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads are not a multiple of {s.num_kv_heads} key/value heads")
        if max(s.head_dim, s.v_head_dim) > api.MASKED_MAX_HEAD:
            raise ValueError(f"attention kernels take head sizes up to {api.MASKED_MAX_HEAD}, not {s.head_dim} / {s.v_head_dim}")
        if s.chunk is not None and s.chunk < 1:
            raise ValueError(f"a chunk of {s.chunk} positions")
        if s.values_in_keys and s.v_head_dim > s.head_dim:
            raise ValueError(f"values of {s.v_head_dim} numbers cannot be the start of key rows of {s.head_dim}")
        self.n_q, self.n_k = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        self.n_v, self.n_mid = s.num_kv_heads * s.v_head_dim, s.num_heads * s.v_head_dim
        self.n_in = self.n_q + self.n_k + self.n_v + (self.n_mid if s.output_gate else 0)
        self.r1 = self.r2 = self.sink = None
        if s.unit_sink:
            if s.sink:
                raise ValueError("a learned sink and a sink fixed at zero exclude each other")
            self.sink = torch.zeros(s.num_heads, dtype=torch.float32, device=rt.device)   # exp(0) = 1 in the denominator
        if s.keep_first < 0 or (s.softcap is not None and not s.softcap > 0):
            raise ValueError(f"keep_first {s.keep_first} / softcap {s.softcap}")
        # what stands between the projection and the cache
        self.taps = int(s.conv_taps or 1)
        if not 1 <= self.taps <= api.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"a convolution of {s.conv_taps} taps (1 to {api.SHORT_CONV_MAX_TAPS})")
        self.qk_norm = s.qk_norm
        self.qk_norm_weights = s.qk_norm is not None and not isinstance(s.qk_norm, UnitRMSNormSpec)
        if s.value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix {s.value_mix!r} (source, blend or none)")
        self.position = build_part(s.position, rt) if s.position is not None else None
        if self.position is not None and self.position.spec.dim > s.head_dim:
            raise ValueError(f"a rotation over {self.position.spec.dim} coordinates of heads of {s.head_dim}")
        if s.talk and (s.chunk is not None or s.distance_bias or s.sink or s.unit_sink or s.output_gate or s.keep_first
                       or s.softcap is not None or s.values_in_keys):
            raise ValueError("attention with mixed head scores takes a window and nothing else of the masks and options")
        if s.talk and (s.num_heads > api.TALK_MAX_HEADS or s.num_heads * s.v_head_dim > api.TALK_MAX_OUT):
            raise ValueError(f"attention with mixed head scores takes up to {api.TALK_MAX_HEADS} heads and heads x value size "
                             f"up to {api.TALK_MAX_OUT}")
        if s.q_temp is not None and not (int(s.q_temp[1]) >= 1):
            raise ValueError(f"a query temperature every {s.q_temp[1]} positions")
        self.bias = self.talk = None
        self.prepares = self.taps > 1 or self.qk_norm is not None or self.position is not None or s.value_mix is not None \
            or s.bias or s.q_temp is not None
        self.n_qkv = self.n_q + self.n_k + self.n_v
        self.q_norm_w = self.k_norm_w = self.w_conv = None
        self.max_positions = 0
        # the tensor-core kernels take bfloat16 with head sizes in steps of 16; everything else (float32, odd
        # head sizes) runs on the float32-arithmetic kernel, which serves every phase
        self.tensor_core = rt.dtype == torch.bfloat16 and api.masked_bf16_takes(s.head_dim, s.v_head_dim)
        # a cap on the scores and kept first tokens are options of the float32-arithmetic kernel, of the tcgen05 prompt
        # kernel and of the split single-token kernel (equal head sizes); the mma.sync kernels for other sizes lack them
        self.plain_options = s.softcap is None and not s.keep_first
        self.tiles = QueryTiles(api.MASKED_TILE_ROWS) if self.tensor_core else None
        # value rows that are the key rows' first numbers, of sizes beyond those kernels: all heads of a group in one
        # block over the key rows alone (prompts and single tokens)
        self.shared_rows = rt.dtype == torch.bfloat16 and not self.tensor_core and s.values_in_keys and self.plain_options \
            and not (s.distance_bias or s.sink or s.unit_sink or s.output_gate) and api.shared_rows_takes(s.head_dim, s.v_head_dim)
        self.row_tiles = QueryTiles(api.shared_rows_tile_queries(s.num_heads // s.num_kv_heads)) if self.shared_rows else None
        # equal head sizes of 64 or 128: prompts run on the tcgen05 kernel (its masked build), in tiles of 128 queries
        self.tc_tiles = QueryTiles(api.TC_TILE_ROWS) if self.tensor_core and s.head_dim == s.v_head_dim \
            and s.head_dim in api.TC_ATTENTION_HEAD_DIMS and not s.values_in_keys else None
        # mixed head scores in bfloat16 with sizes in steps of 16: tiles of 16 queries with all their heads on mma.sync
        self.talk_tiles = QueryTiles(api.TALK_TILE_ROWS) if s.talk and rt.dtype == torch.bfloat16 and \
            api.talk_bf16_takes(s.num_heads, s.num_kv_heads, s.head_dim, s.v_head_dim) else None

    def step_plans(self):
        return [t for t in (self.tiles, self.tc_tiles, self.row_tiles, self.talk_tiles) if t is not None]

    def param_decls(self):
        s = self.spec
        d = [ParamDecl("q", (self.n_q, s.hidden_size)), ParamDecl("k", (self.n_k, s.hidden_size)),
             ParamDecl("v", (self.n_v, s.hidden_size)), ParamDecl("o", (s.hidden_size, self.n_mid))]
        if s.output_gate:
            d.append(ParamDecl("g", (self.n_mid, s.hidden_size)))
        if s.distance_bias:
            d += [ParamDecl("r1", (s.num_heads,), init="positive", keep_float32=True),
                  ParamDecl("r2", (s.num_heads,), init="positive", keep_float32=True)]
        if s.sink:
            d.append(ParamDecl("sink", (s.num_heads,), init="unit", keep_float32=True))
        if self.taps > 1:
            d += [ParamDecl("q.conv", (self.n_q, self.taps), init="taps"), ParamDecl("k.conv", (self.n_k, self.taps), init="taps"),
                  ParamDecl("v.conv", (self.n_v, self.taps), init="taps")]
        if self.qk_norm_weights:
            d += [ParamDecl("q.norm", (s.head_dim,), init="norm", keep_float32=True),
                  ParamDecl("k.norm", (s.head_dim,), init="norm", keep_float32=True)]
        if s.value_mix is not None:
            d.append(ParamDecl("vmix", (), init="fraction", keep_float32=True))
        if s.bias:
            d += [ParamDecl("q.b", (self.n_q,), init="around_zero", keep_float32=True),
                  ParamDecl("k.b", (self.n_k,), init="around_zero", keep_float32=True),
                  ParamDecl("v.b", (self.n_v,), init="around_zero", keep_float32=True)]
        if s.talk:
            d.append(ParamDecl("talk", (s.num_heads, s.num_heads), init="near_identity", keep_float32=True))
        return d

    def bind(self, tensors):
        rows = [tensors.pop("q"), tensors.pop("k"), tensors.pop("v")]
        if self.spec.output_gate:
            rows.append(tensors.pop("g"))
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_o = tensors.pop("o").contiguous()
        if self.spec.distance_bias:
            self.r1 = tensors.pop("r1").to(torch.float32).contiguous()
            self.r2 = tensors.pop("r2").to(torch.float32).contiguous()
        if self.spec.sink:
            self.sink = tensors.pop("sink").to(torch.float32).contiguous()
        if self.taps > 1:
            self.w_conv = torch.cat([tensors.pop("q.conv"), tensors.pop("k.conv"), tensors.pop("v.conv")], 0).contiguous()
        if self.qk_norm_weights:
            self.q_norm_w = tensors.pop("q.norm").to(torch.float32).contiguous()
            self.k_norm_w = tensors.pop("k.norm").to(torch.float32).contiguous()
        if self.spec.value_mix is not None:
            self.v_mix = tensors.pop("vmix").to(torch.float32).reshape(1).contiguous()
        if self.spec.bias:
            self.bias = torch.cat([tensors.pop(n).to(torch.float32).reshape(-1) for n in ("q.b", "k.b", "v.b")]).contiguous()
        if self.spec.talk:
            self.talk = tensors.pop("talk").to(torch.float32).contiguous()

    def step_weights(self):
        return [self.w_in, self.w_o]

    def cache_requests(self):
        s = self.spec
        r = [KVRequest(s.num_kv_heads, s.head_dim, s.window, self.rt.dtype, s.v_head_dim, s.chunk, s.keep_first, s.values_in_keys)]
        if self.taps > 1:     # the convolution's memory: the last taps - 1 projected rows [q | k | v] of a sequence
            r.append(StateRequest((self.taps - 1, self.n_qkv), self.rt.dtype))
        return r

    def prepare(self, max_positions):
        self.max_positions = max_positions
        if self.position is not None:
            self.position.tables(max_positions)

    def prepared_rows(self, ctx, views, proj, writes=True):
        """[q | k | v] of the projection rows after the convolution, the head norm and the rotation, as a dense
        matrix; with ``writes`` the k and v heads also go into the cache; the convolution's state moves on behind it."""
        s = self.spec
        if not writes and self.taps > 1:
            raise ValueError("a layer with a short convolution cannot run on another layer's cache entry")
        out = torch.empty((ctx.n_tok, self.n_qkv), dtype=self.rt.dtype, device=self.rt.device)
        state = views[1].state if self.taps > 1 else None
        cos = sin = None
        rot = 0
        if self.position is not None:
            rot = self.position.spec.dim
            cos, sin = self.position.tables(max(self.max_positions, ctx.max_position + 1))
        pos0 = ctx.row_pos if ctx.is_decode else ctx.seq_pos0     # one token a row: its position is what came before
        qkv = proj[:, :self.n_qkv]
        norm_mode = api.NORM_NONE if self.qk_norm is None else \
            api.NORM_AFTER_ROTATION if s.norm_after_rotation else api.NORM_BEFORE_ROTATION
        v_src = None
        if s.value_mix == "blend":
            v_src = ctx.carry.get(("value_mix", self.n_v))
            if v_src is None:
                raise ValueError("a layer blends its values with a source layer's, but none ran before it in this step")
        api.conv_norm_rope(qkv, out, state, self.w_conv, self.taps, self.q_norm_w, self.k_norm_w,
                           self.qk_norm.eps if self.qk_norm is not None else 0.0, cos, sin, rot, ctx.row_pos, ctx.row_seq,
                           pos0, ctx.seq_slot, s.num_heads, s.num_kv_heads, s.head_dim, s.v_head_dim,
                           views[0].k if writes else None, views[0].v if writes else None,
                           ctx.tables[views[0].group] if writes else None, norm_mode=norm_mode,
                           v_mix=self.v_mix if v_src is not None else None, v_src=v_src, bias=self.bias, q_temp=s.q_temp)
        if s.value_mix == "source":      # this step's values, for the layers that blend theirs with them
            ctx.carry[("value_mix", self.n_v)] = out[:, self.n_q + self.n_k:]
        if self.taps > 1:
            api.conv_state_update(qkv, state, self.taps, None if ctx.is_decode else ctx.cu_q, pos0, ctx.seq_slot, ctx.n_seq)
        return out

    def mix(self, ctx, views, proj, mid, scale, writes=True):
        """``proj`` [tokens, n_in]: this part's rows of a projection (possibly columns of a wider matrix);
        ``mid`` [tokens, n_mid]: where scale * (gated heads) go."""
        s, kv = self.spec, views[0]
        gate = proj[:, self.n_q + self.n_k + self.n_v:] if s.output_gate else None
        if self.prepares:
            proj = self.prepared_rows(ctx, views, proj, writes)
            writes = False          # that kernel has stored the step's keys and values
        q = proj[:, :self.n_q]
        k = proj[:, self.n_q:self.n_q + self.n_k]
        v = proj[:, self.n_q + self.n_k:self.n_q + self.n_k + self.n_v]
        return self.attend(ctx, kv, q, k, v, gate, mid, scale, writes)

    def attend(self, ctx, kv, q, k, v, gate, mid, scale, writes=True):
        """Attention of the query rows ``q`` over the cache entry ``kv``, into ``mid``; with ``writes`` the step's
        ``k`` and ``v`` rows go into the cache first. Picks the kernel by type, phase and head sizes."""
        s = self.spec
        table = ctx.tables[kv.group]
        if self.talk is not None:     # mixed head scores: the tensor-core kernel, or the float32-arithmetic one for every phase and type
            if writes:
                api.kv_write(k, v, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, s.num_kv_heads, s.head_dim, s.v_head_dim)
            if self.talk_tiles is not None and api.talk_operands(q, mid):
                sizes = (s.num_heads, s.num_kv_heads, s.head_dim, s.v_head_dim, s.window, s.scale, self.talk)
                if not ctx.is_decode:
                    return api.attention_talk_bf16(q, mid, scale, kv.k, kv.v, table, *sizes, tiles=ctx.plans[self.talk_tiles.key],
                                                   cu_q=ctx.cu_q, seq_pos0=ctx.seq_pos0)
                nsplit = api.talk_decode_splits(ctx.n_tok, s.num_heads, table.shape[1], s.window)
                ws = ctx.scratch(("talk_decode", ctx.n_tok, s.num_heads, s.v_head_dim, nsplit),
                                 lambda: api.talk_decode_ws(ctx.n_tok, s.num_heads, s.v_head_dim, nsplit, self.rt.device)) \
                    if nsplit > 1 else None
                return api.attention_talk_bf16(q, mid, scale, kv.k, kv.v, table, *sizes, row_pos=ctx.row_pos, nsplit=nsplit, ws=ws)
            return api.attention_talk(q, mid, scale, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, s.num_heads, s.num_kv_heads,
                                      s.head_dim, s.v_head_dim, s.window, s.scale, self.talk)
        sizes = (s.num_heads, s.num_kv_heads, s.head_dim, s.v_head_dim, s.window, s.chunk, s.scale)
        if self.tensor_core and ctx.is_decode and not s.values_in_keys \
                and api.masked_decode_streams(q, mid, gate, s.head_dim, s.v_head_dim):
            # single tokens, keys and values of one size: the library's split decode kernel in its masked build
            if writes:
                api.kv_write(k, v, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, s.num_kv_heads, s.head_dim, s.v_head_dim)
            nsplit = api.masked_decode_splits(ctx.n_seq, s.num_kv_heads, s.num_heads // s.num_kv_heads, table.shape[1],
                                              s.window, s.chunk)
            ws_acc, ws_ml = ctx.scratch(("attn_decode", ctx.n_seq, s.num_heads, s.head_dim, nsplit),
                                        lambda: api.attention_decode_ws(ctx.n_seq, s.num_heads, s.head_dim, nsplit, self.rt.device))
            return api.attention_decode_masked_bf16(q, mid, gate, scale, kv.k, kv.v, ctx.row_pos, table, s.num_heads,
                                                    s.num_kv_heads, s.head_dim, s.window, s.chunk, s.scale, nsplit, ws_acc,
                                                    ws_ml, self.r1, self.r2, self.sink, s.softcap, s.keep_first)
        span = api.masked_decode_span(s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.chunk, table.shape[1], ctx.n_tok) \
            if self.tensor_core and self.plain_options and ctx.is_decode \
            and all(t is None or t.stride(0) % 2 == 0 for t in (q, mid, gate)) else None
        if span is not None:      # single tokens: the kernel stores each token's key and value itself
            ws = None
            if span[1] > 1:
                ws = ctx.scratch(("masked_decode", ctx.n_tok, s.num_heads, s.v_head_dim, span[1]),
                                 lambda: api.masked_decode_ws(ctx.n_tok, s.num_heads, s.v_head_dim, span[1], self.rt.device))
            return api.attention_masked_decode_bf16(q, mid, gate, scale, kv.k, kv.v, ctx.row_pos, table, *sizes, span,
                                                    self.r1, self.r2, self.sink, k if writes else None, v if writes else None, ws)
        if writes:
            api.kv_write(k, v, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, s.num_kv_heads, s.head_dim, s.v_head_dim)
        if self.shared_rows and gate is None and api.shared_rows_operands(q, mid):
            if not ctx.is_decode:
                return api.attention_shared_rows_bf16(q, mid, scale, kv.k, table, *sizes, tiles=ctx.plans[self.row_tiles.key],
                                                      cu_q=ctx.cu_q, seq_pos0=ctx.seq_pos0)
            nsplit = api.shared_rows_splits(ctx.n_tok, s.num_heads, s.num_kv_heads, table.shape[1], s.window, s.chunk)
            ws = ctx.scratch(("shared_rows", ctx.n_tok, s.num_heads, s.v_head_dim, nsplit),
                             lambda: api.shared_rows_ws(ctx.n_tok, s.num_heads, s.v_head_dim, nsplit, self.rt.device)) \
                if nsplit > 1 else None
            return api.attention_shared_rows_bf16(q, mid, scale, kv.k, table, *sizes, row_pos=ctx.row_pos, nsplit=nsplit, ws=ws)
        if self.tc_tiles is not None and not ctx.is_decode and api.masked_tc_takes(q, mid, gate, s.head_dim, s.v_head_dim):
            return api.attention_masked_prefill_tc(q, mid, gate, scale, kv.k, kv.v, ctx.plans[self.tc_tiles.key], ctx.cu_q,
                                                   ctx.seq_pos0, table, s.num_heads, s.num_kv_heads, s.head_dim, s.window,
                                                   s.chunk, s.scale, self.r1, self.r2, self.sink, s.softcap, s.keep_first)
        even = all(t is None or (t.stride(0) % 2 == 0 and t.data_ptr() % 4 == 0) for t in (q, mid, gate))
        if self.tensor_core and self.plain_options and not ctx.is_decode and even:
            return api.attention_masked_prefill_bf16(q, mid, gate, scale, kv.k, kv.v, ctx.plans[self.tiles.key], ctx.cu_q,
                                                     ctx.seq_pos0, table, *sizes, self.r1, self.r2, self.sink)
        api.attention_masked(q, mid, gate, scale, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, *sizes, self.r1, self.r2,
                             self.sink, s.softcap, s.keep_first)

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.mix(ctx, views, proj, mid, 1.0, writes)
        return linear(mid, self.w_o, allow_partial=True)


register_part(MaskedAttentionSpec, MaskedAttention)
