"""Python entry points of the CUDA kernels: thin ctypes wrappers that take torch tensors.

Every function launches on torch's current CUDA stream and returns without synchronising, so
the calls can be captured in a CUDA graph. Arguments are checked here (device, dtype, contiguity,
the sizes a kernel supports); a kernel that cannot take a size raises ``KernelError`` rather than
compute something else. There is no CPU or library fallback behind these functions.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

PAGE = 64  # tokens per cache page; must equal DK_PAGE in common.cuh


class KernelError(RuntimeError):
    pass


_pdl = False


def set_pdl(on):
    """Programmatic dependent launch for every kernel launched from here on."""
    global _pdl
    _pdl = bool(on)
    for lib in list(build._libs.values()):
        lib.dk_set_pdl(int(_pdl))


_cuda_seen = False


def _lib(source, defines=None):
    global _cuda_seen
    if not _cuda_seen:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: the kernels of this library run on an NVIDIA B200 (sm_100a) only")
        _cuda_seen = True
    key = (source, tuple(sorted((defines or {}).items())))
    fresh = key not in build._libs
    lib = build.load_lib(source, defines)
    if fresh:
        lib.dk_set_pdl.argtypes = [c_int]
        lib.dk_set_pdl(int(_pdl))
        lib.dk_error_string.restype = ctypes.c_char_p
    return lib


_sm_count = None


def sm_count():
    """Multiprocessors of the device the kernels run on; every launch plan is sized by it. Without
    a CUDA device (plans looked at on another machine) the B200's 148."""
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _sm_count


_launches = 0


def launch_count():
    """Kernels of this library launched so far through these wrappers (library products not counted)."""
    return _launches


def _check(lib, err, what, kernels=1):
    global _launches
    _launches += kernels
    if err != 0:
        msg = lib.dk_error_string(err).decode()
        raise KernelError(f"{what}: CUDA error {err} ({msg})")


# torch's current stream as a raw pointer. The call through torch.cuda.current_stream() builds a Stream
# object (3.6 us, a quarter of what a launch costs on the host: short prefill steps are bound by that);
# the raw getter takes 0.1 us. One device: its index is looked up once.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream_ptr():
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _stream():
    return c_void_p(_stream_ptr())


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _dt(t):
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 or bfloat16")


def _need(t, name, dtype=None, dim=None):
    if t is None:
        return
    if not t.is_cuda or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


class Partial:
    """The output of a split-K product that has not been added up yet: float32 [slices, rows,
    cols]; the true value is the sum over slices. ``add_rmsnorm`` and ``qk_norm_rope_write`` take
    it in place of a tensor and add the slices up while they read; anything else calls ``sum()``."""

    def __init__(self, ws):
        self.ws = ws

    @property
    def shape(self):
        return self.ws.shape[1:]

    def sum(self, dtype=torch.bfloat16):
        out = torch.empty(self.shape, dtype=torch.bfloat16, device=self.ws.device)
        lib = _lib("gemm.cu")
        _check(lib, lib.dk_sum_partials(_p(self.ws), _p(out), c_longlong(out.numel()), self.ws.shape[0], _stream()),
               "sum_partials")
        return out.to(dtype)


def _parts(x):
    """(tensor or None, partial pointer, slices, stride) of an argument that may be a Partial."""
    if isinstance(x, Partial):
        return None, _p(x.ws), x.ws.shape[0], c_longlong(x.ws.shape[1] * x.ws.shape[2])
    return x, c_void_p(0), 0, c_longlong(0)


# ------------------------------------------------------------------------------------ row kernels
def embed_rmsnorm(tok, embed, norm_w, eps, h_out, a_out):
    """h_out[t] = embed[tok[t]] (float32); a_out[t] = rmsnorm(h_out[t]) * norm_w."""
    _need(tok, "tok", torch.int32, 1), _need(embed, "embed", None, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(h_out, "h_out", torch.float32, 2), _need(a_out, "a_out", embed.dtype, 2)
    lib = _lib("elementwise.cu")
    n, (V, H) = tok.numel(), embed.shape
    _check(lib, lib.dk_embed_rmsnorm(_dt(embed), _p(tok), _p(embed), _p(norm_w), c_float(eps), n, H, V, _p(h_out),
                                     _p(a_out), _stream()), "embed_rmsnorm")


def add_rmsnorm(h, delta, norm_w, eps, a_out, rows=None):
    """h += delta (delta may be None); a_out = rmsnorm(h) * norm_w. With ``rows`` (int32 indices)
    only those rows are normalised into a_out[0..len(rows)) and h is left unchanged."""
    delta, parts, n_parts, stride = _parts(delta)
    _need(h, "h", torch.float32, 2), _need(delta, "delta", a_out.dtype, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(rows, "rows", torch.int32, 1), _need(a_out, "a_out", None, 2)
    lib = _lib("elementwise.cu")
    n = h.shape[0] if rows is None else rows.numel()
    _check(lib, lib.dk_add_rmsnorm(_dt(a_out), _p(h), _p(delta), parts, n_parts, stride, _p(rows), _p(norm_w),
                                   c_float(eps), n, h.shape[1], _p(a_out), _stream()), "add_rmsnorm")


def silu_mul(gu, out):
    """out[r, c] = silu(gu[r, c]) * gu[r, I + c] for gu [rows, 2I]."""
    _need(gu, "gu", None, 2), _need(out, "out", gu.dtype, 2)
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_silu_mul(_dt(gu), _p(gu), _p(out), c_longlong(gu.shape[0]), out.shape[1], _stream()), "silu_mul")


def gather_rows_f32(src, rows, out):
    _need(src, "src", torch.float32, 2), _need(rows, "rows", torch.int32, 1), _need(out, "out", torch.float32, 2)
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_gather_rows_f32(_p(src), _p(rows), _p(out), rows.numel(), src.shape[1], _stream()), "gather_rows")


def qk_norm_rope_write(qkv, q_out, q_norm_w, k_norm_w, cos, sin, row_pos, row_seq, page_table, k_store, v_store,
                       n_heads, n_kv_heads, head_dim, eps, write_kv=True, dense_out=None):
    """Per-head RMSNorm (weights may be None), rotate-half rotation (cos/sin [positions, hd/2]
    float32, may be None), q to q_out [T, nh*hd], k and v into the paged stores
    [pages, n_kv, PAGE, hd] at each token's position. Rows with position < 0 are skipped.
    With ``dense_out`` [T, (nh + 2 nkv) * hd] the heads go there instead (q and k normalised and
    rotated as asked, v copied) and neither q_out nor the cache is written."""
    width, n_tok = qkv.shape[1], qkv.shape[0]
    qkv, parts, n_parts, stride = _parts(qkv)
    if dense_out is not None:
        _need(dense_out, "dense_out", None, 2)
        if tuple(dense_out.shape) != (n_tok, width):
            raise KernelError(f"dense_out {tuple(dense_out.shape)} must have the projection's shape {(n_tok, width)}")
        q_out = dense_out if q_out is None else q_out
    _need(qkv, "qkv", q_out.dtype, 2), _need(q_out, "q_out", None, 2)
    _need(q_norm_w, "q_norm_w", torch.float32, 1), _need(k_norm_w, "k_norm_w", torch.float32, 1)
    _need(cos, "cos", torch.float32, 2), _need(sin, "sin", torch.float32, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", q_out.dtype), _need(v_store, "v_store", q_out.dtype)
    if head_dim % 2 or head_dim > 256:
        raise KernelError(f"head size {head_dim} not supported: even, at most 256")
    if width != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"qkv width {width} != (nh + 2 nkv) * hd")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_qk_norm_rope_write(_dt(q_out), _p(qkv), parts, n_parts, stride, _p(q_out), _p(dense_out), _p(q_norm_w),
                                          _p(k_norm_w), _p(cos), _p(sin), _p(row_pos), _p(row_seq), _p(page_table),
                                          page_table.shape[1], _p(k_store), _p(v_store), n_tok, n_heads, n_kv_heads,
                                          head_dim, c_float(eps), int(bool(write_kv)), _stream()), "qk_norm_rope_write")


# -------------------------------------------------------------------------------------- attention
def attention_generic(q, out, k_store, v_store, row_pos, row_seq, page_table, n_heads, n_kv_heads, head_dim, window,
                      scale):
    """Float32-arithmetic attention of every token row over its sequence's cached keys up to its
    own position (window: keys a query sees, 0 = all). Any phase; float32 or bfloat16 storage."""
    _need(q, "q", None, 2), _need(out, "out", q.dtype, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    if head_dim > 256 or n_heads % n_kv_heads:
        raise KernelError(f"attention: head size {head_dim} (max 256) / heads {n_heads}:{n_kv_heads} not supported")
    lib = _lib("attention_generic.cu")
    _check(lib, lib.dk_attention_generic(_dt(q), _p(q), _p(out), _p(k_store), _p(v_store), _p(row_pos), _p(row_seq),
                                         _p(page_table), page_table.shape[1], q.shape[0], n_heads, n_kv_heads,
                                         head_dim, int(window or 0), c_float(scale), _stream()), "attention_generic")


def _attn_lib(head_dim):
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"bfloat16 attention: head size {head_dim} not supported (multiples of 16 up to 256)")
    return _lib("attention_bf16.cu", {"HD": head_dim})


MMA_TILE_ROWS = 64   # queries a block of attention_prefill_bf16 takes


def attention_prefill_bf16(q, out, k_store, v_store, tiles, cu_q, seq_pos0, page_table, n_heads, n_kv_heads, head_dim,
                           window, scale):
    """Ragged causal attention of query chunks (tensor cores). tiles [n, 2] int32 = (sequence,
    first query of a 64-row tile within its chunk); cu_q [nseq+1]; seq_pos0 [nseq] cached length
    before the chunk."""
    _need(q, "q", torch.bfloat16, 2), _need(out, "out", torch.bfloat16, 2), _need(tiles, "tiles", torch.int32, 2)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    if n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} query heads are not a multiple of {n_kv_heads} kv heads")
    lib = _attn_lib(head_dim)
    _check(lib, lib.dk_attn_prefill_bf16(_p(q), _p(out), _p(k_store), _p(v_store), _p(tiles), tiles.shape[0], _p(cu_q),
                                         _p(seq_pos0), _p(page_table), page_table.shape[1], n_heads, n_kv_heads,
                                         int(window or 0), c_float(scale), _stream()), "attention_prefill_bf16")


DECODE_MAX_SPLITS = 32          # the merge kernel takes 4 x 32 parts a head


def decode_splits(n_seq, n_kv_heads, group, table_pages=0, max_splits=8, resident_blocks=None):
    """Number of key splits for decode attention, fixed for a batch size and a page-table width (it
    must not depend on sequence lengths, which change under a captured graph; the table width is
    the graph's own). While all blocks fit the GPU at once (two per SM with the three-deep rings):
    as many splits as keep it so, up to ``max_splits``, and for long tables up to DECODE_MAX_SPLITS
    while a split keeps 16 pages (one sequence of 32,768 tokens in 8 splits of its 8 kv heads kept
    64 of 296 block slots busy: 0.55 of the copy peak for the step). Beyond that: enough for about
    six waves of blocks, which evens out sequences of unequal lengths (measured at batch 64: 133 us
    unsplit, 115 us in four splits)."""
    if resident_blocks is None:
        resident_blocks = 2 * sm_count()
    blocks = n_seq * n_kv_heads * ((group + 15) // 16)
    if blocks <= resident_blocks:
        room = resident_blocks // blocks
        return max(1, min(max_splits, room), min(DECODE_MAX_SPLITS, room, table_pages // 16))
    return max(1, min(max_splits, -(-6 * resident_blocks // blocks)))


def attention_decode_ws(n_seq, n_heads, head_dim, nsplit, device):
    """Scratch for attention_decode_bf16: float32 partial outputs and (max, sum) pairs, one per warp
    of every block: 4 * nsplit a head."""
    parts = 4 * nsplit
    return (torch.empty(n_seq * n_heads * parts * head_dim, dtype=torch.float32, device=device),
            torch.empty(n_seq * n_heads * parts * 2, dtype=torch.float32, device=device))


def attention_decode_bf16(q, out, k_store, v_store, row_pos, page_table, n_heads, n_kv_heads, head_dim, window, scale,
                          nsplit, ws_acc, ws_ml):
    """One query token per sequence over its cached keys [.., row_pos] (tensor cores). The keys are
    split over ``nsplit`` blocks of four warps; every warp leaves a partial result and a second
    kernel merges the 4 * nsplit of a head."""
    _need(q, "q", torch.bfloat16, 2), _need(out, "out", torch.bfloat16, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(page_table, "page_table", torch.int32, 2)
    _need(ws_acc, "ws_acc", torch.float32), _need(ws_ml, "ws_ml", torch.float32)
    n_seq = q.shape[0]
    if not 1 <= nsplit <= DECODE_MAX_SPLITS:
        raise KernelError(f"attention_decode_bf16: {nsplit} splits, the merge takes 1 to {DECODE_MAX_SPLITS}")
    if ws_acc is None or ws_ml is None or ws_acc.numel() < n_seq * n_heads * 4 * nsplit * head_dim \
            or ws_ml.numel() < n_seq * n_heads * 4 * nsplit * 2:
        raise KernelError("attention_decode_bf16: scratch too small for this batch and split count")
    lib = _attn_lib(head_dim)
    _check(lib, lib.dk_attn_decode_bf16(_p(q), _p(out), _p(ws_acc), _p(ws_ml), _p(k_store), _p(v_store), _p(row_pos),
                                        _p(page_table), page_table.shape[1], n_seq, n_heads, n_kv_heads,
                                        int(window or 0), c_float(scale), nsplit, _stream()), "attention_decode_bf16", 2)


# ---------------------------------------------------------------------------------------- products
MODE_STORE, MODE_STORE_F32, MODE_SILU, MODE_XIELU = 0, 1, 2, 3
GATE_GELU = (1.0, 0.0)      # ``act`` of a MODE_SILU product whose gate goes through the tanh form of GELU instead of SiLU


def gate_clamped(limit):
    """``act`` of a MODE_SILU product with the clamped gate: g' = min(g, limit), u' = clamp(u, -limit, limit),
    out = g' sigmoid(1.702 g') (u' + 1)."""
    return (2.0, float(limit))


def sgemm(x, w, out, mode=MODE_STORE, act=(0.0, 0.0)):
    """float32 out = x . w^T on CUDA cores; mode MODE_SILU: w = [gate; up], out = silu(g) * u; mode MODE_XIELU:
    out = xielu(x . w^T) with the constants ``act`` = (alpha_pos, alpha_neg)."""
    _need(x, "x", torch.float32, 2), _need(w, "w", torch.float32, 2), _need(out, "out", torch.float32, 2)
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N if mode == MODE_SILU else N), K) or out.shape[0] != M:
        raise KernelError(f"sgemm: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not match")
    lib = _lib("gemm.cu")
    _check(lib, lib.dk_sgemm(_p(x), _p(w), _p(out), M, N, K, mode, c_float(act[0]), c_float(act[1]), _stream()), "sgemm")


# ---------------------------------------------------------------------------------------- sampling
def sample_chunks(vocab):
    return _lib("sampling.cu").dk_sample_chunks(vocab)


def sample(logits, temperature, seeds, pos, rows, ws_val, ws_idx, out_tok, advance=False):
    """out_tok[b] = argmax (temperature 0) or Gumbel-max draw of logits[b]. temperature [n]
    float32, seeds [n, 2] int32 (low, high word of each row's 64-bit seed), pos int32 positions
    indexed through ``rows`` (or directly when rows is None); the draw's counter is that position
    + 1, the place the new token will take. ``advance`` moves those positions on by one."""
    _need(logits, "logits", torch.float32, 2), _need(temperature, "temperature", torch.float32, 1)
    _need(seeds, "seeds", torch.int32, 2), _need(pos, "pos", torch.int32, 1), _need(rows, "rows", torch.int32, 1)
    _need(ws_val, "ws_val", torch.float32), _need(ws_idx, "ws_idx", torch.int32), _need(out_tok, "out_tok", torch.int32, 1)
    n, V = logits.shape
    lib = _lib("sampling.cu")
    need = n * lib.dk_sample_chunks(V)
    if ws_val.numel() < need or ws_idx.numel() < need:
        raise KernelError("sample: scratch too small")
    _check(lib, lib.dk_sample(_p(logits), n, V, _p(temperature), _p(seeds), _p(pos), _p(rows), _p(ws_val), _p(ws_idx),
                              _p(out_tok), int(bool(advance)), _stream()), "sample", 2)


# ------------------------------------------------------------------- streaming product (M <= 16)
STREAM_MAX_ROWS = 16
# rows up to which the streaming product is the fastest: with 9 to 16 rows its copy of x doubles and
# the tensor-core product in its decode form wins (measured at 12, 16, 17)
STREAM_BEST_ROWS = 8
_STREAM_SMEM_BLOCK = 227 * 1024              # dynamic shared memory one block may ask for
_STREAM_SMEM_PAIR = (228 * 1024) // 2 - 1024  # ... and what each of two blocks sharing an SM may use


def _stream_smem(rows, K, sk, warps):
    """Shared memory of a block of the streaming product: ``warps`` two-deep rings of 16 weight rows
    x 256 columns, two buffers of the warps' sums, and the rows (8 or 16) of one slice of x. Must
    equal smem_bytes() in gemv_stream.cu."""
    mr = 8 if rows <= 8 else 16
    per = ((K + sk - 1) // sk + 15) // 16 * 16
    return warps * 2 * 16 * (256 * 2 + 16) + 2 * warps * 16 * mr * 4 + mr * (per * 2 + 16)


def stream_plan(M, N, K, mode, allow_partial=False):
    """(slices of K, blocks, streaming warps a block) for gemv_stream, or None if it cannot take
    the shape. Four warps and two persistent blocks per SM while the rows of x leave room for two
    blocks; for a longer K eight warps and one block per SM (as many bytes in flight); beyond that
    K is cut into slices, which needs a caller that takes partial sums (never the SiLU epilogue).
    With partial sums allowed K is cut so that the blocks fill the SMs' shared memory with their
    rings, and further while there are fewer than two tiles per block (more slices cost the
    consumer more partial sums to add)."""
    sms = sm_count()

    def shape(sk):                            # (warps, blocks, whether the SMs' shared memory is full of rings)
        if _stream_smem(M, K, sk, 4) <= _STREAM_SMEM_PAIR:
            return 4, 2 * sms, True
        if _stream_smem(M, K, sk, 8) <= _STREAM_SMEM_BLOCK:
            return 8, sms, True
        if _stream_smem(M, K, sk, 4) <= _STREAM_SMEM_BLOCK:
            return 4, sms, False              # one block of four warps an SM: half the bytes in flight
        return None

    sk = 1
    while shape(sk) is None:
        sk *= 2
        if sk > 64:
            return None
    can_slice = allow_partial and mode not in (MODE_SILU, MODE_XIELU)
    if sk > 1 and not can_slice:
        return None
    if can_slice:
        # two blocks of four warps an SM where up to four slices allow it (what the kernel was tuned on);
        # else the fewest slices that fill the SMs' shared memory at all, rather than half-empty SMs
        pair = next((k for k in (1, 2, 4) if k >= sk and shape(k)[:2] == (4, 2 * sms)), None)
        full = next((k for k in (1, 2, 4, 8) if k >= sk and shape(k)[2]), None)
        sk = pair or full or sk
        tiles = (N + 15) // 16
        while sk < 8 and tiles * sk < 2 * shape(sk)[1] and K // (sk * 2) >= 512 and shape(sk * 2)[2]:
            sk *= 2
    warps, blocks, _ = shape(sk)
    return sk, blocks, warps


def gemv_stream(x, w, out=None, mode=MODE_STORE, plan=None, act=(0.0, 0.0)):
    """The weight-streaming skinny product (asynchronous copies into shared-memory rings,
    tensor-core multiply) for at most 16 rows of x and K a multiple of 16. Returns ``out`` [M, N]
    (bfloat16 for MODE_STORE and MODE_SILU, float32 for MODE_STORE_F32), or, when the plan splits K
    (plan[0] > 1), a ``Partial``."""
    _need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2), _need(out, "out", None, 2)
    M, K = x.shape
    N = w.shape[0] // 2 if mode == MODE_SILU else w.shape[0]
    if M > STREAM_MAX_ROWS or K % 16:
        raise KernelError(f"gemv_stream: {M} rows (max {STREAM_MAX_ROWS}) / inner size {K} (multiple of 16) not supported")
    if w.shape[1] != K:
        raise KernelError(f"gemv_stream: shapes x{tuple(x.shape)} w{tuple(w.shape)} do not match")
    sk, blocks, warps = plan or stream_plan(M, N, K, mode) or (0, 0, 0)
    if sk < 1 or blocks < sk or warps not in (4, 8) or _stream_smem(M, K, sk, warps) > _STREAM_SMEM_BLOCK:
        raise KernelError(f"gemv_stream: K = {K} in {sk} slices on {blocks} blocks of {warps} warps is not supported "
                          f"(the {M} rows of a slice of x must fit a block's shared memory, and there is a block per slice at least)")
    ws = None
    if sk > 1:
        if mode in (MODE_SILU, MODE_XIELU):
            raise KernelError("gemv_stream: an activation in the epilogue cannot be split over K")
        ws = torch.empty((sk, M, N), dtype=torch.float32, device=w.device)
    else:
        want = torch.float32 if mode == MODE_STORE_F32 else torch.bfloat16
        if out is None:
            out = torch.empty((M, N), dtype=want, device=w.device)
        elif out.dtype != want or tuple(out.shape) != (M, N):
            raise KernelError(f"gemv_stream: out {tuple(out.shape)} {out.dtype} does not fit mode {mode}")
    lib = _lib("gemv_stream.cu")
    _check(lib, lib.dk_gemv_stream(_p(x), _p(w), _p(out), _p(ws), M, N, K, mode, sk, blocks, warps, c_float(act[0]),
                                   c_float(act[1]), _stream()), "gemv_stream")
    return Partial(ws) if sk > 1 else out


# ------------------------------------------------------------- tensor-core product for many rows
_tc_err = None


def gemm_tc(x, w, mode=MODE_STORE, out=None, plan=None, act=(0.0, 0.0)):
    """out = x . w^T (mode MODE_STORE, MODE_STORE_F32) or silu(x . gate^T) * (x . up^T) (mode
    MODE_SILU, w = [gate; up]) on tcgen05 tensor cores, TMA-fed, float32 accumulation in tensor
    memory. ``plan`` = (weight rows per tile, one of TC_TILE_HEIGHTS; slices of K): with more than
    one slice (mode MODE_STORE) a ``Partial`` comes back instead of a tensor."""
    global _tc_err
    _need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2), _need(out, "out", None, 2)
    M, K = x.shape
    N = w.shape[0] // 2 if mode == MODE_SILU else w.shape[0]
    bn, sk = plan or (256, 1)
    xielu = mode == MODE_XIELU          # the plain product with the activation on its finished sums
    if xielu:
        mode = MODE_STORE
    if K % 8 or w.shape[1] != K or mode not in (MODE_STORE, MODE_STORE_F32, MODE_SILU) \
            or bn not in TC_TILE_HEIGHTS or (xielu and sk != 1):
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} mode {mode} not supported (K % 8 == 0)")
    kb = (K + 63) // 64
    if sk < 1 or (sk > 1 and (mode != MODE_STORE or (sk - 1) * ((kb + sk - 1) // sk) >= kb)):
        raise KernelError(f"gemm_tc: {sk} slices of K = {K} in mode {mode} not supported")
    ws = None
    if sk > 1:
        ws = torch.empty((sk, M, N), dtype=torch.float32, device=x.device)
    elif mode == MODE_STORE_F32:
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        ws = out
    elif out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    want = torch.float32 if mode == MODE_STORE_F32 else torch.bfloat16
    if sk == 1 and (out.dtype != want or tuple(out.shape) != (M, N)):
        raise KernelError(f"gemm_tc: out {tuple(out.shape)} {out.dtype} does not fit mode {mode}")
    if _tc_err is None:
        _tc_err = torch.zeros(1, dtype=torch.int32, device=x.device)
    lib = _lib("gemm_tc.cu")
    _check(lib, lib.dk_gemm_tc(_p(x), _p(w), _p(None if ws is not None else out), M, N, K,
                               MODE_STORE if mode == MODE_STORE_F32 else mode, _p(_tc_err), sk, _p(ws), bn,
                               (3 if act[0] > 1.5 else 2) if (mode == MODE_SILU and act[0] > 0.5) else int(xielu),
                               c_float(act[1] if (mode == MODE_SILU and act[0] > 1.5) else act[0]), c_float(act[1]), _stream()),
           "gemm_tc")
    return Partial(ws) if sk > 1 else out


TC_QKV_HEAD_DIMS = (64, 128)


def gemm_tc_qkv(x, w, q_out, q_norm_w, k_norm_w, cos, sin, eps, row_pos, row_seq, page_table, k_store, v_store, n_heads,
                n_kv_heads, head_dim, write_kv=True):
    """The fused q/k/v projection x . [Wq; Wk; Wv]^T of a prefill step with ``qk_norm_rope_write``
    in the epilogue of the tensor-core product: the float32 accumulator rows go through the per-head
    norm and the rotation, q to ``q_out``, k and v into the paged cache; the projection itself is
    never written. Head sizes 64 and 128; arguments as ``qk_norm_rope_write``."""
    global _tc_err
    _need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2), _need(q_out, "q_out", torch.bfloat16, 2)
    _need(q_norm_w, "q_norm_w", torch.float32, 1), _need(k_norm_w, "k_norm_w", torch.float32, 1)
    _need(cos, "cos", torch.float32, 2), _need(sin, "sin", torch.float32, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16), _need(v_store, "v_store", torch.bfloat16)
    M, K = x.shape
    if head_dim not in TC_QKV_HEAD_DIMS or K % 8 or tuple(w.shape) != ((n_heads + 2 * n_kv_heads) * head_dim, K) \
            or tuple(q_out.shape) != (M, n_heads * head_dim) or row_pos.numel() < M or row_seq.numel() < M:
        raise KernelError(f"gemm_tc_qkv: x{tuple(x.shape)} w{tuple(w.shape)} heads {n_heads}:{n_kv_heads} of {head_dim} "
                          "not supported (head size 64 or 128, K % 8 == 0)")
    if cos is not None and (cos.shape[1] != head_dim // 2 or sin.shape != cos.shape):
        raise KernelError("gemm_tc_qkv: angle tables must be [positions, head_dim / 2]")
    if _tc_err is None:
        _tc_err = torch.zeros(1, dtype=torch.int32, device=x.device)
    lib = _lib("gemm_tc.cu")
    _check(lib, lib.dk_gemm_tc_qkv(_p(x), _p(w), M, K, _p(_tc_err), _p(q_out), _p(k_store), _p(v_store), _p(q_norm_w),
                                   _p(k_norm_w), _p(cos), _p(sin), _p(row_pos), _p(row_seq), _p(page_table),
                                   page_table.shape[1], n_heads, n_kv_heads, head_dim, c_float(eps), int(bool(write_kv)),
                                   _stream()), "gemm_tc_qkv")


TC_SKINNY_MAX_ROWS = 128


TC_TILE_HEIGHTS = (128, 144, 160, 176, 192, 208, 224, 240, 256)   # weight rows a tile of gemm_tc


def skinny_tc_plan(M, N, K, mode, allow_partial=False):
    """(weight rows per tile, slices of K) for gemm_tc on a decode step of up to 128 rows. A unit of
    work is (tile, slice), with a block of its own while the units fit the SMs; all blocks stream
    at once, so the step takes as long as its largest unit: tile height x blocks of 64 columns in
    a slice (x waves, should the tiles alone exceed the SMs). The plan with the smallest such unit
    wins; among plans within 3 % of it the one with the fewest slices (partial sums are written and
    added up again), then the larger tile. Slices hold at least 8 blocks of 64 columns (fewer
    cannot keep the load ring busy). The gated product has no slices (SiLU needs whole sums)."""
    kb = (K + 63) // 64
    sms = sm_count()
    if mode == MODE_SILU:
        def span(bn):
            tiles = (N + bn // 2 - 1) // (bn // 2)
            return bn * -(-tiles // sms)
        return min(TC_TILE_HEIGHTS, key=lambda bn: (span(bn), bn)), 1
    if mode == MODE_XIELU:        # no slices (the activation needs whole sums): the tile height with the smallest unit
        return min(TC_TILE_HEIGHTS, key=lambda bn: (bn * -(-((N + bn - 1) // bn) // sms), bn)), 1
    if mode != MODE_STORE or not allow_partial:
        return 256, 1
    plans = []
    for bn in TC_TILE_HEIGHTS:
        tiles = (N + bn - 1) // bn
        sk = max(1, min(sms // tiles, kb // 8))
        while sk > 1 and (sk - 1) * ((kb + sk - 1) // sk) >= kb:
            sk -= 1
        waves = -(-tiles * sk // sms)
        plans.append((bn * ((kb + sk - 1) // sk) * waves, sk, bn))
    least = min(p[0] for p in plans)
    _, sk, bn = min((p for p in plans if p[0] <= 1.03 * least), key=lambda p: (p[1], p[0], -p[2]))
    return bn, sk


def gated_tc_plan(M, N):
    """Weight rows per tile for the gated product of a prefill step (gemm_tc, MODE_SILU; N outputs).
    One persistent block an SM works through the tiles in waves, and a step takes waves x what a
    wave of that tile costs. Measured at 512 to 8,192 rows of three model sizes: a wave of 192-row
    tiles costs 0.86 of a wave of 256-row tiles, and lower tiles no less than that (their share of
    the rows of x per output grows), so the choice is between those two: 512 rows of the benchmark
    model are 304 tiles of 256 (3 waves) or 408 of 192 (3 waves at 0.86)."""
    sms = sm_count()
    m_tiles = (M + 127) // 128

    def cost(bn, wave):
        tiles = m_tiles * ((N + bn // 2 - 1) // (bn // 2))
        return -(-tiles // sms) * wave
    return (192 if cost(192, 0.86) < cost(256, 1.0) else 256), 1


def gemm_tc_fills_gpu(M, N, min_fill=0.8):
    """Whether gemm_tc's 128 x 256 output tiles, one persistent block per SM, keep the last wave
    at least ``min_fill`` full on average; below that the library's smaller tiles win."""
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    waves = tiles / sm_count()
    return waves / -(-tiles // sm_count()) >= min_fill


def gemm_tc_check():
    """Raises if a bounded wait inside gemm_tc or attention_prefill_tc ran out since the last check (synchronises)."""
    if _tc_err is not None:
        code = int(_tc_err.item())
        if code:
            _tc_err.zero_()
            for t in _attn_sched.values():
                t.zero_()
            raise KernelError(f"gemm_tc: a bounded wait ran out (code {code}); its results are not valid")


# --------------------------------------------------------------- tensor-core prefill attention
TC_ATTENTION_HEAD_DIMS = (64, 128)
TC_TILE_ROWS = 128
_attn_sched = {}


def attention_prefill_tc(q, out, k_store, v_store, tiles, cu_q, seq_pos0, page_table, n_heads, n_kv_heads, head_dim, window,
                         scale):
    """Ragged causal attention of query chunks on tcgen05 tensor cores (head sizes 64 and 128).
    Arguments as ``attention_prefill_bf16`` except that ``tiles`` lists 128-row tiles."""
    global _tc_err
    _need(q, "q", torch.bfloat16, 2), _need(out, "out", torch.bfloat16, 2), _need(tiles, "tiles", torch.int32, 2)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16, 4)
    if head_dim not in TC_ATTENTION_HEAD_DIMS or n_heads % n_kv_heads:
        raise KernelError(f"attention_prefill_tc: head size {head_dim} (64 or 128) / heads {n_heads}:{n_kv_heads} not supported")
    if _tc_err is None:
        _tc_err = torch.zeros(1, dtype=torch.int32, device=q.device)
    stream = _stream_ptr()
    sched = _attn_sched.get(stream)          # the kernel's work counter: launches of one stream share it, in turn
    if sched is None:
        sched = _attn_sched[stream] = torch.zeros(2, dtype=torch.int32, device=q.device)
    lib = _lib("attention_tc.cu", {"HD": head_dim})
    _check(lib, lib.dk_attn_prefill_tc(_p(q), _p(out), _p(k_store), _p(v_store), c_longlong(q.shape[0]),
                                       c_longlong(k_store.shape[0]), _p(tiles), tiles.shape[0], _p(cu_q), _p(seq_pos0),
                                       _p(page_table), page_table.shape[1], n_heads, n_kv_heads, int(window or 0),
                                       c_float(scale), _p(_tc_err), _p(sched), c_void_p(stream)), "attention_prefill_tc")



# ------------------------------------------------------ embedding with position, stream adds, caps
def _need_rows(t, name, dtype=None):
    """A 2-d CUDA tensor whose rows are contiguous (the rows themselves may lie in a wider matrix)."""
    if t is None:
        return
    if not t.is_cuda or t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be a 2-d CUDA tensor with contiguous rows")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def embed_position_rmsnorm(tok, embed, scale, row_pos, inv_freq, norm_w, eps, h_out, a_out):
    """h_out[t] = embed[tok[t]] * scale + sinusoid(row_pos[t]) (float32; the sinusoid only with
    ``inv_freq``, float64 [H/2]: sine of position * inv_freq[i] at 2i, cosine at 2i+1);
    a_out[t] = rmsnorm(h_out[t]) * norm_w when norm_w is given."""
    _need(tok, "tok", torch.int32, 1), _need(embed, "embed", None, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(row_pos, "row_pos", torch.int32, 1), _need(inv_freq, "inv_freq", torch.float64, 1)
    _need(h_out, "h_out", torch.float32, 2), _need(a_out, "a_out", embed.dtype, 2)
    n, (V, H) = tok.numel(), embed.shape
    if inv_freq is not None and (inv_freq.numel() != H // 2 or row_pos is None or row_pos.numel() < n):
        raise KernelError(f"embed_position_rmsnorm: {inv_freq.numel()} frequencies for width {H}, or positions missing")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_embed_position_rmsnorm(_dt(embed), _p(tok), _p(embed), c_float(scale), _p(row_pos), _p(inv_freq),
                                              _p(norm_w), c_float(eps), n, H, V, _p(h_out), _p(a_out), _stream()),
           "embed_position_rmsnorm")


def stream_add(h, other=None, vec=None):
    """h += other (float32, h's shape) + vec (float32 [H]), whichever is given."""
    _need(h, "h", torch.float32, 2), _need(other, "other", torch.float32, 2), _need(vec, "vec", torch.float32, 1)
    if (other is not None and other.shape != h.shape) or (vec is not None and vec.numel() != h.shape[1]):
        raise KernelError("stream_add: shapes do not match")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_stream_add(_p(h), _p(other), _p(vec), c_longlong(h.shape[0]), h.shape[1], _stream()), "stream_add")


def softcap(x, cap, factor=1.0):
    """x = cap * tanh(factor * x / cap) in place (float32); without a cap (None or 0) x = factor * x."""
    _need(x, "x", torch.float32)
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_softcap(_p(x), c_longlong(x.numel()), c_float(cap or 0.0), c_float(factor), _stream()), "softcap")


def xielu(z, out, alpha_pos, alpha_neg):
    """out = alpha_pos z^2 + z/2 (z > 0), alpha_neg (e^z - 1 - z) + z/2 (z <= 0)."""
    _need(z, "z", None), _need(out, "out", z.dtype)
    if out.shape != z.shape:
        raise KernelError("xielu: shapes do not match")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_xielu(_dt(z), _p(z), _p(out), c_longlong(z.numel()), c_float(alpha_pos), c_float(alpha_neg),
                             _stream()), "xielu")


# ------------------------------------------------------------- attention with mask, bias and sink
def kv_write(k, v, k_store, v_store, row_pos, row_seq, page_table, n_kv_heads, head_dim, v_head_dim):
    """k [T, nkv*hd] and v [T, nkv*hdv] (rows of a wider matrix, one common row stride) into the paged
    stores [pages, nkv, PAGE, hd] / [pages, nkv, PAGE, hdv] at each token's position."""
    _need_rows(k, "k"), _need_rows(v, "v", k.dtype)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", k.dtype), _need(v_store, "v_store", k.dtype)
    if k.stride(0) != v.stride(0) or k.shape[1] != n_kv_heads * head_dim or v.shape[1] != n_kv_heads * v_head_dim:
        raise KernelError("kv_write: k and v must be rows of one matrix, nkv*hd and nkv*hdv wide")
    lib = _lib("attention_masked.cu")
    _check(lib, lib.dk_kv_write(_dt(k), _p(k), _p(v), c_longlong(k.stride(0)), _p(k_store), _p(v_store), _p(row_pos),
                                _p(row_seq), _p(page_table), page_table.shape[1], k.shape[0], n_kv_heads, head_dim,
                                v_head_dim, _stream()), "kv_write")


def attention_masked(q, out, gate, out_scale, k_store, v_store, row_pos, row_seq, page_table, n_heads, n_kv_heads,
                     head_dim, v_head_dim, window, chunk, scale, r1=None, r2=None, sink=None, softcap=None, keep_first=0):
    """Float32-arithmetic attention of every token row over its sequence's cached keys: causal, inside
    the row's chunk (``chunk`` positions, 0: none) and window (0: none); score = q.k * scale
    - r1_h * ln(1 + r2_h * distance) (with r1, r2 float32 [nh]); exp(sink_h) joins the denominator (with
    sink); out = heads * sigmoid(gate) (with gate) * out_scale. ``softcap``: the score (before the bias)
    becomes cap * tanh(score / cap). ``keep_first``: keys at positions below it stay in sight when the window
    has moved on. q, gate and out may be rows of wider matrices. Any phase; float32 or bfloat16 storage."""
    _need_rows(q, "q"), _need_rows(out, "out", q.dtype), _need_rows(gate, "gate", q.dtype)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", q.dtype), _need(v_store, "v_store", q.dtype)
    _need(r1, "r1", torch.float32, 1), _need(r2, "r2", torch.float32, 1), _need(sink, "sink", torch.float32, 1)
    if head_dim > MASKED_MAX_HEAD or v_head_dim > MASKED_MAX_HEAD or n_heads % n_kv_heads or (r1 is None) != (r2 is None):
        raise KernelError(f"attention_masked: head sizes {head_dim}/{v_head_dim} (max {MASKED_MAX_HEAD}), heads {n_heads}:{n_kv_heads}")
    if q.shape[1] != n_heads * head_dim or out.shape[1] != n_heads * v_head_dim or \
            (gate is not None and gate.shape[1] != n_heads * v_head_dim):
        raise KernelError("attention_masked: q, gate or out of the wrong width")
    lib = _lib("attention_masked.cu")
    _check(lib, lib.dk_attention_masked(_dt(q), _p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)),
                                        _p(gate), c_longlong(gate.stride(0) if gate is not None else 0),
                                        c_float(out_scale), _p(k_store), _p(v_store), _p(row_pos), _p(row_seq),
                                        _p(page_table), page_table.shape[1], q.shape[0], n_heads, n_kv_heads, head_dim,
                                        v_head_dim, int(window or 0), int(chunk or 0), c_float(scale), _p(r1), _p(r2),
                                        _p(sink), c_float(softcap or 0.0), int(keep_first or 0), _stream()), "attention_masked")


MASKED_TILE_ROWS = 64            # queries a block of attention_masked_prefill_bf16 takes
_MASKED_DECODE_SMEM = 224 * 1024 - 32 * 1024      # a block's shared memory less the 32 KB where partial sums meet


def _masked_lib(head_dim, v_head_dim):
    if head_dim % 16 or v_head_dim % 16 or not 16 <= head_dim <= 256 or not 16 <= v_head_dim <= 256:
        raise KernelError(f"bfloat16 masked attention: head sizes {head_dim}/{v_head_dim} not supported (multiples of 16 up to 256)")
    return _lib("attention_masked_bf16.cu", {"HD": head_dim, "HDV": v_head_dim})


MASKED_MAX_HEAD = 640      # the float32-arithmetic kernel's largest head (a cached row of latents may be that wide)


def masked_bf16_takes(head_dim, v_head_dim):
    return head_dim % 16 == 0 and v_head_dim % 16 == 0 and 16 <= head_dim <= 256 and 16 <= v_head_dim <= 256


def attention_masked_prefill_bf16(q, out, gate, out_scale, k_store, v_store, tiles, cu_q, seq_pos0, page_table, n_heads,
                                  n_kv_heads, head_dim, v_head_dim, window, chunk, scale, r1=None, r2=None, sink=None):
    """``attention_masked`` for ragged query portions on the tensor cores (bfloat16). tiles [n, 2] int32 =
    (sequence, first query of a 64-row tile within its portion); cu_q [nseq+1]; seq_pos0 [nseq]."""
    _need_rows(q, "q", torch.bfloat16), _need_rows(out, "out", torch.bfloat16), _need_rows(gate, "gate", torch.bfloat16)
    _need(tiles, "tiles", torch.int32, 2), _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16), _need(v_store, "v_store", torch.bfloat16)
    _need(r1, "r1", torch.float32, 1), _need(r2, "r2", torch.float32, 1), _need(sink, "sink", torch.float32, 1)
    if n_heads % n_kv_heads or (r1 is None) != (r2 is None) or q.stride(0) % 2 or out.stride(0) % 2 or \
            (gate is not None and gate.stride(0) % 2):
        raise KernelError("attention_masked_prefill_bf16: head counts or row strides not supported")
    lib = _masked_lib(head_dim, v_head_dim)
    _check(lib, lib.dk_attn_masked_prefill_bf16(_p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), _p(gate),
                                                c_longlong(gate.stride(0) if gate is not None else 0), c_float(out_scale),
                                                _p(k_store), _p(v_store), _p(tiles), tiles.shape[0], _p(cu_q), _p(seq_pos0),
                                                _p(page_table), page_table.shape[1], n_heads, n_kv_heads, int(window or 0),
                                                int(chunk or 0), c_float(scale), _p(r1), _p(r2), _p(sink), _stream()),
           "attention_masked_prefill_bf16")


SHARED_ROWS_MAX_SPLITS = 16


def shared_rows_takes(head_dim, v_head_dim):
    """Whether the kernel for cached rows that are key and value at once is built for these sizes."""
    return head_dim % 16 == 0 and v_head_dim % 32 == 0 and 32 <= v_head_dim <= min(512, head_dim) and head_dim <= 640


def shared_rows_tile_queries(group):
    """Queries of a prompt that one block of ``attention_shared_rows_bf16`` takes: 64 rows = queries x heads of a group."""
    return max(1, 64 // min(group, 64))


def shared_rows_operands(q, out):
    return q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0


def shared_rows_splits(rows, n_heads, n_kv_heads, table_pages, window, chunk):
    """Blocks that share a single token's keys: enough to give every SM one, at least two half pages each."""
    most = min([x for x in (chunk, window, table_pages * PAGE) if x])
    blocks = rows * n_kv_heads * -(-(n_heads // n_kv_heads) // 64)
    return max(1, min(SHARED_ROWS_MAX_SPLITS, sm_count() // blocks, (most // 32 + 2) // 2))


def shared_rows_ws(rows, n_heads, v_head_dim, nsplit, device):
    return (torch.empty(rows * n_heads * nsplit * v_head_dim, dtype=torch.float32, device=device),
            torch.empty(rows * n_heads * nsplit * 2, dtype=torch.float32, device=device))


def attention_shared_rows_bf16(q, out, out_scale, k_store, page_table, n_heads, n_kv_heads, head_dim, v_head_dim, window, chunk,
                               scale, tiles=None, cu_q=None, seq_pos0=None, row_pos=None, nsplit=1, ws=None):
    """Masked softmax attention (bfloat16, mma.sync) whose values are the first ``v_head_dim`` numbers of the cached key
    rows, all query heads of a group in one block. Prompts: ``tiles`` [n, 2] = (sequence, first query of a tile of
    ``shared_rows_tile_queries`` queries), ``cu_q``, ``seq_pos0``. Single tokens: ``row_pos`` [rows] (negative: padding),
    page table row i for row i, the keys of a row in ``nsplit`` runs with ``ws`` = ``shared_rows_ws`` when nsplit > 1."""
    _need_rows(q, "q", torch.bfloat16), _need_rows(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16)
    if not shared_rows_takes(head_dim, v_head_dim) or n_heads % n_kv_heads or not shared_rows_operands(q, out):
        raise KernelError(f"attention_shared_rows_bf16: sizes {head_dim}/{v_head_dim}, head counts or row strides not supported")
    if tiles is not None:
        _need(tiles, "tiles", torch.int32, 2), _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
        n_items, nsplit = tiles.shape[0], 1
    else:
        _need(row_pos, "row_pos", torch.int32, 1)
        n_items = row_pos.shape[0]
        if q.shape[0] != n_items or (nsplit > 1 and (ws is None or ws[0].numel() < n_items * n_heads * nsplit * v_head_dim)):
            raise KernelError("attention_shared_rows_bf16: one query row per position, and scratch for the parts of a split")
    lib = _lib("attention_shared_rows.cu", {"HD": head_dim, "HDV": v_head_dim})
    _check(lib, lib.dk_attn_shared_rows_bf16(_p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), c_float(out_scale),
                                             _p(k_store), _p(tiles), n_items, _p(cu_q), _p(seq_pos0), _p(row_pos), _p(page_table),
                                             page_table.shape[1], n_heads, n_kv_heads, int(window or 0), int(chunk or 0),
                                             c_float(scale), nsplit, _p(ws[0]) if nsplit > 1 else None,
                                             _p(ws[1]) if nsplit > 1 else None, _stream()),
           "attention_shared_rows_bf16", kernels=2 if nsplit > 1 else 1)


def masked_tc_takes(q, out, gate, head_dim, v_head_dim):
    """Whether the tcgen05 prefill attention in its masked build takes these operands: equal head sizes of
    64 or 128, rows a multiple of 8 elements apart and on 16-byte boundaries."""
    if head_dim != v_head_dim or head_dim not in TC_ATTENTION_HEAD_DIMS:
        return False
    return all(t is None or (t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) for t in (q, out, gate))


def attention_masked_prefill_tc(q, out, gate, out_scale, k_store, v_store, tiles, cu_q, seq_pos0, page_table, n_heads,
                                n_kv_heads, head_dim, window, chunk, scale, r1=None, r2=None, sink=None, softcap=None, keep_first=0):
    """``attention_masked`` for ragged query portions on tcgen05 tensor cores (bfloat16, equal head sizes of
    64 or 128): the masked build of ``attention_prefill_tc``'s kernel. ``tiles`` lists 128-row tiles."""
    global _tc_err
    _need_rows(q, "q", torch.bfloat16), _need_rows(out, "out", torch.bfloat16), _need_rows(gate, "gate", torch.bfloat16)
    _need(tiles, "tiles", torch.int32, 2), _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16, 4), _need(v_store, "v_store", torch.bfloat16, 4)
    _need(r1, "r1", torch.float32, 1), _need(r2, "r2", torch.float32, 1), _need(sink, "sink", torch.float32, 1)
    if n_heads % n_kv_heads or (r1 is None) != (r2 is None) or not masked_tc_takes(q, out, gate, head_dim, head_dim) \
            or k_store.shape != v_store.shape:
        raise KernelError("attention_masked_prefill_tc: head sizes, head counts or row strides not supported")
    if _tc_err is None:
        _tc_err = torch.zeros(1, dtype=torch.int32, device=q.device)
    stream = _stream_ptr()
    sched = _attn_sched.get(stream)
    if sched is None:
        sched = _attn_sched[stream] = torch.zeros(2, dtype=torch.int32, device=q.device)
    lib = _lib("attention_tc.cu", {"HD": head_dim, "DK_MASKED": 1})
    _check(lib, lib.dk_attn_prefill_tc_masked(_p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), _p(gate),
                                              c_longlong(gate.stride(0) if gate is not None else 0), c_float(out_scale),
                                              _p(k_store), _p(v_store), c_longlong(q.shape[0]), c_longlong(k_store.shape[0]),
                                              _p(tiles), tiles.shape[0], _p(cu_q), _p(seq_pos0), _p(page_table),
                                              page_table.shape[1], n_heads, n_kv_heads, int(window or 0), int(chunk or 0),
                                              c_float(scale), _p(r1), _p(r2), _p(sink), c_float(softcap or 0.0),
                                              int(keep_first or 0), _p(_tc_err), _p(sched), c_void_p(stream)),
           "attention_masked_prefill_tc")


def masked_decode_streams(q, out, gate, head_dim, v_head_dim):
    """Whether single tokens of a masked attention run on the library's split decode kernel (its masked
    build): keys and values of one head size in steps of 16, rows on 8-byte boundaries."""
    if head_dim != v_head_dim or head_dim % 16 or not 16 <= head_dim <= 256:
        return False
    return all(t is None or (t.stride(0) % 4 == 0 and t.data_ptr() % 8 == 0) for t in (q, out, gate))


def masked_decode_splits(n_seq, n_kv_heads, group, table_pages, window, chunk):
    """Key splits for ``attention_decode_masked_bf16``: those of ``decode_splits`` for the pages a row can see at
    most (its chunk or window bounds them, whatever the page table holds), never more than those pages."""
    pages = table_pages
    for bound in (window, chunk):
        if bound:
            pages = min(pages, bound // PAGE + 2)
    return max(1, min(decode_splits(n_seq, n_kv_heads, group, pages), pages))


def attention_decode_masked_bf16(q, out, gate, out_scale, k_store, v_store, row_pos, page_table, n_heads, n_kv_heads,
                                 head_dim, window, chunk, scale, nsplit, ws_acc, ws_ml, r1=None, r2=None, sink=None,
                                 softcap=None, keep_first=0):
    """``attention_decode_bf16`` in its masked build: one query token per sequence over its cached keys inside
    its chunk and window, with the distance bias in the scores and the sink, the gate and ``out_scale`` in the
    merge. q, gate and out may be rows of wider matrices. Scratch as ``attention_decode_ws``."""
    _need_rows(q, "q", torch.bfloat16), _need_rows(out, "out", torch.bfloat16), _need_rows(gate, "gate", torch.bfloat16)
    _need(row_pos, "row_pos", torch.int32, 1), _need(page_table, "page_table", torch.int32, 2)
    _need(ws_acc, "ws_acc", torch.float32), _need(ws_ml, "ws_ml", torch.float32)
    _need(r1, "r1", torch.float32, 1), _need(r2, "r2", torch.float32, 1), _need(sink, "sink", torch.float32, 1)
    n_seq = q.shape[0]
    if not 1 <= nsplit <= DECODE_MAX_SPLITS or (r1 is None) != (r2 is None) or n_heads % n_kv_heads \
            or not masked_decode_streams(q, out, gate, head_dim, head_dim):
        raise KernelError("attention_decode_masked_bf16: splits, head counts, head size or row strides not supported")
    if ws_acc is None or ws_ml is None or ws_acc.numel() < n_seq * n_heads * 4 * nsplit * head_dim \
            or ws_ml.numel() < n_seq * n_heads * 4 * nsplit * 2:
        raise KernelError("attention_decode_masked_bf16: scratch too small for this batch and split count")
    lib = _lib("attention_bf16.cu", {"HD": head_dim, "DK_MASKED": 1})
    _check(lib, lib.dk_attn_decode_masked_bf16(_p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), _p(gate),
                                               c_longlong(gate.stride(0) if gate is not None else 0), c_float(out_scale),
                                               _p(ws_acc), _p(ws_ml), _p(k_store), _p(v_store), _p(row_pos), _p(page_table),
                                               page_table.shape[1], n_seq, n_heads, n_kv_heads, int(window or 0),
                                               int(chunk or 0), c_float(scale), _p(r1), _p(r2), _p(sink), c_float(softcap or 0.0),
                                               int(keep_first or 0), nsplit, _stream()),
           "attention_decode_masked_bf16", 2)


MASKED_DECODE_MAX_SPLITS = 16


def masked_decode_span(n_heads, n_kv_heads, head_dim, window, chunk, table_pages, rows=None):
    """(most keys a block of a decode step handles, splits of a row's keys over blocks), or None when the
    scores of a kv head's query heads over that many keys do not fit a block's shared memory. A row sees at
    most a chunk, a window, or what the page table can hold; its keys are split so that the blocks fill the
    GPU about twice (fixed by the batch and the sizes, not by the sequences' lengths: a captured step replays
    it), while a split keeps at least 128 keys."""
    most = min([x for x in (chunk, window, table_pages * PAGE) if x])
    g = n_heads // n_kv_heads
    nsplit = 1
    if rows:
        nsplit = max(1, min(MASKED_DECODE_MAX_SPLITS, -(-2 * sm_count() // (rows * n_kv_heads)), most // 128))
    span = -(-most // nsplit)
    while 4 * g * (head_dim + span) > _MASKED_DECODE_SMEM and nsplit < MASKED_DECODE_MAX_SPLITS:
        nsplit += 1
        span = -(-most // nsplit)
    return (span, nsplit) if 4 * g * (head_dim + span) <= _MASKED_DECODE_SMEM else None


def masked_decode_ws(rows, n_heads, v_head_dim, nsplit, device):
    """Scratch of a split attention_masked_decode_bf16: the parts' unnormalised outputs and (maximum, sum) pairs."""
    return (torch.empty(rows * n_heads * nsplit * v_head_dim, dtype=torch.float32, device=device),
            torch.empty(rows * n_heads * nsplit * 2, dtype=torch.float32, device=device))


def attention_masked_decode_bf16(q, out, gate, out_scale, k_store, v_store, row_pos, page_table, n_heads, n_kv_heads,
                                 head_dim, v_head_dim, window, chunk, scale, span, r1=None, r2=None, sink=None,
                                 k_new=None, v_new=None, ws=None):
    """``attention_masked`` for one query token per sequence (bfloat16 storage, float32 arithmetic): a block
    per (kv head, row, run of keys) for all query heads of the group, and a merge kernel when the keys are
    split. ``span`` = (keys a block, splits) from ``masked_decode_span``, ``ws`` from ``masked_decode_ws``. With
    ``k_new`` / ``v_new`` (rows of the step's projection) the kernel writes each token's key and value into
    the cache itself before it reads it."""
    _need_rows(k_new, "k_new", torch.bfloat16), _need_rows(v_new, "v_new", torch.bfloat16)
    if (k_new is None) != (v_new is None) or (k_new is not None and k_new.stride(0) != v_new.stride(0)):
        raise KernelError("attention_masked_decode_bf16: k_new and v_new come together, as rows of one matrix")
    _need_rows(q, "q", torch.bfloat16), _need_rows(out, "out", torch.bfloat16), _need_rows(gate, "gate", torch.bfloat16)
    _need(row_pos, "row_pos", torch.int32, 1), _need(page_table, "page_table", torch.int32, 2)
    _need(k_store, "k_store", torch.bfloat16), _need(v_store, "v_store", torch.bfloat16)
    _need(r1, "r1", torch.float32, 1), _need(r2, "r2", torch.float32, 1), _need(sink, "sink", torch.float32, 1)
    if n_heads % n_kv_heads or (r1 is None) != (r2 is None) or q.stride(0) % 2 or out.stride(0) % 2 or \
            (gate is not None and gate.stride(0) % 2):
        raise KernelError("attention_masked_decode_bf16: head counts or row strides not supported")
    span, nsplit = span
    if nsplit > 1 and (ws is None or ws[0].numel() < q.shape[0] * n_heads * nsplit * v_head_dim
                       or ws[1].numel() < q.shape[0] * n_heads * nsplit * 2):
        raise KernelError("attention_masked_decode_bf16: scratch missing or too small for this batch and split count")
    lib = _masked_lib(head_dim, v_head_dim)
    _check(lib, lib.dk_attn_masked_decode_bf16(_p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), _p(gate),
                                               c_longlong(gate.stride(0) if gate is not None else 0), c_float(out_scale),
                                               _p(k_store), _p(v_store), _p(row_pos), _p(page_table), page_table.shape[1],
                                               q.shape[0], n_heads, n_kv_heads, int(window or 0), int(chunk or 0),
                                               c_float(scale), _p(r1), _p(r2), _p(sink), int(span), _p(k_new), _p(v_new),
                                               c_longlong(k_new.stride(0) if k_new is not None else 0), nsplit,
                                               _p(ws[0] if nsplit > 1 else None), _p(ws[1] if nsplit > 1 else None), _stream()),
           "attention_masked_decode_bf16", 1 if nsplit == 1 else 2)


# ------------------------------------------------------------------------ decayed linear attention
def linear_attention_step(q, k, v, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, n_heads, head_dim, v_head_dim):
    """The recurrence S <- d_h S + silu(k) silu(v)^T, o = S^T silu(q), token by token, for the token rows
    [cu_q[s], cu_q[s+1]) of each sequence (``cu_q`` None: row s alone); state float32
    [slots, nh, hd, hdv] at row seq_slot[s], read and written back; out float32 [T, nh*hdv]. A sequence
    with seq_pos0[s] < 0 is padding (zeros out, state untouched)."""
    _need_rows(q, "q"), _need_rows(k, "k", q.dtype), _need_rows(v, "v", q.dtype)
    _need(out, "out", torch.float32, 2), _need(state, "state", torch.float32, 4), _need(decay, "decay", torch.float32, 1)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1), _need(seq_slot, "seq_slot", torch.int32, 1)
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.shape[1] != n_heads * head_dim or \
            v.shape[1] != n_heads * v_head_dim or tuple(state.shape[1:]) != (n_heads, head_dim, v_head_dim) or \
            decay.numel() != n_heads or head_dim > 256 or v_head_dim > 256:
        raise KernelError("linear_attention_step: shapes do not match (head sizes up to 256)")
    lib = _lib("linear_attention.cu")
    _check(lib, lib.dk_linear_attention_step(_dt(q), _p(q), _p(k), _p(v), c_longlong(q.stride(0)), _p(out), _p(state),
                                             _p(cu_q), _p(seq_pos0), _p(seq_slot), _p(decay), n_seq, n_heads, head_dim,
                                             v_head_dim, _stream()), "linear_attention_step")


CHUNK_MIN_TOKENS = 16     # portions at least this long go to the 64-token-block kernel


def linear_attention(q, k, v, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, n_heads, head_dim, v_head_dim,
                     max_len=None):
    """The recurrence of ``linear_attention_step`` by the kernel that suits the step. ``max_len``: the most
    tokens a sequence brings in this step, if the host knows it (None or 1: single tokens). bfloat16
    portions of ``CHUNK_MIN_TOKENS`` tokens or more run in blocks of 64 tokens on the tensor cores (head sizes
    in steps of 16, keys up to 128, rows on 16-byte boundaries); everything else token by token."""
    if q.dtype == torch.bfloat16 and cu_q is not None and max_len is not None and max_len >= CHUNK_MIN_TOKENS \
            and head_dim % 16 == 0 and head_dim <= 128 and v_head_dim % 16 == 0 and q.stride(0) % 8 == 0 \
            and all(t.data_ptr() % 16 == 0 for t in (q, k, v)):
        return linear_attention_chunk_bf16(q, k, v, out, state, cu_q, seq_slot, decay, n_seq, n_heads, head_dim, v_head_dim)
    return linear_attention_step(q, k, v, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, n_heads, head_dim, v_head_dim)


def linear_attention_chunk_bf16(q, k, v, out, state, cu_q, seq_slot, decay, n_seq, n_heads, head_dim, v_head_dim):
    """``linear_attention_step`` for portions of many tokens in bfloat16: blocks of 64 tokens, the products
    inside a block and with the state on the tensor cores, the state itself in float32. q, k and v are
    overwritten by their activation."""
    _need_rows(q, "q", torch.bfloat16), _need_rows(k, "k", torch.bfloat16), _need_rows(v, "v", torch.bfloat16)
    _need(out, "out", torch.float32, 2), _need(state, "state", torch.float32, 4), _need(decay, "decay", torch.float32, 1)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_slot, "seq_slot", torch.int32, 1)
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.shape[1] != n_heads * head_dim or \
            v.shape[1] != n_heads * v_head_dim or tuple(state.shape[1:]) != (n_heads, head_dim, v_head_dim) or \
            decay.numel() != n_heads or head_dim % 16 or v_head_dim % 16 or not 16 <= head_dim <= 128 or \
            q.stride(0) % 8 or any(t.data_ptr() % 16 for t in (q, k, v)):
        raise KernelError("linear_attention_chunk_bf16: shapes not supported (head sizes in steps of 16, keys up to 128, aligned rows)")
    lib = _lib("linear_attention_bf16.cu", {"HD": head_dim})
    _check(lib, lib.dk_linear_attention_chunk_bf16(_p(q), _p(k), _p(v), c_longlong(q.stride(0)), c_longlong(q.shape[0]), _p(out),
                                                   _p(state), _p(cu_q), _p(seq_slot), _p(decay), n_seq, n_heads, v_head_dim,
                                                   _stream()), "linear_attention_chunk_bf16", 2)


def norm_gate(o, weight, eps, gate, out_scale, out, group=None, gate_act="sigmoid"):
    """out = rmsnorm(o) * weight * sigmoid(gate) * out_scale, the norm over each whole row of o
    (float32 [T, n]), or with ``group`` over each run of that many columns (one head) with a weight of
    that size; ``gate_act`` "silu": gate * sigmoid(gate) instead. gate and out in the storage type,
    possibly rows of wider matrices."""
    _need(o, "o", torch.float32, 2), _need(weight, "weight", torch.float32, 1)
    _need_rows(gate, "gate", out.dtype), _need_rows(out, "out")
    n = o.shape[1]
    group = n if group is None else int(group)
    if group < 1 or n % group or weight.numel() != group or out.shape != o.shape or \
            (gate is not None and gate.shape != o.shape) or gate_act not in ("sigmoid", "silu"):
        raise KernelError("norm_gate: shapes do not match")
    lib = _lib("linear_attention.cu")
    _check(lib, lib.dk_norm_gate(_dt(out), _p(o), _p(weight), c_float(eps), _p(gate),
                                 c_longlong(gate.stride(0) if gate is not None else 0), c_float(out_scale), _p(out),
                                 c_longlong(out.stride(0)), o.shape[0], n, group, int(gate_act == "silu"), _stream()),
           "norm_gate")


def gated_linear_attention_step(q, k, v, out, state, cu_q, seq_pos0, seq_slot, z, z_bias, tau, q_scale, n_seq, n_heads,
                                head_dim, v_head_dim):
    """Gated linear attention token by token: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_scale q_t) with the
    decay of every key channel alpha_t = sigmoid(z_t + z_bias)^(1/tau) (z float32 [T, nh*hd], worked out in
    float32 inside the kernel). Rows, state, padding and ``cu_q`` as in ``linear_attention_step``."""
    _need_rows(q, "q"), _need_rows(k, "k", q.dtype), _need_rows(v, "v", q.dtype)
    _need(out, "out", torch.float32, 2), _need(state, "state", torch.float32, 4)
    _need(z, "z", torch.float32, 2), _need(z_bias, "z_bias", torch.float32, 1)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1), _need(seq_slot, "seq_slot", torch.int32, 1)
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.shape[1] != n_heads * head_dim or \
            v.shape[1] != n_heads * v_head_dim or tuple(state.shape[1:]) != (n_heads, head_dim, v_head_dim) or \
            z.shape != (q.shape[0], n_heads * head_dim) or z_bias.numel() != n_heads * head_dim or \
            head_dim > 256 or v_head_dim > 256 or not tau > 0:
        raise KernelError("gated_linear_attention_step: shapes do not match (head sizes up to 256)")
    lib = _lib("linear_attention.cu")
    _check(lib, lib.dk_gated_linear_attention_step(_dt(q), _p(q), _p(k), _p(v), c_longlong(q.stride(0)), _p(out), _p(state),
                                                   _p(cu_q), _p(seq_pos0), _p(seq_slot), _p(z), _p(z_bias),
                                                   c_float(1.0 / tau), c_float(q_scale), n_seq, n_heads, head_dim,
                                                   v_head_dim, _stream()), "gated_linear_attention_step")


# ------------------------------------------------------------------------ norm after the sum, casts
def scale_add_rmsnorm(h, alpha, delta, norm_w, eps, a_out):
    """h = rmsnorm(alpha * h + delta) * norm_w, written back to the float32 stream, and a_out = the same in
    the storage type. ``delta`` a tensor or a ``Partial``."""
    delta, parts, n_parts, stride = _parts(delta)
    _need(h, "h", torch.float32, 2), _need(delta, "delta", a_out.dtype, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(a_out, "a_out", None, 2)
    if a_out.shape != h.shape or norm_w.numel() != h.shape[1] or (delta is not None and delta.shape != h.shape):
        raise KernelError("scale_add_rmsnorm: shapes do not match")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_scale_add_rmsnorm(_dt(a_out), _p(h), c_float(alpha), _p(delta), parts, n_parts, stride, _p(norm_w),
                                         c_float(eps), h.shape[0], h.shape[1], _p(a_out), _stream()), "scale_add_rmsnorm")


def normed_add_rmsnorm(h, delta, delta_w, delta_eps, norm_w, eps, a_out, rows=None):
    """h += rmsnorm(delta) * delta_w (eps ``delta_eps``); a_out = rmsnorm(h) * norm_w. ``delta`` a tensor or a
    ``Partial``. With ``rows`` (int32 indices) only those rows are worked out, into a_out[0..len(rows)), and h is
    left unchanged."""
    delta, parts, n_parts, stride = _parts(delta)
    _need(h, "h", torch.float32, 2), _need(delta, "delta", a_out.dtype, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(delta_w, "delta_w", torch.float32, 1), _need(rows, "rows", torch.int32, 1), _need(a_out, "a_out", None, 2)
    H = h.shape[1]
    if norm_w.numel() != H or delta_w.numel() != H or (delta is not None and delta.shape != h.shape):
        raise KernelError("normed_add_rmsnorm: shapes do not match")
    n = h.shape[0] if rows is None else rows.numel()
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_normed_add_rmsnorm(_dt(a_out), _p(h), _p(delta), parts, n_parts, stride, _p(rows), _p(delta_w),
                                          c_float(delta_eps), _p(norm_w), c_float(eps), n, H, _p(a_out), _stream()),
           "normed_add_rmsnorm")


def cast_rows(h, a_out):
    """a_out = h (float32) in a_out's type."""
    _need(h, "h", torch.float32, 2), _need(a_out, "a_out", None, 2)
    if a_out.shape != h.shape:
        raise KernelError("cast_rows: shapes do not match")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_cast_rows(_dt(a_out), _p(h), _p(a_out), c_longlong(h.numel()), _stream()), "cast_rows")


ACT_SILU, ACT_GELU_TANH, ACT_CLAMPED = 0, 1, 2


def act_mul(gu, out, act, limit=0.0):
    """out[r, c] = act(gu[r, c]) * gu[r, I + c] for gu [rows, 2I]; act ACT_SILU or ACT_GELU_TANH, or ACT_CLAMPED with
    ``limit``: g' = min(g, limit), u' = clamp(u, -limit, limit), out = g' sigmoid(1.702 g') (u' + 1)."""
    _need(gu, "gu", None, 2), _need(out, "out", gu.dtype, 2)
    if gu.shape != (out.shape[0], 2 * out.shape[1]):
        raise KernelError("act_mul: shapes do not match")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_act_mul(_dt(gu), _p(gu), _p(out), c_longlong(gu.shape[0]), out.shape[1], int(act), c_float(limit),
                               _stream()), "act_mul")


# ------------------------------------------- short convolution, head norm and rotation before a cache
SHORT_CONV_MAX_TAPS = 9


NORM_NONE, NORM_BEFORE_ROTATION, NORM_AFTER_ROTATION = 0, 1, 2


def conv_norm_rope(proj, out, state, w_conv, taps, q_norm_w, k_norm_w, eps, cos, sin, rot_dims, row_pos, row_seq, seq_pos0,
                   seq_slot, n_heads, n_kv_heads, head_dim, v_head_dim, k_store=None, v_store=None, page_table=None,
                   norm_mode=None, v_mix=None, v_src=None, bias=None, q_temp=None, q_split=1):
    """Rows [q | k | v] of a fused projection -> ``out`` rows of the same layout: a causal convolution of
    ``taps`` taps over time on every channel (``w_conv`` [channels, taps]; earlier rows of the same step, or
    the sequence's ``state`` [slots, taps-1, channels] for positions before it), then per q and k head an RMS
    norm with weights of the head's size, then the rotate-half rotation of the first ``rot_dims`` coordinates
    by cos/sin [positions, rot_dims/2]. Each step optional (taps 1, weights None, rot_dims 0). ``norm_mode``: by
    default the norm runs before the rotation when weights are given; ``NORM_AFTER_ROTATION`` puts it behind, and with
    either mode and no weights the heads are divided by their root mean square alone. ``v_src`` (rows of v heads, the
    projection's type) with ``v_mix`` (float32, one number): v <- (1 - v_mix) v + v_mix v_src. The state is
    only read: ``conv_state_update`` moves it on afterwards. ``bias`` (float32 [channels]) is added to the projection
    before the norm; ``q_temp`` = (coef, every) multiplies every q head by 1 + coef * ln(floor((p + 1) / every) + 1) at
    position p, last of all; ``q_split`` = s makes s query heads of each query head (part i of the head at its place in
    head i, zeros elsewhere), so ``out`` is (s - 1) * n_heads * head_dim wider than ``proj``. With ``k_store`` / ``v_store`` [pages, nkv, PAGE, size] and
    ``page_table`` the k and v heads also go to each token's place in the paged cache."""
    _need_rows(proj, "proj"), _need_rows(out, "out", proj.dtype), _need_rows(v_src, "v_src", proj.dtype)
    _need(bias, "bias", torch.float32, 1)
    q_split = int(q_split)
    if q_split < 1 or head_dim % q_split or (q_temp is not None and int(q_temp[1]) < 1):
        raise KernelError(f"conv_norm_rope: q_split {q_split} of heads of {head_dim}, q_temp {q_temp}")
    if norm_mode is None:
        norm_mode = NORM_BEFORE_ROTATION if q_norm_w is not None else NORM_NONE
    if (v_src is None) != (v_mix is None) or (v_src is not None and (v_src.shape != (proj.shape[0], n_kv_heads * v_head_dim)
                                                                     or v_mix.numel() != 1 or v_mix.dtype != torch.float32)):
        raise KernelError("conv_norm_rope: v_src [tokens, nkv * hdv] and v_mix (one float32) come together")
    C = (n_heads + n_kv_heads) * head_dim + n_kv_heads * v_head_dim
    _need(state, "state", proj.dtype, 3), _need(w_conv, "w_conv", proj.dtype, 2)
    _need(q_norm_w, "q_norm_w", torch.float32, 1), _need(k_norm_w, "k_norm_w", torch.float32, 1)
    _need(cos, "cos", torch.float32, 2), _need(sin, "sin", torch.float32, 2)
    for t, n in ((row_pos, "row_pos"), (row_seq, "row_seq"), (seq_pos0, "seq_pos0"), (seq_slot, "seq_slot")):
        _need(t, n, torch.int32, 1)
    if proj.shape[1] != C or out.shape != (proj.shape[0], C + (q_split - 1) * n_heads * head_dim) or \
            (bias is not None and bias.numel() != C) or not 1 <= taps <= SHORT_CONV_MAX_TAPS or \
            (taps > 1 and (state is None or w_conv is None or tuple(state.shape[1:]) != (taps - 1, C) or tuple(w_conv.shape) != (C, taps))) or \
            rot_dims % 2 or rot_dims > head_dim or (rot_dims and (cos is None or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape)) or \
            max(head_dim, v_head_dim) > 256 or (q_norm_w is not None and q_norm_w.numel() != head_dim) or \
            (k_norm_w is not None and k_norm_w.numel() != head_dim):
        raise KernelError("conv_norm_rope: shapes do not match")
    if k_store is not None:
        _need(k_store, "k_store", proj.dtype, 4), _need(v_store, "v_store", proj.dtype, 4), _need(page_table, "page_table", torch.int32, 2)
        if k_store.shape[1:] != (n_kv_heads, PAGE, head_dim) or \
                (v_store is not None and v_store.shape[1:] != (n_kv_heads, PAGE, v_head_dim)):
            raise KernelError("conv_norm_rope: key/value stores of the wrong shape")
    lib = _lib("short_conv.cu")
    _check(lib, lib.dk_conv_norm_rope(_dt(proj), _p(proj), c_longlong(proj.stride(0)), _p(out), c_longlong(out.stride(0)),
                                      _p(state), _p(w_conv), int(taps), int(norm_mode), _p(q_norm_w), _p(k_norm_w),
                                      c_float(eps), _p(v_mix), _p(v_src), c_longlong(v_src.stride(0) if v_src is not None else 0), _p(cos),
                                      _p(sin), int(rot_dims), _p(row_pos), _p(row_seq), _p(seq_pos0), _p(seq_slot),
                                      proj.shape[0], n_heads, n_kv_heads, head_dim, v_head_dim, _p(k_store), _p(v_store),
                                      _p(page_table), page_table.shape[1] if page_table is not None else 0, _p(bias),
                                      c_float(q_temp[0] if q_temp is not None else 0.0),
                                      int(q_temp[1]) if q_temp is not None else 0, q_split, _stream()),
           "conv_norm_rope")


def conv_state_update(proj, state, taps, cu_q, seq_pos0, seq_slot, n_seq):
    """state[slot] <- the last taps-1 rows of each sequence's projection as it stands after this step
    (``cu_q`` None: row s is sequence s with one token; seq_pos0[s] < 0: padding)."""
    _need_rows(proj, "proj"), _need(state, "state", proj.dtype, 3)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1), _need(seq_slot, "seq_slot", torch.int32, 1)
    if tuple(state.shape[1:]) != (taps - 1, proj.shape[1]) or not 2 <= taps <= SHORT_CONV_MAX_TAPS:
        raise KernelError("conv_state_update: shapes do not match")
    lib = _lib("short_conv.cu")
    _check(lib, lib.dk_conv_state_update(_dt(proj), _p(proj), c_longlong(proj.stride(0)), _p(state), int(taps), proj.shape[1],
                                         _p(cu_q), _p(seq_pos0), _p(seq_slot), n_seq, _stream()), "conv_state_update")


# ------------------------------------------------------------------- attention through low-rank latents
def latent_norm_rope_write(proj, cq_out, q_norm_w, kv_norm_w, eps, cos, sin, rot_dims, row_pos, row_seq, q_rank, kv_rank,
                           rot_dim, k_store=None, v_store=None, page_table=None):
    """Rows [a (q_rank) | b (kv_rank) | r (rot_dim)] of a fused down projection: cq_out = rmsnorm(a) * q_norm_w;
    rmsnorm(b) * kv_norm_w and r, its first ``rot_dims`` coordinates rotated by neighbouring pairs (cos/sin
    [positions, rot_dims/2]), go to each token's place in the paged cache of one kv head: key row [c | r]
    (k_store [pages, 1, PAGE, kv_rank + rot_dim]), and, where the cache keeps a store of values, value row c
    (v_store [pages, 1, PAGE, kv_rank] or None)."""
    _need_rows(proj, "proj"), _need_rows(cq_out, "cq_out", proj.dtype)
    _need(q_norm_w, "q_norm_w", torch.float32, 1), _need(kv_norm_w, "kv_norm_w", torch.float32, 1)
    _need(cos, "cos", torch.float32, 2), _need(sin, "sin", torch.float32, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    if proj.shape[1] != q_rank + kv_rank + rot_dim or cq_out.shape != (proj.shape[0], q_rank) or q_norm_w.numel() != q_rank \
            or kv_norm_w.numel() != kv_rank or rot_dims % 2 or rot_dims > rot_dim or \
            (rot_dims and (cos is None or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape)):
        raise KernelError("latent_norm_rope_write: shapes do not match")
    if k_store is not None:
        _need(k_store, "k_store", proj.dtype, 4), _need(v_store, "v_store", proj.dtype, 4), _need(page_table, "page_table", torch.int32, 2)
        if k_store.shape[1:] != (1, PAGE, kv_rank + rot_dim) or (v_store is not None and v_store.shape[1:] != (1, PAGE, kv_rank)):
            raise KernelError("latent_norm_rope_write: key/value stores of the wrong shape")
    lib = _lib("latent.cu")
    _check(lib, lib.dk_latent_norm_rope_write(_dt(proj), _p(proj), c_longlong(proj.stride(0)), _p(cq_out), c_longlong(cq_out.stride(0)),
                                              _p(q_norm_w), _p(kv_norm_w), c_float(eps), _p(cos), _p(sin), int(rot_dims),
                                              _p(row_pos), _p(row_seq), proj.shape[0], q_rank, kv_rank, rot_dim, _p(k_store),
                                              _p(v_store), _p(page_table), page_table.shape[1] if page_table is not None else 0,
                                              _stream()), "latent_norm_rope_write")


def latent_query(q, w_uk, out, cos, sin, rot_dims, row_pos, n_heads, dim, rot_dim, kv_rank, plain=True):
    """q [tokens, heads * (dim + rot_dim)], head by head [plain | rot] -> out [tokens, heads * (kv_rank + rot_dim)],
    head by head [W_uk_h^T plain | rot rotated by neighbouring pairs], with w_uk [heads * dim, kv_rank]. Rows with
    position < 0 become zeros. ``plain=False``: only the rotated parts are written (the plain parts come from a
    product of the caller's)."""
    _need_rows(q, "q"), _need_rows(out, "out", q.dtype), _need(w_uk, "w_uk", q.dtype, 2)
    _need(cos, "cos", torch.float32, 2), _need(sin, "sin", torch.float32, 2), _need(row_pos, "row_pos", torch.int32, 1)
    if q.shape[1] != n_heads * (dim + rot_dim) or out.shape != (q.shape[0], n_heads * (kv_rank + rot_dim)) or \
            tuple(w_uk.shape) != (n_heads * dim, kv_rank) or rot_dims % 2 or rot_dims > rot_dim or \
            (rot_dims and (cos is None or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape)):
        raise KernelError("latent_query: shapes do not match")
    lib = _lib("latent.cu")
    _check(lib, lib.dk_latent_query(_dt(q), _p(q), c_longlong(q.stride(0)), _p(w_uk), _p(out), c_longlong(out.stride(0)), _p(cos),
                                    _p(sin), int(rot_dims), _p(row_pos), q.shape[0], n_heads, dim, rot_dim, kv_rank,
                                    int(bool(plain)), _stream()), "latent_query")


def latent_value(o_lat, w_uv, out, n_heads, kv_rank, vdim):
    """o_lat [tokens, heads * kv_rank] -> out [tokens, heads * vdim]: head h's row times w_uv[h * vdim : (h + 1) * vdim]
    ([heads * vdim, kv_rank])."""
    _need_rows(o_lat, "o_lat"), _need_rows(out, "out", o_lat.dtype), _need(w_uv, "w_uv", o_lat.dtype, 2)
    if o_lat.shape[1] != n_heads * kv_rank or out.shape != (o_lat.shape[0], n_heads * vdim) or \
            tuple(w_uv.shape) != (n_heads * vdim, kv_rank):
        raise KernelError("latent_value: shapes do not match")
    lib = _lib("latent.cu")
    _check(lib, lib.dk_latent_value(_dt(o_lat), _p(o_lat), c_longlong(o_lat.stride(0)), _p(w_uv), _p(out),
                                    c_longlong(out.stride(0)), o_lat.shape[0], n_heads, kv_rank, vdim, _stream()), "latent_value")


# ------------------------------------------------------------------------------ mixture of experts
MOE_MAX_EXPERTS = 256


def moe_route(x, w_router, correction, w_shared_gate, top, groups, keep, scale, idx, wt, shared_gate, scores=None,
              renorm=True):
    """Router of a mixture of experts, float32 arithmetic: s = sigmoid(w_router x); the ``top`` experts with the
    largest s + correction among the ``keep`` best of ``groups`` groups of neighbours (group score: its two
    largest s + correction) -> ``idx`` int32 [T, top]; ``wt`` float32 [T, top] = their s over the sum, times
    ``scale`` (``renorm`` False: the chosen s themselves, times ``scale``; ``correction`` None: the choice goes by s);
    ``shared_gate`` float32 [T] = sigmoid(w_shared_gate . x) when that vector is given. Without a correction and with one
    group the choice goes by the sums w_router x themselves (the same order as their sigmoids, also where two float32
    sigmoids have both reached 1), and ``scores`` then holds those sums. Two kernels: the
    scores (``scores`` float32 [T, E], scratch), then the choice."""
    _need(x, "x", None, 2), _need(w_router, "w_router", torch.float32, 2), _need(correction, "correction", torch.float32, 1)
    _need(w_shared_gate, "w_shared_gate", torch.float32, 1), _need(idx, "idx", torch.int32, 2), _need(wt, "wt", torch.float32, 2)
    _need(shared_gate, "shared_gate", torch.float32, 1)
    T, W = x.shape
    E = w_router.shape[0]
    if w_router.shape[1] != W or idx.shape != (T, top) or wt.shape != (T, top) or E > MOE_MAX_EXPERTS or E % groups or \
            not 1 <= keep <= groups or not 1 <= top <= min(E, 32) or (correction is not None and correction.numel() != E) or \
            (w_shared_gate is not None and (w_shared_gate.numel() != W or shared_gate is None or shared_gate.numel() != T)):
        raise KernelError("moe_route: shapes do not match (up to 256 experts, up to 32 chosen)")
    if scores is None:
        scores = torch.empty((T, E), dtype=torch.float32, device=x.device)
    _need(scores, "scores", torch.float32, 2)
    if scores.shape != (T, E):
        raise KernelError("moe_route: scores must be float32 [tokens, experts]")
    lib = _lib("moe.cu")
    _check(lib, lib.dk_moe_route(_dt(x), _p(x), W, _p(w_router), _p(correction), _p(w_shared_gate), E, int(top), int(groups),
                                 int(keep), c_float(scale), _p(idx), _p(wt), _p(shared_gate), _p(scores), T, int(bool(renorm)),
                                 _stream()),
           "moe_route", 2)


def moe_up_rows(x, w_gate_up, idx, mid, act=0, in_wt=None, limit=0.0):
    """mid[t * top + j] = act(gate_e x_t) * (up_e x_t) for e = idx[t, j]; w_gate_up [E, 2 ff, W] with an expert's
    gate rows before its up rows. A warp per output, float32 sums. ``in_wt`` float32 [T, top]: the pair's weight on the
    expert's input (both sums times it before the activation). ``act`` ACT_CLAMPED with ``limit``: g' = min(g, limit),
    u' = clamp(u, -limit, limit), out = g' sigmoid(1.702 g') (u' + 1)."""
    _need(in_wt, "in_wt", torch.float32, 2)
    _need(x, "x", None, 2), _need(w_gate_up, "w_gate_up", x.dtype, 3), _need(idx, "idx", torch.int32, 2), _need(mid, "mid", x.dtype, 2)
    T, W = x.shape
    top, ff = idx.shape[1], mid.shape[1]
    if w_gate_up.shape[1:] != (2 * ff, W) or mid.shape[0] != T * top or idx.shape[0] != T:
        raise KernelError("moe_up_rows: shapes do not match")
    lib = _lib("moe.cu")
    _check(lib, lib.dk_moe_up_rows(_dt(x), _p(x), W, _p(w_gate_up), _p(idx), _p(mid), ff, top, T, int(act), _p(in_wt),
                                   c_float(limit), _stream()), "moe_up_rows")


def moe_down_rows(mid, w_down, idx, wt, shared, shared_gate, out):
    """out[t] = sum_j wt[t, j] * down_e mid[t * top + j] (e = idx[t, j]) + shared_gate[t] * shared[t]; w_down
    [E, W, ff]; ``shared`` [T, W] and its gate optional."""
    _need(mid, "mid", None, 2), _need(w_down, "w_down", mid.dtype, 3), _need(idx, "idx", torch.int32, 2)
    _need(wt, "wt", torch.float32, 2), _need(shared, "shared", mid.dtype, 2), _need(shared_gate, "shared_gate", torch.float32, 1)
    _need(out, "out", mid.dtype, 2)
    T, top = idx.shape
    W, ff = w_down.shape[1:]
    if mid.shape != (T * top, ff) or out.shape != (T, W) or (wt is not None and wt.shape != (T, top)) or (shared is not None and shared.shape != (T, W)):
        raise KernelError("moe_down_rows: shapes do not match")
    lib = _lib("moe.cu")
    _check(lib, lib.dk_moe_down_rows(_dt(mid), _p(mid), _p(w_down), _p(idx), _p(wt), _p(shared), _p(shared_gate), _p(out), W, ff,
                                     top, T, _stream()), "moe_down_rows")


MOE_TILE_ROWS = 64


def moe_tiles_take(x, expert_ff):
    """Whether a step's routed experts run as tiles on the tensor cores: bfloat16, more than 32 tokens, inner
    sizes (width and expert size) that are multiples of 32."""
    return x.dtype == torch.bfloat16 and x.shape[0] > 32 and x.shape[1] % 32 == 0 and expert_ff % 32 == 0


def moe_experts_tiles(x, w_gate_up, w_down, idx, wt, shared, shared_gate, out, act=0, scratch=None, in_wt=None, limit=0.0):
    """The routed experts for many tokens: pairs sorted by expert on the device, tiles of 64 pairs as matrix
    products on mma.sync tensor cores (gate/up with the activation, then down), then the weighted sum per token
    plus shared_gate * shared. ``scratch(key, make)``: where buffers that outlive the call may be kept. ``wt`` None: the
    plain sum; ``in_wt``, ``limit``: as in ``moe_up_rows``."""
    _need(in_wt, "in_wt", torch.float32, 2)
    _need(x, "x", torch.bfloat16, 2), _need(w_gate_up, "w_gate_up", torch.bfloat16, 3), _need(w_down, "w_down", torch.bfloat16, 3)
    _need(idx, "idx", torch.int32, 2), _need(wt, "wt", torch.float32, 2), _need(shared, "shared", torch.bfloat16, 2)
    _need(shared_gate, "shared_gate", torch.float32, 1), _need(out, "out", torch.bfloat16, 2)
    T, W = x.shape
    top = idx.shape[1]
    E, ff = w_down.shape[0], w_down.shape[2]
    if w_gate_up.shape != (E, 2 * ff, W) or w_down.shape[1] != W or idx.shape[0] != T or \
            any(w is not None and w.shape != idx.shape for w in (wt, in_wt)) or \
            out.shape != (T, W) or W % 32 or ff % 32 or E > MOE_MAX_EXPERTS or (shared is not None and shared.shape != (T, W)):
        raise KernelError("moe_experts_tiles: shapes do not match (inner sizes in steps of 32)")
    P = T * top
    max_tiles = (P + MOE_TILE_ROWS - 1) // MOE_TILE_ROWS + E
    dev = x.device

    def make():
        return (torch.empty(P, dtype=torch.int32, device=dev), torch.empty(P, dtype=torch.int32, device=dev),
                torch.empty((max_tiles, 3), dtype=torch.int32, device=dev), torch.empty((P, ff), dtype=torch.bfloat16, device=dev),
                torch.empty((P, W), dtype=torch.bfloat16, device=dev))
    perm, inv, tiles, mid, y = scratch(("moe_tiles", T, top, E, ff, W), make) if scratch is not None else make()
    lib = _lib("moe_tiles.cu")
    _check(lib, lib.dk_moe_sort(_p(idx), P, E, _p(perm), _p(inv), _p(tiles), max_tiles, _stream()), "moe_sort")
    _check(lib, lib.dk_moe_up_tiles(_p(x), _p(w_gate_up), _p(tiles), max_tiles, _p(perm), top, _p(mid), ff, W, int(act), _p(in_wt),
                                    c_float(limit), _stream()), "moe_up_tiles")
    _check(lib, lib.dk_moe_down_tiles(_p(mid), _p(w_down), _p(tiles), max_tiles, _p(y), W, ff, _stream()), "moe_down_tiles")
    _check(lib, lib.dk_moe_sum(_p(y), _p(inv), _p(wt), _p(shared), _p(shared_gate), _p(out), T, W, top, _stream()), "moe_sum")


def gated_linear_attention_takes_warps(head_dim, v_head_dim):
    """Head sizes of the warp form of gated linear attention: keys of 32, 64, 128 or 256, values in steps of 8."""
    return head_dim in (32, 64, 128, 256) and v_head_dim % 8 == 0 and v_head_dim <= 256


def gated_linear_attention(q, k, v, out, state, cu_q, seq_pos0, seq_slot, z, z_bias, tau, q_scale, n_seq, n_heads, head_dim,
                           v_head_dim):
    """``gated_linear_attention_step`` by the kernel that suits the head sizes: a warp per 8 value columns with
    the state in registers (after a kernel that turns ``z`` into the decays, in place) where
    ``gated_linear_attention_takes_warps``, else the block form. Either runs the recurrence token by token in
    float32, for prompts, portions and single tokens alike."""
    if not gated_linear_attention_takes_warps(head_dim, v_head_dim):
        return gated_linear_attention_step(q, k, v, out, state, cu_q, seq_pos0, seq_slot, z, z_bias, tau, q_scale, n_seq, n_heads,
                                           head_dim, v_head_dim)
    _need_rows(q, "q"), _need_rows(k, "k", q.dtype), _need_rows(v, "v", q.dtype)
    _need(out, "out", torch.float32, 2), _need(state, "state", torch.float32, 4)
    _need(z, "z", torch.float32, 2), _need(z_bias, "z_bias", torch.float32, 1)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1), _need(seq_slot, "seq_slot", torch.int32, 1)
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.shape[1] != n_heads * head_dim or \
            v.shape[1] != n_heads * v_head_dim or tuple(state.shape[1:]) != (n_heads, head_dim, v_head_dim) or \
            z.shape != (q.shape[0], n_heads * head_dim) or z_bias.numel() != n_heads * head_dim or not tau > 0 or \
            out.shape != (q.shape[0], n_heads * v_head_dim):
        raise KernelError("gated_linear_attention: shapes do not match")
    lib = _lib("linear_attention.cu")
    _check(lib, lib.dk_gated_linear_attention_warp(_dt(q), _p(q), _p(k), _p(v), c_longlong(q.stride(0)), _p(z), _p(z_bias),
                                                   c_float(1.0 / tau), c_longlong(q.shape[0]), _p(out), _p(state), _p(cu_q),
                                                   _p(seq_pos0), _p(seq_slot), c_float(q_scale), n_seq, n_heads, head_dim,
                                                   v_head_dim, _stream()), "gated_linear_attention", 2)


# ----------------------------------------------------------------- norms over parts of a row, and what ends in one
def add_group_rmsnorm(h, delta, norm_w, eps, groups, a_out, rows=None):
    """h += delta (a tensor, a ``Partial`` or None); a_out = norm_w * (each of ``groups`` equal consecutive parts of
    the row over its own root mean square, eps inside the root). With ``rows`` (int32 indices) only those rows, into
    a_out[0..len(rows)), and h is left as it is."""
    delta, parts, n_parts, stride = _parts(delta)
    _need(h, "h", torch.float32, 2), _need(delta, "delta", a_out.dtype, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(rows, "rows", torch.int32, 1), _need(a_out, "a_out", None, 2)
    H = h.shape[1]
    if groups < 1 or H % groups or norm_w.numel() != H or (delta is not None and delta.shape != h.shape):
        raise KernelError(f"add_group_rmsnorm: {groups} parts of rows of {H}, or shapes that do not match")
    n = h.shape[0] if rows is None else rows.numel()
    lib = _lib("group_norm.cu")
    _check(lib, lib.dk_add_group_rmsnorm(_dt(a_out), _p(h), _p(delta), parts, n_parts, stride, _p(rows), _p(norm_w),
                                         c_float(eps), n, H, int(groups), _p(a_out), _stream()), "add_group_rmsnorm")


def gate_group_norm(o, x, skip, z, weight, eps, groups, out_scale, out):
    """out = weight * grouped_rmsnorm((o + skip_h * x) * silu(z)) * out_scale: o and x float32 [T, n] (x rows of a wider matrix) with n = heads *
    value size, ``skip`` float32 [heads] (None: no such term), the gate rows ``z`` and ``out`` in the storage type (rows
    of wider matrices), the norm over each of ``groups`` equal parts of the row."""
    _need(o, "o", torch.float32, 2), _need_rows(x, "x", torch.float32), _need(skip, "skip", torch.float32, 1)
    _need(weight, "weight", torch.float32, 1), _need_rows(z, "z", out.dtype), _need_rows(out, "out")
    T, n = o.shape
    heads = skip.numel() if skip is not None else 1
    if x.shape != o.shape or z.shape != o.shape or out.shape != o.shape or weight.numel() != n or groups < 1 or n % groups \
            or n % heads:
        raise KernelError("gate_group_norm: shapes do not match")
    lib = _lib("group_norm.cu")
    _check(lib, lib.dk_gate_group_norm(_dt(out), _p(o), _p(x), c_longlong(x.stride(0)), _p(skip), n // heads, _p(z), c_longlong(z.stride(0)),
                                       _p(weight),
                                       c_float(eps), c_float(out_scale), _p(out), c_longlong(out.stride(0)), T, n, int(groups),
                                       _stream()), "gate_group_norm")


def diff_combine(a, lam, eps, out_scale, out, n_heads, v_head_dim):
    """``a`` [T, 2 * n_heads * v_head_dim]: head 2h holds the first map's output of head h, head 2h + 1 the second's.
    out[t, h] = unit_rms(a1 - lam * a2) * out_scale per head (eps inside the root, no weight)."""
    _need_rows(a, "a"), _need_rows(out, "out", a.dtype)
    if a.shape[1] != 2 * n_heads * v_head_dim or out.shape != (a.shape[0], n_heads * v_head_dim) or v_head_dim > 256:
        raise KernelError("diff_combine: shapes do not match (value heads up to 256)")
    lib = _lib("group_norm.cu")
    _check(lib, lib.dk_diff_combine(_dt(a), _p(a), c_longlong(a.stride(0)), c_float(lam), c_float(eps), c_float(out_scale),
                                    _p(out), c_longlong(out.stride(0)), a.shape[0], n_heads, v_head_dim, _stream()), "diff_combine")


# ------------------------------------------------------------- recurrences over a float32 state, and what feeds them
def recurrence_operands(rows, n_qk, n_v, device):
    """One float32 matrix whose column ranges are the recurrence's q, k (n_qk wide) and v (n_v wide), so that the three
    share a row stride, and the dense decays: -> (q, k, v, decay)."""
    buf = torch.empty((rows, 2 * n_qk + n_v), dtype=torch.float32, device=device)
    return buf[:, :n_qk], buf[:, n_qk:2 * n_qk], buf[:, 2 * n_qk:], torch.empty((rows, n_qk), dtype=torch.float32, device=device)


def _need_operands(q, k, v, decay, what):
    for t, nm in ((q, "q"), (k, "k"), (v, "v")):
        _need_rows(t, nm, torch.float32)
    _need(decay, "decay", torch.float32, 2)
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or k.shape != q.shape or decay.shape != q.shape or v.shape[0] != q.shape[0]:
        raise KernelError(f"{what}: q, k, v must be column ranges of one float32 matrix, the decays dense and as wide as q")


def hgrn2_prepare(proj, f_bias, lower, q32, k32, a32, v32):
    """Rows [q | f | v] of a projection (n, n and nv wide) -> float32 q32 = silu(q), a32 = l + (1 - l) sigmoid(f + b),
    k32 = 1 - a32, v32 = v (operands from ``recurrence_operands``)."""
    _need_rows(proj, "proj"), _need(f_bias, "f_bias", torch.float32, 1), _need(lower, "lower", torch.float32, 1)
    _need_operands(q32, k32, v32, a32, "hgrn2_prepare")
    T, n, nv = proj.shape[0], q32.shape[1], v32.shape[1]
    if proj.shape[1] != 2 * n + nv or f_bias.numel() != n or lower.numel() != n or q32.shape[0] != T:
        raise KernelError("hgrn2_prepare: shapes do not match")
    lib = _lib("recurrence.cu")
    _check(lib, lib.dk_hgrn2_prepare(_dt(proj), _p(proj), c_longlong(proj.stride(0)), _p(f_bias), _p(lower), _p(q32), _p(k32),
                                     _p(a32), _p(v32), c_longlong(q32.stride(0)), T, n, nv, _stream()), "hgrn2_prepare")


def ssd_prepare(xbc, dt, state, w_conv, conv_bias, taps, dt_bias, a_log, row_pos, row_seq, seq_pos0, seq_slot, groups, q32, k32, a32, v32):
    """``xbc`` [T, inner + 2 groups N] = [x | B | C] and ``dt`` [T, heads]: columns of one projection (one row stride).
    y = silu(conv(xbc) + bias) with ``w_conv`` [C, taps] whose last column is the current token's and the sequence's
    ``state`` [slots, taps - 1, C] for positions before the step (read only: ``conv_state_update`` moves it on);
    dt <- softplus(dt + dt_bias). Out, head by head (head h of group g): q32 = C_g, k32 = dt_h B_g, a32 = exp(-exp(a_log_h)
    dt_h) on every channel, v32 = x (operands from ``recurrence_operands``)."""
    _need_rows(xbc, "xbc"), _need_rows(dt, "dt", xbc.dtype), _need(state, "state", xbc.dtype, 3), _need(w_conv, "w_conv", xbc.dtype, 2)
    _need(conv_bias, "conv_bias", torch.float32, 1), _need(dt_bias, "dt_bias", torch.float32, 1), _need(a_log, "a_log", torch.float32, 1)
    for t, nm in ((row_pos, "row_pos"), (row_seq, "row_seq"), (seq_pos0, "seq_pos0"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32, 1)
    _need_operands(q32, k32, v32, a32, "ssd_prepare")
    T, C = xbc.shape
    nh, inner = dt.shape[1], v32.shape[1]
    nbc = (C - inner) // 2
    if xbc.stride(0) != dt.stride(0) or tuple(w_conv.shape) != (C, taps) or not 1 <= taps <= SHORT_CONV_MAX_TAPS or \
            (taps > 1 and (state is None or tuple(state.shape[1:]) != (taps - 1, C))) or dt_bias.numel() != nh or a_log.numel() != nh or \
            inner + 2 * nbc != C or groups < 1 or nh % groups or nbc % groups or q32.shape != (T, nh * (nbc // groups)) or \
            (conv_bias is not None and conv_bias.numel() != C):
        raise KernelError("ssd_prepare: shapes do not match")
    lib = _lib("recurrence.cu")
    _check(lib, lib.dk_ssd_prepare(_dt(xbc), _p(xbc), _p(dt), c_longlong(xbc.stride(0)), _p(state), _p(w_conv), _p(conv_bias), int(taps),
                                   _p(dt_bias), _p(a_log), _p(row_pos), _p(row_seq), _p(seq_pos0), _p(seq_slot), _p(q32), _p(k32),
                                   _p(a32), _p(v32), c_longlong(q32.stride(0)), T, inner, nbc, nh, int(groups), _stream()), "ssd_prepare")


def recurrence(q, k, decay, v, out, state, cu_q, seq_pos0, seq_slot, n_seq, n_heads, head_dim, v_head_dim):
    """S <- diag(decay_t) S + k_t v_t^T, o_t = S^T q_t per (sequence, head), token by token, all float32: q, k, decay
    [T, n_heads * head_dim], v and out [T, n_heads * v_head_dim], state [slots, n_heads, head_dim, v_head_dim] (operands
    from ``recurrence_operands``). Rows of sequence s are cu_q[s] .. cu_q[s + 1] (``cu_q`` None: row s alone);
    seq_pos0[s] < 0 marks a padding row. Portions of key sizes 32, 64, 128 and 256 with value sizes in steps of 8 run on
    the staged warp kernel of gated linear attention (rows ahead by cp.async), everything else (single tokens, other
    sizes) on a kernel that keeps a warp's part of the state in registers and asks for the next token's rows a token ahead."""
    _need_operands(q, k, v, decay, "recurrence")
    _need(out, "out", torch.float32, 2), _need(state, "state", torch.float32, 4)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1), _need(seq_slot, "seq_slot", torch.int32, 1)
    T = q.shape[0]
    if q.shape[1] != n_heads * head_dim or v.shape != (T, n_heads * v_head_dim) or out.shape != v.shape or head_dim > 256 or \
            tuple(state.shape[1:]) != (n_heads, head_dim, v_head_dim):
        raise KernelError("recurrence: shapes do not match (key sizes up to 256)")
    if cu_q is not None and gated_linear_attention_takes_warps(head_dim, v_head_dim):
        lib = _lib("linear_attention.cu")
        _check(lib, lib.dk_decayed_recurrence_warp(0, _p(q), _p(k), _p(v), c_longlong(q.stride(0)), _p(decay), c_longlong(T), _p(out),
                                                   _p(state), _p(cu_q), _p(seq_pos0), _p(seq_slot), n_seq, n_heads, head_dim,
                                                   v_head_dim, _stream()), "recurrence")
        return
    lib = _lib("recurrence.cu")
    _check(lib, lib.dk_recurrence(_p(q), _p(k), _p(v), c_longlong(q.stride(0)), _p(decay), _p(out), _p(state), _p(cu_q), _p(seq_pos0),
                                  _p(seq_slot), n_seq, n_heads, head_dim, v_head_dim, _stream()), "recurrence")


# ------------------------------------------------------------------ attention whose heads' scores are mixed
TALK_MAX_HEADS = 64
TALK_MAX_OUT = 16 * 256     # n_heads * v_head_dim a block of attention_talk holds


def attention_talk(q, out, out_scale, k_store, v_store, row_pos, row_seq, page_table, n_heads, n_kv_heads, head_dim, v_head_dim,
                   window, scale, talk):
    """Float32-arithmetic attention of every token row over its sequence's cached keys in which the heads' scores are
    mixed before the softmax: s'_h = sum_g talk[h, g] (q_g . k) * scale; causal, inside ``window`` (0 or None: none);
    out = heads * out_scale. q and out may be rows of wider matrices. Any phase; float32 or bfloat16 storage."""
    _need_rows(q, "q"), _need_rows(out, "out", q.dtype), _need(talk, "talk", torch.float32, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", q.dtype), _need(v_store, "v_store", q.dtype)
    if n_heads > TALK_MAX_HEADS or n_heads % n_kv_heads or n_heads * v_head_dim > TALK_MAX_OUT or tuple(talk.shape) != (n_heads, n_heads) \
            or q.shape[1] != n_heads * head_dim or out.shape != (q.shape[0], n_heads * v_head_dim):
        raise KernelError(f"attention_talk: {n_heads}:{n_kv_heads} heads of {head_dim}/{v_head_dim} (up to {TALK_MAX_HEADS} heads, "
                          f"heads x value size up to {TALK_MAX_OUT})")
    lib = _lib("attention_talk.cu")
    _check(lib, lib.dk_attention_talk(_dt(q), _p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), c_float(out_scale),
                                      _p(k_store), _p(v_store), _p(row_pos), _p(row_seq), _p(page_table), page_table.shape[1],
                                      q.shape[0], n_heads, n_kv_heads, head_dim, v_head_dim, int(window or 0), c_float(scale),
                                      _p(talk), _stream()), "attention_talk")


TALK_TILE_ROWS = 16           # queries a block of attention_talk_bf16 takes
TALK_MAX_SPLITS = 16
_TALK_SMEM = 220 * 1024


def _talk_lib(head_dim, v_head_dim):
    return _lib("attention_talk_bf16.cu", {"HD": head_dim, "HDV": v_head_dim})


def talk_bf16_takes(n_heads, n_kv_heads, head_dim, v_head_dim):
    """Whether the tensor-core form of attention with mixed head scores takes these sizes: key and value sizes in steps
    of 16 up to 256, and a run of 32 keys and values of every kv head beside the heads' score tiles in shared memory."""
    if head_dim % 16 or v_head_dim % 16 or max(head_dim, v_head_dim) > 256 or n_heads > TALK_MAX_HEADS:
        return False
    smem = 2 * n_kv_heads * 32 * (head_dim + 8 + v_head_dim + 8) + 4 * (n_heads * 16 * 40 + n_heads * n_heads)
    return smem <= _TALK_SMEM


def talk_operands(q, out):
    """Rows the tensor-core kernel can read and write two numbers at a time."""
    return all(t.stride(0) % 2 == 0 and t.data_ptr() % 4 == 0 for t in (q, out))


def talk_decode_splits(rows, n_heads, table_pages, window):
    """Runs of keys a single-token step of attention_talk_bf16 deals out over blocks (one block an SM at a time): the count
    that makes waves of blocks times runs a block smallest, no more than there are runs of 32 keys in sight; a function of
    the step's shape alone (a captured graph keeps it)."""
    keys = table_pages * PAGE if not window else min(window + 32, table_pages * PAGE)
    runs = max(1, (keys + 31) // 32)
    blocks = rows * ((n_heads + 15) // 16)
    sms = sm_count()
    best, best_cost = 1, None
    for ns in range(1, min(TALK_MAX_SPLITS, runs) + 1):
        cost = -(-blocks * ns // sms) * (-(-runs // ns) + 0.5)       # a block's start and its part of the merge count as half a run
        if best_cost is None or cost < best_cost:
            best, best_cost = ns, cost
    return best


def talk_decode_ws(rows, n_heads, v_head_dim, nsplit, device):
    return (torch.empty((rows, n_heads, nsplit, v_head_dim), dtype=torch.float32, device=device),
            torch.empty((rows, n_heads, nsplit, 2), dtype=torch.float32, device=device))


def attention_talk_bf16(q, out, out_scale, k_store, v_store, page_table, n_heads, n_kv_heads, head_dim, v_head_dim, window, scale, talk,
                        tiles=None, cu_q=None, seq_pos0=None, row_pos=None, nsplit=1, ws=None):
    """``attention_talk`` on mma.sync tensor cores, bfloat16. Prompts and portions: ``tiles`` (the ``QueryTiles(16)`` plan), ``cu_q``,
    ``seq_pos0``. Single tokens: ``row_pos`` (row r is sequence r, -1: padding), the keys in ``nsplit`` runs with ``ws`` from
    ``talk_decode_ws`` when nsplit > 1."""
    _need_rows(q, "q", torch.bfloat16), _need_rows(out, "out", torch.bfloat16), _need(talk, "talk", torch.float32, 2)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16), _need(v_store, "v_store", torch.bfloat16)
    _need(tiles, "tiles", torch.int32), _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(row_pos, "row_pos", torch.int32, 1)
    if not talk_bf16_takes(n_heads, n_kv_heads, head_dim, v_head_dim) or n_heads % n_kv_heads or tuple(talk.shape) != (n_heads, n_heads) or \
            q.shape[1] != n_heads * head_dim or out.shape != (q.shape[0], n_heads * v_head_dim) or not talk_operands(q, out) or \
            (tiles is None) == (row_pos is None) or (tiles is not None and (cu_q is None or seq_pos0 is None or nsplit != 1)) or \
            (nsplit > 1 and (ws is None or ws[0].shape != (q.shape[0], n_heads, nsplit, v_head_dim))):
        raise KernelError("attention_talk_bf16: sizes or operands the kernel does not take")
    n_tiles = tiles.numel() // 2 if tiles is not None else q.shape[0]
    lib = _talk_lib(head_dim, v_head_dim)
    _check(lib, lib.dk_attention_talk_bf16(_p(q), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), c_float(out_scale),
                                           _p(k_store), _p(v_store), _p(tiles), n_tiles, _p(cu_q), _p(seq_pos0), _p(row_pos),
                                           _p(page_table), page_table.shape[1], n_heads, n_kv_heads, int(window or 0), c_float(scale),
                                           _p(talk), int(nsplit), _p(ws[0]) if ws is not None else c_void_p(0),
                                           _p(ws[1]) if ws is not None else c_void_p(0), _stream()),
           "attention_talk_bf16", 2 if nsplit > 1 else 1)
