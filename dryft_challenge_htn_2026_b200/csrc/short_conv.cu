// What stands between an attention mixer's fused projection and its cache, for mixers that ask for it:
//   * a short causal convolution over time on every channel of q, k and v,
//       y_t[c] = sum_j w[c][j] * u_(t - taps + 1 + j)[c],   zeros before the sequence's start,
//     whose memory, the last taps - 1 projected rows of each sequence, is a per-sequence state
//     [slots, taps - 1, channels] (zero when a slot is taken, so that the zeros come by themselves);
//   * an RMS norm over each query and key head, with a weight of the head's size or without one, before the
//     rotation (norm_mode 1) or after it (norm_mode 2),
//   * a rotate-half rotation of the first rot_dims coordinates of each query and key head (coordinate i
//     with i + rot_dims / 2) by angles from a table [positions, rot_dims / 2]; the rest pass,
//   * values blended with another layer's values of the same token: v <- (1 - lam) v + lam v_src, lam a
//     learned number on the device.
//   * a bias per channel of q, k and v (float32 [channels]), added to the projection (behind the convolution,
//     before the norm),
//   * a query temperature: every q head times 1 + coef * ln(floor((p + 1) / every) + 1) at position p (last of all),
//   * query heads split into q_split equal parts: each part becomes a query head of the full size of its own
//     that holds the part at its place and zeros elsewhere (out then has q_split * nh query heads), so that a
//     key row made of q_split maps side by side is scored one map at a time by ordinary attention.
// Each option may be left out (taps = 1, norm_mode 0, rot_dims = 0, no v_src, no bias, every = 0, q_split = 1). The result is a dense row
// [q heads | k heads | v heads] in the storage type; sums, norms and the rotation are float32. Given the paged
// key and value stores, the kernel also writes each token's k and v heads to their place there (the step's cache write).
// A second kernel moves the state on once the first has read it.
#include "common.cuh"

#define SC_THREADS 128
#define SC_MAX_TAPS 9

__device__ __forceinline__ float query_temperature(int pos, float coef, int every) {
    return 1.f + coef * logf((float)((pos + 1) / every) + 1.f);
}
// coordinate d of a query head of size hd into its part's head (of the parts heads that stand for it), zeros into the others
template <typename T>
__device__ __forceinline__ void write_split(T* heads, int d, int hd, int parts, T value) {
    const int part = d / (hd / parts);
    for (int m = 0; m < parts; m++) heads[(size_t)m * hd + d] = m == part ? value : from_f<T>(0.f);
}

// One block per (token row, head of q, k or v). Rows with position < 0 are padding.
template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
conv_norm_rope_kernel(const T* proj, long long ld, T* out, long long ldo, const T* state, const T* __restrict__ wconv,
                      int taps, int norm_mode, const float* __restrict__ qn, const float* __restrict__ kn, float eps,
                      const float* __restrict__ vmix, const T* v_src, long long ld_src,
                      const float* __restrict__ cosv, const float* __restrict__ sinv, int rot_dims, const int* row_pos,
                      const int* row_seq, const int* seq_pos0, const int* seq_slot, int nh, int nkv, int hd, int hdv,
                      T* k_store, T* v_store, const int* page_table, int pt_stride, const float* __restrict__ bias,
                      float qt_coef, int qt_every, int q_split) {
    __shared__ float red[33];
    __shared__ float ys[256];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, head = blockIdx.y;
    const int pos = row_pos[t];
    if (pos < 0) return;
    const int s = row_seq[t];
    const int p0 = seq_pos0[s];
    const int C = nh * hd + nkv * hd + nkv * hdv;
    int c0, size;
    const float* wn = nullptr;
    if (head < nh) { c0 = head * hd; size = hd; wn = qn; }
    else if (head < nh + nkv) { c0 = nh * hd + (head - nh) * hd; size = hd; wn = kn; }
    else { c0 = (nh + nkv) * hd + (head - nh - nkv) * hdv; size = hdv; }
    const bool rotates = head < nh + nkv && rot_dims > 0;
    const bool norms = head < nh + nkv && norm_mode != 0;
    const T* st = taps > 1 ? state + (size_t)seq_slot[s] * (taps - 1) * C : nullptr;
    float y[2];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int d = threadIdx.x + r * SC_THREADS;
        y[r] = 0.f;
        if (d < size) {
            const int c = c0 + d;
            float acc = 0.f;
            for (int j = 0; j < taps; j++) {
                const int back = taps - 1 - j;                 // u at position pos - back
                const int pp = pos - back;
                const float u = pp >= p0 ? to_f(proj[(size_t)(t - back) * ld + c])
                                         : to_f(st[(size_t)(taps - 1 - (p0 - pp)) * C + c]);
                const float w = taps > 1 ? to_f(wconv[(size_t)c * taps + j]) : 1.f;
                acc = fmaf(w, u, acc);
            }
            if (bias != nullptr) acc += bias[c];
            y[r] = acc;
            ss += acc * acc;
        }
    }
    if (norms) {     // the rotation turns pairs of coordinates and leaves the sum of squares as it is up to rounding; the
                     // norm behind it is taken of the rotated numbers all the same (below)
        if (norm_mode == 1) {
            ss = block_sum(ss, red);
            const float rs = 1.f / sqrtf(ss / (float)size + eps);
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int d = threadIdx.x + r * SC_THREADS;
                if (d < size) y[r] *= wn ? rs * wn[d] : rs;
            }
        }
    } else if (head >= nh + nkv && v_src != nullptr) {
        const float lam = vmix[0];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int d = threadIdx.x + r * SC_THREADS;
            if (d < size)
                y[r] = (1.f - lam) * y[r] + lam * to_f(v_src[(size_t)t * ld_src + (size_t)(head - nh - nkv) * hdv + d]);
        }
    }
    if (rotates) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int d = threadIdx.x + r * SC_THREADS;
            if (d < size) ys[d] = y[r];
        }
        __syncthreads();
        const int half = rot_dims / 2;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int d = threadIdx.x + r * SC_THREADS;
            if (d < rot_dims) {
                const int i = d < half ? d : d - half;
                const float c = cosv[(size_t)pos * half + i], sn = sinv[(size_t)pos * half + i];
                y[r] = d < half ? ys[d] * c - ys[d + half] * sn : ys[d] * c + ys[d - half] * sn;
            }
        }
    }
    if (norms && norm_mode == 2) {
        ss = 0.f;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int d = threadIdx.x + r * SC_THREADS;
            if (d < size) ss += y[r] * y[r];
        }
        ss = block_sum(ss, red);
        const float rs = 1.f / sqrtf(ss / (float)size + eps);
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int d = threadIdx.x + r * SC_THREADS;
            if (d < size) y[r] *= wn ? rs * wn[d] : rs;
        }
    }
    // k and v heads also go to the token's place in the paged stores when those are given (the cache write of the step)
    T* cached = nullptr;
    if (k_store != nullptr && head >= nh) {
        const int page = page_table[(size_t)s * pt_stride + pos / DK_PAGE];
        if (page >= 0 && (head < nh + nkv || v_store != nullptr))      // no store of values: only the keys are cached
            cached = head < nh + nkv ? k_store + kv_offset(page, nkv, head - nh, pos % DK_PAGE, hd)
                                     : v_store + kv_offset(page, nkv, head - nh - nkv, pos % DK_PAGE, hdv);
    }
    const float temp = head < nh && qt_every > 0 ? query_temperature(pos, qt_coef, qt_every) : 1.f;
    const int shift = (q_split - 1) * nh * hd;     // k and v stand behind q_split * nh query heads in ``out``
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int d = threadIdx.x + r * SC_THREADS;
        if (d < size) {
            const T o = from_f<T>(y[r] * temp);
            if (head < nh && q_split > 1) write_split(out + (size_t)t * ldo + (size_t)head * q_split * hd, d, hd, q_split, o);
            else out[(size_t)t * ldo + c0 + (head < nh ? 0 : shift) + d] = o;
            if (cached != nullptr) cached[d] = o;
        }
    }
}

// The same without a convolution (taps = 1): a warp per (token row, head), the head in registers (coordinate
// lane + 32 i), sums by shuffles, the rotation's partners through the warp's own piece of shared memory. No block
// barrier; eight heads a block.
#define SC_ROW_WARPS 8
template <typename T>
__global__ void __launch_bounds__(32 * SC_ROW_WARPS)
norm_rope_rows_kernel(const T* proj, long long ld, T* out, long long ldo, int norm_mode, const float* __restrict__ qn,
                      const float* __restrict__ kn, float eps, const float* __restrict__ vmix, const T* v_src,
                      long long ld_src, const float* __restrict__ cosv, const float* __restrict__ sinv, int rot_dims,
                      const int* row_pos, const int* row_seq, int n_tok, int nh, int nkv, int hd, int hdv, T* k_store,
                      T* v_store, const int* page_table, int pt_stride, const float* __restrict__ bias, float qt_coef,
                      int qt_every, int q_split) {
    __shared__ float ys_all[SC_ROW_WARPS][256];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = nh + 2 * nkv;
    const long long item = (long long)blockIdx.x * SC_ROW_WARPS + warp;
    if (item >= (long long)n_tok * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    const int pos = row_pos[t];
    if (pos < 0) return;
    float* ys = ys_all[warp];
    int c0, size;
    const float* wn = nullptr;
    if (head < nh) { c0 = head * hd; size = hd; wn = qn; }
    else if (head < nh + nkv) { c0 = nh * hd + (head - nh) * hd; size = hd; wn = kn; }
    else { c0 = (nh + nkv) * hd + (head - nh - nkv) * hdv; size = hdv; }
    const bool qk = head < nh + nkv;
    const T* src = proj + (size_t)t * ld + c0;
    float y[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        y[i] = d < size ? to_f(src[d]) + (bias != nullptr ? bias[c0 + d] : 0.f) : 0.f;
        ss += y[i] * y[i];
    }
    if (qk && norm_mode == 1) {
        const float rs = 1.f / sqrtf(warp_sum(ss) / (float)size + eps);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            if (d < size) y[i] *= wn ? rs * wn[d] : rs;
        }
    }
    if (!qk && v_src != nullptr) {
        const float lam = vmix[0];
        const T* vs = v_src + (size_t)t * ld_src + (size_t)(head - nh - nkv) * hdv;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            if (d < size) y[i] = (1.f - lam) * y[i] + lam * to_f(vs[d]);
        }
    }
    if (qk && rot_dims > 0) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            if (d < rot_dims) ys[d] = y[i];
        }
        __syncwarp();
        const int half = rot_dims / 2;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            if (d < rot_dims) {
                const int j = d < half ? d : d - half;
                const float c = cosv[(size_t)pos * half + j], sn = sinv[(size_t)pos * half + j];
                y[i] = d < half ? ys[d] * c - ys[d + half] * sn : ys[d] * c + ys[d - half] * sn;
            }
        }
    }
    if (qk && norm_mode == 2) {
        ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) ss += y[i] * y[i];        // coordinates past the head's size are zero
        const float rs = 1.f / sqrtf(warp_sum(ss) / (float)size + eps);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            if (d < size) y[i] *= wn ? rs * wn[d] : rs;
        }
    }
    T* cached = nullptr;
    if (k_store != nullptr && head >= nh) {
        const int page = page_table[(size_t)row_seq[t] * pt_stride + pos / DK_PAGE];
        if (page >= 0 && (head < nh + nkv || v_store != nullptr))      // no store of values: only the keys are cached
            cached = head < nh + nkv ? k_store + kv_offset(page, nkv, head - nh, pos % DK_PAGE, hd)
                                     : v_store + kv_offset(page, nkv, head - nh - nkv, pos % DK_PAGE, hdv);
    }
    const float temp = head < nh && qt_every > 0 ? query_temperature(pos, qt_coef, qt_every) : 1.f;
    T* dst = out + (size_t)t * ldo + c0 + (head < nh ? 0 : (q_split - 1) * nh * hd);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        if (d < size) {
            const T o = from_f<T>(y[i] * temp);
            if (head < nh && q_split > 1) write_split(out + (size_t)t * ldo + (size_t)head * q_split * hd, d, hd, q_split, o);
            else dst[d] = o;
            if (cached != nullptr) cached[d] = o;
        }
    }
}

// state[slot] <- the last taps - 1 projected rows of the sequence as it stands after this step: rows of
// this step where it brought enough, the newest of the old state before them where it did not.
template <typename T>
__global__ void conv_state_update_kernel(const T* proj, long long ld, T* state, int taps, int C, const int* cu_q,
                                         const int* seq_pos0, const int* seq_slot) {
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C || seq_pos0[s] < 0) return;
    const int r0 = cu_q ? cu_q[s] : s, len = cu_q ? cu_q[s + 1] - r0 : 1;   // no cu_q: row s is sequence s, one token
    T* st = state + (size_t)seq_slot[s] * (taps - 1) * C;
    T old[SC_MAX_TAPS - 1];
#pragma unroll
    for (int i = 0; i < SC_MAX_TAPS - 1; i++)
        if (i < taps - 1) old[i] = st[(size_t)i * C + c];
#pragma unroll
    for (int i = 0; i < SC_MAX_TAPS - 1; i++) {
        if (i < taps - 1) {
            const int r = len - (taps - 1) + i;              // row of this step that lands in place i
            st[(size_t)i * C + c] = r >= 0 ? proj[(size_t)(r0 + r) * ld + c] : old[i + len];
        }
    }
}

DK_EXPORT int dk_conv_norm_rope(int dtype, const void* proj, long long ld, void* out, long long ldo, const void* state,
                                const void* wconv, int taps, int norm_mode, const float* qn, const float* kn, float eps,
                                const float* vmix, const void* v_src, long long ld_src, const float* cosv, const float* sinv, int rot_dims, const int* row_pos,
                                const int* row_seq, const int* seq_pos0, const int* seq_slot, int n_tok, int nh, int nkv,
                                int hd, int hdv, void* k_store, void* v_store, const int* page_table, int pt_stride,
                                const float* bias, float qt_coef, int qt_every, int q_split, cudaStream_t st) {
    if (hd > 256 || hdv > 256 || taps < 1 || taps > SC_MAX_TAPS || rot_dims > hd || rot_dims % 2 || q_split < 1 ||
        hd % q_split || qt_every < 0)
        return (int)cudaErrorInvalidValue;
    if (taps == 1) {
        const long long items = (long long)n_tok * (nh + 2 * nkv);
        const dim3 rgrid((unsigned)((items + SC_ROW_WARPS - 1) / SC_ROW_WARPS)), rblock(32 * SC_ROW_WARPS);
        if (dtype == 0)
            return dk_launch(norm_rope_rows_kernel<float>, rgrid, rblock, 0, st, (const float*)proj, ld, (float*)out, ldo,
                             norm_mode, qn, kn, eps, vmix, (const float*)v_src, ld_src, cosv, sinv, rot_dims, row_pos,
                             row_seq, n_tok, nh, nkv, hd, hdv, (float*)k_store, (float*)v_store, page_table, pt_stride, bias, qt_coef,
                             qt_every, q_split);
        return dk_launch(norm_rope_rows_kernel<bf16>, rgrid, rblock, 0, st, (const bf16*)proj, ld, (bf16*)out, ldo, norm_mode,
                         qn, kn, eps, vmix, (const bf16*)v_src, ld_src, cosv, sinv, rot_dims, row_pos, row_seq, n_tok, nh,
                         nkv, hd, hdv, (bf16*)k_store, (bf16*)v_store, page_table, pt_stride, bias, qt_coef, qt_every, q_split);
    }
    const dim3 grid(n_tok, nh + 2 * nkv), block(SC_THREADS);
    if (dtype == 0)
        return dk_launch(conv_norm_rope_kernel<float>, grid, block, 0, st, (const float*)proj, ld, (float*)out, ldo,
                         (const float*)state, (const float*)wconv, taps, norm_mode, qn, kn, eps, vmix, (const float*)v_src, ld_src, cosv, sinv, rot_dims, row_pos,
                         row_seq, seq_pos0, seq_slot, nh, nkv, hd, hdv, (float*)k_store, (float*)v_store, page_table, pt_stride,
                         bias, qt_coef, qt_every, q_split);
    return dk_launch(conv_norm_rope_kernel<bf16>, grid, block, 0, st, (const bf16*)proj, ld, (bf16*)out, ldo,
                     (const bf16*)state, (const bf16*)wconv, taps, norm_mode, qn, kn, eps, vmix, (const bf16*)v_src, ld_src, cosv, sinv, rot_dims, row_pos, row_seq,
                     seq_pos0, seq_slot, nh, nkv, hd, hdv, (bf16*)k_store, (bf16*)v_store, page_table, pt_stride, bias, qt_coef,
                     qt_every, q_split);
}

DK_EXPORT int dk_conv_state_update(int dtype, const void* proj, long long ld, void* state, int taps, int C,
                                   const int* cu_q, const int* seq_pos0, const int* seq_slot, int n_seq, cudaStream_t st) {
    if (taps < 2 || taps > SC_MAX_TAPS) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_seq, (C + 127) / 128), block(128);
    if (dtype == 0)
        return dk_launch(conv_state_update_kernel<float>, grid, block, 0, st, (const float*)proj, ld, (float*)state,
                         taps, C, cu_q, seq_pos0, seq_slot);
    return dk_launch(conv_state_update_kernel<bf16>, grid, block, 0, st, (const bf16*)proj, ld, (bf16*)state, taps, C,
                     cu_q, seq_pos0, seq_slot);
}
