// Linear recurrences over a float32 state per (sequence, head), S [D, V], token by token:
//     S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T,     o_t = S_t^T q_t
// with q, k [tokens, groups of heads, D] (head h reads group h / (heads / groups)), an optional factor c [tokens, heads]
// on k, the decay a either per key channel [tokens, heads, D] or one number a head [tokens, heads], and v [tokens,
// heads, V]. Every operand is float32: what enters the recurrence is made in float32 by the kernels in front of it.
// Two mixers use it:
//   * a gated recurrence whose forget gate also decides what is written (hgrn2_prepare): from projection rows
//     [q | f | v]: q <- silu(q), a = l + (1 - l) sigmoid(f + b) with a lower bound l per channel, k = 1 - a;
//   * a state-space mixer (ssd_prepare): from projection rows [.. | x B C | dt]: a causal convolution with bias over
//     time on every channel of x, B, C (its memory, the last taps - 1 projected rows, is a per-sequence state), then
//     SiLU; dt <- softplus(dt + bias); a = exp(-exp(A_log_h) dt), c = dt, k = B, q = C, v = x.
// The recurrence kernel serves prompts, portions and single tokens alike (rows of a sequence are cu_q[s] ..
// cu_q[s + 1], or row s alone without cu_q; seq_pos0[s] < 0 marks a padding row: zeros out, state untouched).
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// proj rows [q (n) | f (n) | v (nv)] in the storage type -> q32 = silu(q), a = l + (1 - l) sigmoid(f + b), k32 = 1 - a, v32
template <typename T>
__global__ void hgrn2_prepare_kernel(const T* proj, long long ld, const float* __restrict__ fbias, const float* __restrict__ lower,
                                     float* q32, float* k32, float* a32, float* v32, int n, int nv, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / (n + nv);
    const int c = (int)(i % (n + nv));
    const T* row = proj + t * ld;
    if (c < n) {
        const float q = to_f(row[c]);
        const float l = lower[c];
        const float a = l + (1.f - l) * sigmoid_f(to_f(row[n + c]) + fbias[c]);
        q32[t * n + c] = q * sigmoid_f(q);
        a32[t * n + c] = a;
        k32[t * n + c] = 1.f - a;
    } else {
        v32[t * nv + (c - n)] = to_f(row[2 * n + c - n]);
    }
}

// xbc rows [x (inner) | B | C] (C channels in all) and dt rows [heads] of a projection in the storage type:
// conv + bias + SiLU -> x32 [tokens, inner], b32 and c32 [tokens, nbc]; dt32 = softplus(dt + dt_bias); a32 = exp(-exp(A_log) dt32).
// state [slots, taps - 1, C] holds each sequence's last taps - 1 projected xbc rows (read only here).
template <typename T>
__global__ void ssd_prepare_kernel(const T* xbc, const T* dt, long long ld, const T* state, const T* __restrict__ wconv,
                                   const float* __restrict__ cbias, int taps, const float* __restrict__ dt_bias,
                                   const float* __restrict__ a_log, const int* row_pos, const int* row_seq, const int* seq_pos0,
                                   const int* seq_slot, float* x32, float* b32, float* c32, float* dt32, float* a32, int C, int inner,
                                   int nbc, int nh) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = row_pos[t];
    if (pos < 0) {        // a padding row: zeros, so that what follows stays finite
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            if (c < inner) x32[(size_t)t * inner + c] = 0.f;
            else if (c < inner + nbc) b32[(size_t)t * nbc + c - inner] = 0.f;
            else c32[(size_t)t * nbc + c - inner - nbc] = 0.f;
        }
        for (int h = threadIdx.x; h < nh; h += blockDim.x) dt32[(size_t)t * nh + h] = a32[(size_t)t * nh + h] = 0.f;
        return;
    }
    const int s = row_seq[t];
    const int p0 = seq_pos0[s];
    const T* st = state + (size_t)seq_slot[s] * (taps - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = cbias ? cbias[c] : 0.f;
        for (int j = 0; j < taps; j++) {
            const int back = taps - 1 - j;                   // the input at position pos - back
            const int pp = pos - back;
            const float u = pp >= p0 ? to_f(xbc[(size_t)(t - back) * ld + c]) : to_f(st[(size_t)(taps - 1 - (p0 - pp)) * C + c]);
            acc = fmaf(to_f(wconv[(size_t)c * taps + j]), u, acc);
        }
        const float y = acc * sigmoid_f(acc);
        if (c < inner) x32[(size_t)t * inner + c] = y;
        else if (c < inner + nbc) b32[(size_t)t * nbc + c - inner] = y;
        else c32[(size_t)t * nbc + c - inner - nbc] = y;
    }
    for (int h = threadIdx.x; h < nh; h += blockDim.x) {
        const float z = to_f(dt[(size_t)t * ld + h]) + dt_bias[h];
        const float d = z > 20.f ? z : log1pf(expf(z));
        dt32[(size_t)t * nh + h] = d;
        a32[(size_t)t * nh + h] = expf(-expf(a_log[h]) * d);
    }
}

#define REC_WARPS 4
#define REC_VC 4
// A warp per (sequence, head, REC_VC value columns): lane l holds the state's rows l, l + 32, .. (DPL of them) of its
// columns in registers for the whole portion. The next token's operands are requested before this token's arithmetic.
template <int DPL>
__global__ void __launch_bounds__(32 * REC_WARPS)
recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k, int qk_heads, const float* __restrict__ kfac,
                  const float* __restrict__ a, int a_per_head, const float* __restrict__ v, float* __restrict__ out, float* state,
                  const int* cu_q, const int* seq_pos0, const int* seq_slot, int nh, int hd, int hdv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = blockIdx.x, h = blockIdx.y;
    const int c0 = (blockIdx.z * REC_WARPS + warp) * REC_VC;
    if (c0 >= hdv) return;
    const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
    const size_t ow = (size_t)nh * hdv;
    if (seq_pos0[s] < 0) {
        if (lane < REC_VC && c0 + lane < hdv)
            for (int t = r0; t < r1; t++) out[(size_t)t * ow + (size_t)h * hdv + c0 + lane] = 0.f;
        return;
    }
    const int g = h / (nh / qk_heads);
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)hd * hdv;
    float st[DPL][REC_VC];
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < REC_VC; c++) st[i][c] = d < hd && c0 + c < hdv ? S[(size_t)d * hdv + c0 + c] : 0.f;
    }
    float qn[DPL], kn[DPL], an[DPL], vn[REC_VC];
    auto fetch = [&](int t) {
        const float* qr = q + ((size_t)t * qk_heads + g) * hd;
        const float* kr = k + ((size_t)t * qk_heads + g) * hd;
        const float kf = kfac ? kfac[(size_t)t * nh + h] : 1.f;
        const float ah = a_per_head ? a[(size_t)t * nh + h] : 0.f;
        const float* ar = a + ((size_t)t * nh + h) * hd;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            const int d = lane + 32 * i;
            qn[i] = d < hd ? qr[d] : 0.f;
            kn[i] = d < hd ? kr[d] * kf : 0.f;
            an[i] = a_per_head ? ah : (d < hd ? ar[d] : 0.f);
        }
#pragma unroll
        for (int c = 0; c < REC_VC; c++) vn[c] = c0 + c < hdv ? v[(size_t)t * ow + (size_t)h * hdv + c0 + c] : 0.f;
    };
    fetch(r0);
    for (int t = r0; t < r1; t++) {
        float qv[DPL], kv[DPL], av[DPL], vv[REC_VC];
#pragma unroll
        for (int i = 0; i < DPL; i++) { qv[i] = qn[i]; kv[i] = kn[i]; av[i] = an[i]; }
#pragma unroll
        for (int c = 0; c < REC_VC; c++) vv[c] = vn[c];
        if (t + 1 < r1) fetch(t + 1);
        float o[REC_VC];
#pragma unroll
        for (int c = 0; c < REC_VC; c++) o[c] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++)
#pragma unroll
            for (int c = 0; c < REC_VC; c++) {
                st[i][c] = fmaf(av[i], st[i][c], kv[i] * vv[c]);
                o[c] = fmaf(st[i][c], qv[i], o[c]);
            }
#pragma unroll
        for (int c = 0; c < REC_VC; c++) o[c] = warp_sum(o[c]);
        if (lane < REC_VC && c0 + lane < hdv) {
            float r = o[0];
#pragma unroll
            for (int c = 1; c < REC_VC; c++) r = lane == c ? o[c] : r;
            out[(size_t)t * ow + (size_t)h * hdv + c0 + lane] = r;
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < REC_VC; c++)
            if (d < hd && c0 + c < hdv) S[(size_t)d * hdv + c0 + c] = st[i][c];
    }
}

DK_EXPORT int dk_hgrn2_prepare(int dtype, const void* proj, long long ld, const float* fbias, const float* lower, float* q32,
                               float* k32, float* a32, float* v32, int n_tok, int n, int nv, cudaStream_t st) {
    const size_t total = (size_t)n_tok * (n + nv);
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
    if (dtype == 0)
        return dk_launch(hgrn2_prepare_kernel<float>, grid, block, 0, st, (const float*)proj, ld, fbias, lower, q32, k32, a32, v32,
                         n, nv, total);
    return dk_launch(hgrn2_prepare_kernel<bf16>, grid, block, 0, st, (const bf16*)proj, ld, fbias, lower, q32, k32, a32, v32, n, nv,
                     total);
}

DK_EXPORT int dk_ssd_prepare(int dtype, const void* xbc, const void* dt, long long ld, const void* state, const void* wconv,
                             const float* cbias, int taps, const float* dt_bias, const float* a_log, const int* row_pos,
                             const int* row_seq, const int* seq_pos0, const int* seq_slot, float* x32, float* b32, float* c32,
                             float* dt32, float* a32, int n_tok, int inner, int nbc, int nh, cudaStream_t st) {
    const int C = inner + 2 * nbc;
    if (taps < 1 || (taps > 1 && state == nullptr)) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_tok), block(C >= 1024 ? 256 : 128);
    if (dtype == 0)
        return dk_launch(ssd_prepare_kernel<float>, grid, block, 0, st, (const float*)xbc, (const float*)dt, ld, (const float*)state,
                         (const float*)wconv, cbias, taps, dt_bias, a_log, row_pos, row_seq, seq_pos0, seq_slot, x32, b32, c32, dt32, a32, C,
                         inner, nbc, nh);
    return dk_launch(ssd_prepare_kernel<bf16>, grid, block, 0, st, (const bf16*)xbc, (const bf16*)dt, ld, (const bf16*)state,
                     (const bf16*)wconv, cbias, taps, dt_bias, a_log, row_pos, row_seq, seq_pos0, seq_slot, x32, b32, c32, dt32, a32, C,
                         inner, nbc, nh);
}

DK_EXPORT int dk_recurrence(const float* q, const float* k, int qk_heads, const float* kfac, const float* a, int a_per_head,
                            const float* v, float* out, float* state, const int* cu_q, const int* seq_pos0, const int* seq_slot,
                            int n_seq, int nh, int hd, int hdv, cudaStream_t st) {
    if (hd < 1 || hd > 256 || hdv < 1 || qk_heads < 1 || nh % qk_heads) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_seq, nh, (hdv + REC_WARPS * REC_VC - 1) / (REC_WARPS * REC_VC)), block(32 * REC_WARPS);
#define REC_LAUNCH(D)                                                                                                      \
    if (hd <= 32 * D)                                                                                                      \
        return dk_launch(recurrence_kernel<D>, grid, block, 0, st, q, k, qk_heads, kfac, a, a_per_head, v, out, state, cu_q, \
                         seq_pos0, seq_slot, nh, hd, hdv);
    REC_LAUNCH(1) REC_LAUNCH(2) REC_LAUNCH(3) REC_LAUNCH(4) REC_LAUNCH(6) REC_LAUNCH(8)
#undef REC_LAUNCH
    return (int)cudaErrorInvalidValue;
}
