// Linear recurrences over a float32 state per (sequence, head), S [D, V], token by token:
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t
// with q, k [tokens, heads, D], the decay a per key channel [tokens, heads, D] and v [tokens, heads, V]. Every operand
// is float32: what enters the recurrence is made in float32, head by head, by the kernels in front of it.
// Two mixers use it:
//   * a gated recurrence whose forget gate also decides what is written (hgrn2_prepare): from projection rows
//     [q | f | v]: q <- silu(q), a = l + (1 - l) sigmoid(f + b) with a lower bound l per channel, k = 1 - a;
//   * a state-space mixer (ssd_prepare): from projection rows [.. | x B C | dt]: a causal convolution with bias over
//     time on every channel of x, B, C (its memory, the last taps - 1 projected rows, is a per-sequence state), then
//     SiLU; dt <- softplus(dt + bias); a = exp(-exp(A_log_h) dt) on every channel, k = dt B, q = C, v = x.
// The recurrence kernel serves prompts, portions and single tokens alike (rows of a sequence are cu_q[s] ..
// cu_q[s + 1], or row s alone without cu_q; seq_pos0[s] < 0 marks a padding row: zeros out, state untouched).
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// proj rows [q (n) | f (n) | v (nv)] in the storage type -> q32 = silu(q), a = l + (1 - l) sigmoid(f + b), k32 = 1 - a, v32;
// q32, k32, v32 are column ranges of one float32 matrix of row stride ldo, a32 is dense [tokens, n]
template <typename T>
__global__ void hgrn2_prepare_kernel(const T* proj, long long ld, const float* __restrict__ fbias, const float* __restrict__ lower,
                                     float* q32, float* k32, float* a32, float* v32, long long ldo, int n, int nv, size_t total) {
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
        q32[t * ldo + c] = q * sigmoid_f(q);
        a32[t * n + c] = a;
        k32[t * ldo + c] = 1.f - a;
    } else {
        v32[t * ldo + (c - n)] = to_f(row[2 * n + c - n]);
    }
}

// xbc rows [x (inner) | B | C] (C channels in all) and dt rows [heads] of a projection in the storage type: conv + bias +
// SiLU on every channel; dt = softplus(dt + dt_bias). Out, per head h of group g: q32[t, h] = C[t, g], k32[t, h] = dt_h B[t, g],
// a32[t, h, :] = exp(-exp(A_log_h) dt_h) on every channel, v32[t, h] = x[t, h]: the operands of the recurrence, head by head.
// q32, k32, v32 are column ranges of one float32 matrix of row stride ldo; a32 is dense [tokens, heads * N].
// state [slots, taps - 1, C] holds each sequence's last taps - 1 projected xbc rows (read only here).
template <typename T>
__global__ void ssd_prepare_kernel(const T* xbc, const T* dt, long long ld, const T* state, const T* __restrict__ wconv,
                                   const float* __restrict__ cbias, int taps, const float* __restrict__ dt_bias,
                                   const float* __restrict__ a_log, const int* row_pos, const int* row_seq, const int* seq_pos0,
                                   const int* seq_slot, float* q32, float* k32, float* a32, float* v32, long long ldo, int inner,
                                   int nbc, int nh, int groups) {
    extern __shared__ float sp_smem[];       // [C] the row after the convolution and SiLU, then [nh] dt, [nh] decay
    pdl_wait();
    pdl_launch_dependents();
    const int C = inner + 2 * nbc, N = nbc / groups, hpg = nh / groups;
    float* row = sp_smem;
    float* dts = sp_smem + C;
    float* dec = dts + nh;
    const int t = blockIdx.x;
    const int pos = row_pos[t];
    if (pos < 0) {        // a padding row: zeros, so that what follows stays finite
        for (int c = threadIdx.x; c < inner; c += blockDim.x) v32[(size_t)t * ldo + c] = 0.f;
        for (int i = threadIdx.x; i < nh * N; i += blockDim.x) {
            q32[(size_t)t * ldo + i] = 0.f;
            k32[(size_t)t * ldo + i] = 0.f;
            a32[(size_t)t * nh * N + i] = 0.f;
        }
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
        row[c] = y;
        if (c < inner) v32[(size_t)t * ldo + c] = y;
    }
    for (int h = threadIdx.x; h < nh; h += blockDim.x) {
        const float z = to_f(dt[(size_t)t * ld + h]) + dt_bias[h];
        const float d = z > 20.f ? z : log1pf(expf(z));
        dts[h] = d;
        dec[h] = expf(-expf(a_log[h]) * d);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * N; i += blockDim.x) {
        const int h = i / N, n = i % N, g = h / hpg;
        q32[(size_t)t * ldo + i] = row[inner + nbc + g * N + n];
        k32[(size_t)t * ldo + i] = dts[h] * row[inner + g * N + n];
        a32[(size_t)t * nh * N + i] = dec[h];
    }
}

#define REC_WARPS 4
#define REC_VC 4
// A warp per (sequence, head, REC_VC value columns): lane l holds the state's rows l, l + 32, .. (DPL of them) of its
// columns in registers for the whole portion (16 bytes a row where the value size allows: VEC). The next token's operands
// are requested before this token's arithmetic. q, k, v [tokens, heads * size] of one row stride ld, a dense.
template <int DPL, bool VEC>
__global__ void __launch_bounds__(32 * REC_WARPS)
recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, long long ld,
                  const float* __restrict__ a, float* __restrict__ out, float* state, const int* cu_q, const int* seq_pos0,
                  const int* seq_slot, int nh, int hd, int hdv) {
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
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)hd * hdv;
    float st[DPL][REC_VC];
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
        if (VEC) {
            const float4 x = d < hd ? *reinterpret_cast<const float4*>(S + (size_t)d * hdv + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
            st[i][0] = x.x, st[i][1] = x.y, st[i][2] = x.z, st[i][3] = x.w;
        } else {
#pragma unroll
            for (int c = 0; c < REC_VC; c++) st[i][c] = d < hd && c0 + c < hdv ? S[(size_t)d * hdv + c0 + c] : 0.f;
        }
    }
    float qn[DPL], kn[DPL], an[DPL], vn[REC_VC];
    auto fetch = [&](int t) {
        const float* qr = q + (size_t)t * ld + (size_t)h * hd;
        const float* kr = k + (size_t)t * ld + (size_t)h * hd;
        const float* ar = a + ((size_t)t * nh + h) * hd;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            const int d = lane + 32 * i;
            qn[i] = d < hd ? qr[d] : 0.f;
            kn[i] = d < hd ? kr[d] : 0.f;
            an[i] = d < hd ? ar[d] : 0.f;
        }
#pragma unroll
        for (int c = 0; c < REC_VC; c++) vn[c] = c0 + c < hdv ? v[(size_t)t * ld + (size_t)h * hdv + c0 + c] : 0.f;
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
        // the four column sums side by side: their shuffles are independent chains
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
#pragma unroll
            for (int c = 0; c < REC_VC; c++) o[c] += __shfl_xor_sync(0xffffffffu, o[c], off);
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
        if (VEC) {
            if (d < hd) *reinterpret_cast<float4*>(S + (size_t)d * hdv + c0) = make_float4(st[i][0], st[i][1], st[i][2], st[i][3]);
        } else {
#pragma unroll
            for (int c = 0; c < REC_VC; c++)
                if (d < hd && c0 + c < hdv) S[(size_t)d * hdv + c0 + c] = st[i][c];
        }
    }
}

DK_EXPORT int dk_hgrn2_prepare(int dtype, const void* proj, long long ld, const float* fbias, const float* lower, float* q32,
                               float* k32, float* a32, float* v32, long long ldo, int n_tok, int n, int nv, cudaStream_t st) {
    const size_t total = (size_t)n_tok * (n + nv);
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
    if (dtype == 0)
        return dk_launch(hgrn2_prepare_kernel<float>, grid, block, 0, st, (const float*)proj, ld, fbias, lower, q32, k32, a32, v32,
                         ldo, n, nv, total);
    return dk_launch(hgrn2_prepare_kernel<bf16>, grid, block, 0, st, (const bf16*)proj, ld, fbias, lower, q32, k32, a32, v32, ldo, n,
                     nv, total);
}

DK_EXPORT int dk_ssd_prepare(int dtype, const void* xbc, const void* dt, long long ld, const void* state, const void* wconv,
                             const float* cbias, int taps, const float* dt_bias, const float* a_log, const int* row_pos,
                             const int* row_seq, const int* seq_pos0, const int* seq_slot, float* q32, float* k32, float* a32,
                             float* v32, long long ldo, int n_tok, int inner, int nbc, int nh, int groups, cudaStream_t st) {
    const int C = inner + 2 * nbc;
    if (taps < 1 || (taps > 1 && state == nullptr) || groups < 1 || nh % groups || nbc % groups) return (int)cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * (size_t)(C + 2 * nh);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_tok), block(C >= 1024 ? 256 : 128);
    if (dtype == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(ssd_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return dk_launch(ssd_prepare_kernel<float>, grid, block, smem, st, (const float*)xbc, (const float*)dt, ld, (const float*)state,
                         (const float*)wconv, cbias, taps, dt_bias, a_log, row_pos, row_seq, seq_pos0, seq_slot, q32, k32, a32, v32,
                         ldo, inner, nbc, nh, groups);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(ssd_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return dk_launch(ssd_prepare_kernel<bf16>, grid, block, smem, st, (const bf16*)xbc, (const bf16*)dt, ld, (const bf16*)state,
                     (const bf16*)wconv, cbias, taps, dt_bias, a_log, row_pos, row_seq, seq_pos0, seq_slot, q32, k32, a32, v32, ldo,
                     inner, nbc, nh, groups);
}

DK_EXPORT int dk_recurrence(const float* q, const float* k, const float* v, long long ld, const float* a, float* out, float* state,
                            const int* cu_q, const int* seq_pos0, const int* seq_slot, int n_seq, int nh, int hd, int hdv,
                            cudaStream_t st) {
    if (hd < 1 || hd > 256 || hdv < 1) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_seq, nh, (hdv + REC_WARPS * REC_VC - 1) / (REC_WARPS * REC_VC)), block(32 * REC_WARPS);
    const bool vec = hdv % 4 == 0 && (uintptr_t)state % 16 == 0;
#define REC_LAUNCH(D)                                                                                                        \
    if (hd <= 32 * D) {                                                                                                      \
        if (vec)                                                                                                             \
            return dk_launch(recurrence_kernel<D, true>, grid, block, 0, st, q, k, v, ld, a, out, state, cu_q, seq_pos0, seq_slot, \
                             nh, hd, hdv);                                                                                   \
        return dk_launch(recurrence_kernel<D, false>, grid, block, 0, st, q, k, v, ld, a, out, state, cu_q, seq_pos0, seq_slot, nh, \
                         hd, hdv);                                                                                           \
    }
    REC_LAUNCH(1) REC_LAUNCH(2) REC_LAUNCH(3) REC_LAUNCH(4) REC_LAUNCH(6) REC_LAUNCH(8)
#undef REC_LAUNCH
    return (int)cudaErrorInvalidValue;
}
