// Matrix products out[M,N] = x[M,K] . W[N,K]^T (weights row-major [out, in], no bias), reference:
// engine/engine.py:131-146 (linear, gate/up + SiLU).
//
//  * sgemm: true float32 on CUDA cores (FMA, no tensor-core mode), any M, N, K. Each output is
//    one sequential sum over K, so a row's result does not depend on the other rows of the batch.
//    Epilogues: 0/1 store, 2 W = [gate; up]: store silu(gate)*up (with act_pos = 1: the tanh form of GELU instead of SiLU;
//    act_pos = 2: g' = min(gate, L), u' = clamp(up, -L, L), store g' sigmoid(1.702 g') (u' + 1) with L = act_neg).
//  * sum_partials: adds up the float32 partial sums of a split-K bfloat16 product for a consumer
//    that cannot do it while it reads.
#include "common.cuh"

// ------------------------------------------------------------------------------------------ sgemm
#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

// The gate of a gated product: v * sigmoid(a) with a = v for SiLU, and a = 2 sqrt(2/pi) (v + 0.044715 v^3) for the tanh
// form of GELU (0.5 v (1 + tanh(u)) = v sigmoid(2u)).
__device__ __forceinline__ float gate_arg(float v, bool gelu) { return gelu ? 1.5957691216057308f * v * fmaf(0.044715f * v, v, 1.f) : v; }
template <bool SILU, bool XIELU>
__global__ void __launch_bounds__(256)
sgemm_kernel(const float* x, const float* __restrict__ W, float* out, int M, int N, int K, float act_pos, float act_neg) {
    __shared__ float xs[SG_BK][SG_BM + 4];
    __shared__ float ws[SG_BK][SG_BN + 4];
    __shared__ float us[SILU ? SG_BK : 1][SG_BN + 4];
    pdl_wait();
    pdl_launch_dependents();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;  // loader: row in tile, first k
    float acc[4][4] = {}, acu[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int k = k0 + lk + e;
            const int m = m0 + lr, n = n0 + lr;
            xs[lk + e][lr] = (m < M && k < K) ? x[(size_t)m * K + k] : 0.f;
            ws[lk + e][lr] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
            if (SILU) us[lk + e][lr] = (n < N && k < K) ? W[(size_t)(n + N) * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; kk++) {
            float a[4], b[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[kk][tx * 4 + j];
            if (SILU) {
#pragma unroll
                for (int j = 0; j < 4; j++) u[j] = us[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (SILU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                float v = acc[i][j];
                if (SILU) {
                    if (act_pos > 1.5f) {     // act_pos 2: the clamped gate with the limit act_neg
                        const float g = fminf(v, act_neg), u = fminf(fmaxf(acu[i][j], -act_neg), act_neg);
                        v = g / (1.f + expf(-1.702f * g)) * (u + 1.f);
                    } else {
                        v = v / (1.f + expf(-gate_arg(v, act_pos > 0.5f))) * acu[i][j];   // act_pos 1: GELU gate
                    }
                }
                if (XIELU) v = xielu_f(v, act_pos, act_neg);
                out[(size_t)m * N + n] = v;
            }
        }
}

// mode 0/1: plain; mode 2: W has 2N rows [gate; up], out [M, N]; mode 3: xIELU(x . W^T) with the two constants
DK_EXPORT int dk_sgemm(const float* x, const float* W, float* out, int M, int N, int K, int mode, float act_pos, float act_neg,
                       cudaStream_t st) {
    dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
    if (mode == 2) return dk_launch(sgemm_kernel<true, false>, grid, dim3(256), 0, st, x, W, out, M, N, K, act_pos, act_neg);
    if (mode == 3) return dk_launch(sgemm_kernel<false, true>, grid, dim3(256), 0, st, x, W, out, M, N, K, act_pos, act_neg);
    return dk_launch(sgemm_kernel<false, false>, grid, dim3(256), 0, st, x, W, out, M, N, K, 0.f, 0.f);
}

// ----------------------------------------------------------------------------------- partial sums
// out[m][n] = sum over slices of ws[slice][m][n], stored as bf16: for a consumer that cannot add
// the partial sums up itself.
__global__ void sum_partials_kernel(const float* ws, bf16* out, size_t mn, int SK) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= mn) return;
    float s = 0.f;
    for (int k = 0; k < SK; k++) s += ws[(size_t)k * mn + i];
    out[i] = __float2bfloat16_rn(s);
}

DK_EXPORT int dk_sum_partials(const float* ws, void* out, long long mn, int SK, cudaStream_t st) {
    return dk_launch(sum_partials_kernel, dim3((unsigned)((mn + 255) / 256)), dim3(256), 0, st, ws, (bf16*)out, (size_t)mn, SK);
}
