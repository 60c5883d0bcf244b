// Mixture of experts: the router and the routed experts' feed-forward.
//
// Router (float32 throughout): z = W_r x, s = sigmoid(z); the choice is made on s + correction, among the
// experts of the `keep` best of `groups` equal groups of neighbouring experts (a group's score is the sum of
// its two largest choice scores; the others' choice scores count as minus infinity), the `top` largest;
// the weights are the chosen experts' s (without the correction) over their sum, times a constant. The same
// kernel works out the gate of a shared expert, sigmoid(w_sg . x), one number a token.
//
// Experts, row form (this file): every (token, chosen expert) pair is a row of its own,
//   mid[pair] = act(W_gate[e] x) * (W_up[e] x),   out[token] = sum_j weight_j W_down[e_j] mid[pair_j]
//                                                              + gate * shared[token],
// a warp per output column, float32 sums. It serves single-token steps, where a pair reads its expert's
// matrices once, and every float32 step; prompts in bfloat16 go through the tiled form (moe_tiles.cu).
#include "common.cuh"

#define MOE_MAX_EXPERTS 256
#define ROUTE_WARPS 8
#define ROUTE_TOKENS 8

// (value, index) with the larger value, the lower index among equal values, over the warp
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// The router in two kernels. Scores: block (8 tokens, 8 experts), the tokens' rows in shared memory, a warp an expert
// (the row after the last expert is the shared expert's gate): its row of the router is read once for the 8 tokens, 16
// bytes a lane where the width allows; sigmoid of the float32 sums -> scores [tokens, experts] (and the gate).
template <typename T>
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_scores_kernel(const T* x, int W, const float* __restrict__ wr, const float* __restrict__ wsg, int E, float* scores,
                  float* sgate, int n_tok, int by_logit) {
    extern __shared__ __align__(16) unsigned char route_smem[];
    T* xs = reinterpret_cast<T*>(route_smem);          // [ROUTE_TOKENS][W]
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int t0 = blockIdx.x * ROUTE_TOKENS;
    const int nt = min(ROUTE_TOKENS, n_tok - t0);
    const int e = blockIdx.y * ROUTE_WARPS + w;
    const bool vec = W % 8 == 0;
    if (vec) {
        const int pieces = nt * W * (int)sizeof(T) / 16;
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t0 * W);
        for (int i = threadIdx.x; i < pieces; i += blockDim.x) reinterpret_cast<uint4*>(xs)[i] = src[i];
    } else {
        for (int i = threadIdx.x; i < nt * W; i += blockDim.x) xs[i] = x[(size_t)t0 * W + i];
    }
    __syncthreads();
    const float* row = e < E ? wr + (size_t)e * W : (e == E ? wsg : nullptr);
    if (row == nullptr) return;
    float acc[ROUTE_TOKENS];
#pragma unroll
    for (int tt = 0; tt < ROUTE_TOKENS; tt++) acc[tt] = 0.f;
    if (vec) {
#pragma unroll 4
        for (int k = lane * 4; k < W; k += 128) {
            const float4 r = __ldg(reinterpret_cast<const float4*>(row + k));
#pragma unroll
            for (int tt = 0; tt < ROUTE_TOKENS; tt++)
                if (tt < nt) {
                    float xv[4];
                    if (sizeof(T) == 2) {
                        const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(xs) + tt * W + k);
                        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
                        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
                        xv[0] = a.x, xv[1] = a.y, xv[2] = b.x, xv[3] = b.y;
                    } else {
                        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(xs) + tt * W + k);
                        xv[0] = a.x, xv[1] = a.y, xv[2] = a.z, xv[3] = a.w;
                    }
                    acc[tt] = fmaf(r.x, xv[0], fmaf(r.y, xv[1], fmaf(r.z, xv[2], fmaf(r.w, xv[3], acc[tt]))));
                }
        }
    } else {
        for (int k = lane; k < W; k += 32)
#pragma unroll
            for (int tt = 0; tt < ROUTE_TOKENS; tt++)
                if (tt < nt) acc[tt] = fmaf(row[k], to_f(xs[tt * W + k]), acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < ROUTE_TOKENS; tt++) {
        if (tt >= nt) continue;
        const float z = warp_sum(acc[tt]);
        if (lane == 0) {
            const float sg = 1.f / (1.f + expf(-z));
            if (e < E) scores[(size_t)(t0 + tt) * E + e] = by_logit ? z : sg;     // the sum itself where the choice goes by it
            else sgate[t0 + tt] = sg;
        }
    }
}

// Choice: a warp a token, from the token's scores.
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_choose_kernel(const float* scores, const float* __restrict__ corr, int E, int top, int groups, int keep, float scale,
                  int* idx, float* wt, int n_tok, int renorm, int by_logit) {
    extern __shared__ __align__(16) unsigned char route_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int t = blockIdx.x * ROUTE_WARPS + w;
    if (t >= n_tok) return;
    float* s = reinterpret_cast<float*>(route_smem) + (size_t)w * 3 * E;
    float* c = s + E;
    float* gs = c + E;
    for (int e = lane; e < E; e += 32) {
        const float v = scores[(size_t)t * E + e];
        if (by_logit) {      // no correction, one group: the largest scores are the largest sums, and two float32 scores that
                             // have both reached 1 still differ in their sums
            s[e] = 1.f / (1.f + expf(-v));
            c[e] = v;
        } else {
            s[e] = v;
            c[e] = v + (corr ? corr[e] : 0.f);
        }
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {       // a group's score: its two largest choice scores
            float a = -INFINITY, b = -INFINITY;
            for (int i = 0; i < per; i++) {
                const float v = c[g * per + i];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the keep best groups are marked by +inf; all others' experts then leave the choice
        for (int it = 0; it < keep; it++) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] != INFINITY && (gs[g] > bv || bi == 0x7fffffff)) { bv = gs[g]; bi = g; }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < groups) gs[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f;
    for (int j = 0; j < top; j++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (c[e] > bv) { bv = c[e]; bi = e; }
        warp_argmax(bv, bi);
        if (bi >= E) bi = 0;                             // nothing left to choose from (more picks than allowed experts)
        wsum += s[bi];
        if (lane == 0) {
            idx[(size_t)t * top + j] = bi;
            c[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane < top) {
        const int e = idx[(size_t)t * top + lane];
        wt[(size_t)t * top + lane] = (renorm ? s[e] / (wsum + 1e-20f) : s[e]) * scale;    // the scores as they are, or over their sum
    }
}

// act 0: silu(g) u; 1: gelu_tanh(g) u; 2: with g' = min(g, limit) and u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1)
__device__ __forceinline__ float moe_gated(float g, float u, int act, float limit) {
    if (act == 2) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
    }
    if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    return g / (1.f + expf(-g)) * u;
}

// 16 bytes of a row as floats: 8 bfloat16 or 4 float32 values
template <typename T> struct Vec;
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void load(const bf16* p, float (&f)[8]) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x, f[2 * i + 1] = x.y;
        }
    }
};
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p));
        f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
    }
};

// Block (pair, slice of ff): mid[pair][f] = act(W_gu[e][f] . x) * (W_gu[e][ff + f] . x), W_gu [E, 2 ff, W]. A warp an
// output: its gate row and its up row streamed 16 bytes a lane at a time (VEC; rows then start on 16-byte
// boundaries), several requests in flight, or element by element for other widths.
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
moe_up_rows_kernel(const T* x, int W, const T* __restrict__ wgu, const int* idx, T* mid, int ff, int top, int rows_per_block,
                   int act, const float* in_wt, float limit) {
    extern __shared__ float xs[];
    pdl_wait();
    pdl_launch_dependents();
    const int pair = blockIdx.x, t = pair / top;
    const int e = idx[pair];
    for (int k = threadIdx.x; k < W; k += blockDim.x) xs[k] = to_f(x[(size_t)t * W + k]);
    __syncthreads();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int f_end = min(ff, (int)(blockIdx.y + 1) * rows_per_block);
    const T* base = wgu + (size_t)e * 2 * ff * W;
    constexpr int N = Vec<T>::N;
    for (int f = blockIdx.y * rows_per_block + w; f < f_end; f += 4) {
        const T* g = base + (size_t)f * W;
        const T* u = base + (size_t)(ff + f) * W;
        float ag = 0.f, au = 0.f;
        if (VEC) {
#pragma unroll 4
            for (int k = lane * N; k < W; k += 32 * N) {
                float gv[N], uv[N], xv[N];
                Vec<T>::load(g + k, gv);
                Vec<T>::load(u + k, uv);
#pragma unroll
                for (int i = 0; i < N; i += 4) *reinterpret_cast<float4*>(xv + i) = *reinterpret_cast<const float4*>(xs + k + i);
#pragma unroll
                for (int i = 0; i < N; i++) {
                    ag = fmaf(gv[i], xv[i], ag);
                    au = fmaf(uv[i], xv[i], au);
                }
            }
        } else {
            for (int k = lane; k < W; k += 32) {
                ag = fmaf(to_f(g[k]), xs[k], ag);
                au = fmaf(to_f(u[k]), xs[k], au);
            }
        }
        ag = warp_sum(ag);
        au = warp_sum(au);
        if (in_wt != nullptr) {      // the pair's weight on the expert's input: W (w x) = w (W x)
            ag *= in_wt[pair];
            au *= in_wt[pair];
        }
        if (lane == 0) mid[(size_t)pair * ff + f] = from_f<T>(moe_gated(ag, au, act, limit));
    }
}

// Block (token, slice of the width): out[t][c] = sum_j wt[t][j] (W_d[e_j][c] . mid[t*top + j]) + sgate[t] * shared[t][c].
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
moe_down_rows_kernel(const T* mid, const T* __restrict__ wd, const int* idx, const float* wt, const T* shared,
                     const float* sgate, T* out, int W, int ff, int top, int rows_per_block) {
    extern __shared__ float ms[];        // [top][ff], already times the pair's weight
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x)
        ms[i] = to_f(mid[(size_t)t * top * ff + i]) * (wt != nullptr ? wt[(size_t)t * top + i / ff] : 1.f);
    __syncthreads();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c_end = min(W, (int)(blockIdx.y + 1) * rows_per_block);
    constexpr int N = Vec<T>::N;
    for (int c = blockIdx.y * rows_per_block + w; c < c_end; c += 4) {
        float acc = 0.f;
        for (int j = 0; j < top; j++) {
            const T* row = wd + ((size_t)idx[(size_t)t * top + j] * W + c) * ff;
            float a = 0.f;
            if (VEC) {
#pragma unroll 4
                for (int k = lane * N; k < ff; k += 32 * N) {
                    float rv[N], mv[N];
                    Vec<T>::load(row + k, rv);
#pragma unroll
                    for (int i = 0; i < N; i += 4) *reinterpret_cast<float4*>(mv + i) = *reinterpret_cast<const float4*>(ms + j * ff + k + i);
#pragma unroll
                    for (int i = 0; i < N; i++) a = fmaf(rv[i], mv[i], a);
                }
            } else {
                for (int k = lane; k < ff; k += 32) a = fmaf(to_f(row[k]), ms[j * ff + k], a);
            }
            acc += a;
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (shared != nullptr) acc = fmaf(sgate ? sgate[t] : 1.f, to_f(shared[(size_t)t * W + c]), acc);
            out[(size_t)t * W + c] = from_f<T>(acc);
        }
    }
}

template <typename T>
static int launch_scores(const void* x, int W, const float* wr, const float* wsg, int E, float* scores, float* sgate, int n_tok,
                         int by_logit, cudaStream_t st) {
    const size_t smem = sizeof(T) * (size_t)ROUTE_TOKENS * W;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_scores_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int rows = E + (wsg != nullptr ? 1 : 0);
    return dk_launch(moe_scores_kernel<T>, dim3((n_tok + ROUTE_TOKENS - 1) / ROUTE_TOKENS, (rows + ROUTE_WARPS - 1) / ROUTE_WARPS),
                     dim3(32 * ROUTE_WARPS), smem, st, (const T*)x, W, wr, wsg, E, scores, sgate, n_tok, by_logit);
}

// scores: float32 scratch [n_tok, E]
DK_EXPORT int dk_moe_route(int dtype, const void* x, int W, const float* wr, const float* corr, const float* wsg, int E,
                           int top, int groups, int keep, float scale, int* idx, float* wt, float* sgate, float* scores, int n_tok,
                           int renorm, cudaStream_t st) {
    if (E < 1 || E > MOE_MAX_EXPERTS || top < 1 || top > 32 || top > E || groups < 1 || E % groups || keep < 1 || keep > groups ||
        scores == nullptr || (sizeof(float) * ROUTE_TOKENS * W > 200 * 1024))
        return (int)cudaErrorInvalidValue;
    const int by_logit = corr == nullptr && groups == 1;
    int e = dtype == 0 ? launch_scores<float>(x, W, wr, wsg, E, scores, sgate, n_tok, by_logit, st)
                       : launch_scores<bf16>(x, W, wr, wsg, E, scores, sgate, n_tok, by_logit, st);
    if (e) return e;
    const size_t smem = sizeof(float) * 3 * (size_t)E * ROUTE_WARPS;
    return dk_launch(moe_choose_kernel, dim3((n_tok + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(32 * ROUTE_WARPS), smem, st, scores, corr,
                     E, top, groups, keep, scale, idx, wt, n_tok, renorm, by_logit);
}

template <typename T, bool VEC>
static int launch_up(const void* x, int W, const void* wgu, const int* idx, void* mid, int ff, int top, int n_tok, int act,
                     const float* in_wt, float limit, cudaStream_t st) {
    const int rpb = 16;
    const dim3 grid(n_tok * top, (ff + rpb - 1) / rpb), block(128);
    const size_t smem = sizeof(float) * (size_t)W;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_rows_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return dk_launch(moe_up_rows_kernel<T, VEC>, grid, block, smem, st, (const T*)x, W, (const T*)wgu, idx, (T*)mid, ff, top, rpb, act,
                     in_wt, limit);
}

template <typename T, bool VEC>
static int launch_down(const void* mid, const void* wd, const int* idx, const float* wt, const void* shared, const float* sgate,
                       void* out, int W, int ff, int top, int n_tok, cudaStream_t st) {
    const int rpb = 16;
    const dim3 grid(n_tok, (W + rpb - 1) / rpb), block(128);
    const size_t smem = sizeof(float) * (size_t)top * ff;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_rows_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return dk_launch(moe_down_rows_kernel<T, VEC>, grid, block, smem, st, (const T*)mid, (const T*)wd, idx, wt, (const T*)shared,
                     sgate, (T*)out, W, ff, top, rpb);
}

DK_EXPORT int dk_moe_up_rows(int dtype, const void* x, int W, const void* wgu, const int* idx, void* mid, int ff, int top,
                             int n_tok, int act, const float* in_wt, float limit, cudaStream_t st) {
    const bool vec = (uintptr_t)wgu % 16 == 0 && W % (dtype == 0 ? 4 : 8) == 0;
    if (dtype == 0)
        return vec ? launch_up<float, true>(x, W, wgu, idx, mid, ff, top, n_tok, act, in_wt, limit, st)
                   : launch_up<float, false>(x, W, wgu, idx, mid, ff, top, n_tok, act, in_wt, limit, st);
    return vec ? launch_up<bf16, true>(x, W, wgu, idx, mid, ff, top, n_tok, act, in_wt, limit, st)
               : launch_up<bf16, false>(x, W, wgu, idx, mid, ff, top, n_tok, act, in_wt, limit, st);
}

DK_EXPORT int dk_moe_down_rows(int dtype, const void* mid, const void* wd, const int* idx, const float* wt,
                               const void* shared, const float* sgate, void* out, int W, int ff, int top, int n_tok,
                               cudaStream_t st) {
    const bool vec = (uintptr_t)wd % 16 == 0 && ff % (dtype == 0 ? 4 : 8) == 0;
    if (dtype == 0)
        return vec ? launch_down<float, true>(mid, wd, idx, wt, shared, sgate, out, W, ff, top, n_tok, st)
                   : launch_down<float, false>(mid, wd, idx, wt, shared, sgate, out, W, ff, top, n_tok, st);
    return vec ? launch_down<bf16, true>(mid, wd, idx, wt, shared, sgate, out, W, ff, top, n_tok, st)
               : launch_down<bf16, false>(mid, wd, idx, wt, shared, sgate, out, W, ff, top, n_tok, st);
}
