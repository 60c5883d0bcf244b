// Row kernels around RMS norms that work on equal consecutive parts of a row, float32 arithmetic:
//   * add_group_rmsnorm: h += delta; a = w * (each of ``groups`` parts of h over its own root mean square). The residual
//     stream h is float32; delta comes as a tensor in the storage type or as float32 split-K partial sums; with
//     ``rows`` the kernel gathers those rows and leaves h alone (the final norm at the wanted places).
//   * gate_group_norm: y = (o + skip_h * x) * silu(z), then the grouped norm times w, times a constant: the output
//     side of a state-space mixer (the gate comes before the norm).
//   * diff_combine: per head o = a1 - lambda * a2, then o over its root mean square (no weight), times a constant:
//     the output side of differential attention, whose two maps come as neighbouring heads.
// eps stands inside the root everywhere.
#include "common.cuh"

#define GN_THREADS 256
#define GN_WARPS (GN_THREADS / 32)

// Sum of squares of each part, in a fixed order: warp w of a part's ``wpg`` warps takes every wpg-th run of 32
// columns; the warps' sums meet in shared memory and are added in the order of the warps. With more parts than
// warps a warp takes several parts one after the other.
template <typename F>
__device__ __forceinline__ void group_scales(F value, int n, int groups, float eps, float* part_sums, float* scales) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gs = n / groups;
    if (groups >= GN_WARPS) {
        for (int g = warp; g < groups; g += GN_WARPS) {
            float ss = 0.f;
            for (int i = lane; i < gs; i += 32) {
                const float v = value(g * gs + i);
                ss += v * v;
            }
            ss = warp_sum(ss);
            if (lane == 0) scales[g] = 1.f / sqrtf(ss / (float)gs + eps);
        }
        __syncthreads();
        return;
    }
    const int wpg = GN_WARPS / groups;                 // warps that share a part
    const int g = warp / wpg, k = warp % wpg;
    float ss = 0.f;
    if (g < groups)
        for (int i = k * 32 + lane; i < gs; i += 32 * wpg) {
            const float v = value(g * gs + i);
            ss += v * v;
        }
    ss = warp_sum(ss);
    if (lane == 0) part_sums[warp] = ss;
    __syncthreads();
    if (threadIdx.x < groups) {
        float t = 0.f;
        for (int i = 0; i < wpg; i++) t += part_sums[threadIdx.x * wpg + i];
        scales[threadIdx.x] = 1.f / sqrtf(t / (float)gs + eps);
    }
    __syncthreads();
}

__device__ __forceinline__ float4 gn_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 gn_ld4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void gn_st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void gn_st4(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = o;
}

// VEC: four columns a thread at a time (the row's and a part's size are multiples of 4, rows on 16-byte boundaries)
template <typename T, bool VEC>
__global__ void __launch_bounds__(GN_THREADS)
add_group_rmsnorm_kernel(float* h, const T* delta, const float* parts, int n_parts, size_t part_stride, const int* rows,
                         const float* __restrict__ w, float eps, int H, int groups, T* a) {
    extern __shared__ __align__(16) float gn_smem[];       // [H] the row as it stands after the sum, then [groups] scales
    __shared__ float part_sums[GN_WARPS];
    float* vals = gn_smem;
    float* scales = gn_smem + H;
    pdl_wait();
    pdl_launch_dependents();
    const size_t out_row = blockIdx.x;
    const size_t row = rows ? (size_t)rows[out_row] : out_row;
    float* hr = h + row * H;
    const T* dr = delta ? delta + row * H : nullptr;
    if (VEC) {
        for (int i = 4 * threadIdx.x; i < H; i += 4 * GN_THREADS) {
            float4 v = gn_ld4(hr + i);
            if (dr) {
                const float4 d = gn_ld4(dr + i);
                v.x += d.x, v.y += d.y, v.z += d.z, v.w += d.w;
            }
            if (parts) {
                float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int k = 0; k < n_parts; k++) {
                    const float4 u = gn_ld4(parts + (size_t)k * part_stride + row * H + i);
                    d.x += u.x, d.y += u.y, d.z += u.z, d.w += u.w;
                }
                v.x += d.x, v.y += d.y, v.z += d.z, v.w += d.w;
            }
            gn_st4(vals + i, v);
            if (!rows && (dr || parts)) gn_st4(hr + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += GN_THREADS) {
            float v = hr[i];
            if (dr) v += to_f(dr[i]);
            if (parts) {
                float d = 0.f;
                for (int k = 0; k < n_parts; k++) d += parts[(size_t)k * part_stride + row * H + i];
                v += d;
            }
            vals[i] = v;
            if (!rows && (dr || parts)) hr[i] = v;
        }
    }
    __syncthreads();
    group_scales([&](int i) { return vals[i]; }, H, groups, eps, part_sums, scales);
    const int gs = H / groups;
    T* ar = a + out_row * H;
    if (VEC) {
        for (int i = 4 * threadIdx.x; i < H; i += 4 * GN_THREADS) {
            const float4 v = gn_ld4(vals + i), ww = gn_ld4(w + i);
            const float sc = scales[i / gs];
            gn_st4(ar + i, make_float4(v.x * sc * ww.x, v.y * sc * ww.y, v.z * sc * ww.z, v.w * sc * ww.w));
        }
    } else {
        for (int i = threadIdx.x; i < H; i += GN_THREADS) ar[i] = from_f<T>(vals[i] * scales[i / gs] * w[i]);
    }
}

template <typename T>
__global__ void __launch_bounds__(GN_THREADS)
gate_group_norm_kernel(const float* o, const float* x, long long ldx, const float* __restrict__ skip, int hdv, const T* z, long long ldz,
                       const float* __restrict__ w, float eps, float out_scale, T* out, long long ldo, int n, int groups) {
    extern __shared__ float gn_smem[];
    __shared__ float part_sums[GN_WARPS];
    float* vals = gn_smem;
    float* scales = gn_smem + n;
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < n; i += GN_THREADS) {
        float v = o[t * n + i];
        if (skip != nullptr) v = fmaf(skip[i / hdv], x[t * ldx + i], v);
        const float g = to_f(z[t * ldz + i]);
        vals[i] = v * (g / (1.f + expf(-g)));
    }
    __syncthreads();
    group_scales([&](int i) { return vals[i]; }, n, groups, eps, part_sums, scales);
    const int gs = n / groups;
    for (int i = threadIdx.x; i < n; i += GN_THREADS) out[t * ldo + i] = from_f<T>(vals[i] * scales[i / gs] * w[i] * out_scale);
}

// a [T, 2 * nh * hdv]: head 2h holds map 1 of head h, head 2h + 1 map 2. A warp per (token, head).
template <typename T>
__global__ void diff_combine_kernel(const T* a, long long lda, float lambda, float eps, float out_scale, T* out, long long ldo,
                                    int n_tok, int nh, int hdv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (long long)n_tok * nh) return;
    const size_t t = (size_t)(wid / nh);
    const int h = (int)(wid % nh);
    const T* a1 = a + t * lda + (size_t)(2 * h) * hdv;
    const T* a2 = a1 + hdv;
    float v[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        v[i] = d < hdv ? to_f(a1[d]) - lambda * to_f(a2[d]) : 0.f;
        ss += v[i] * v[i];
    }
    const float rs = out_scale / sqrtf(warp_sum(ss) / (float)hdv + eps);
    T* o = out + t * ldo + (size_t)h * hdv;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        if (d < hdv) o[d] = from_f<T>(v[i] * rs);
    }
}

DK_EXPORT int dk_add_group_rmsnorm(int dtype, float* h, const void* delta, const float* parts, int n_parts,
                                   long long part_stride, const int* rows, const float* w, float eps, int n_rows, int H,
                                   int groups, void* a, cudaStream_t st) {
    if (groups < 1 || H % groups) return (int)cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * (size_t)(H + groups);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const bool vec = H % 4 == 0 && (H / groups) % 4 == 0 && part_stride % 4 == 0 &&
                     ((uintptr_t)h | (uintptr_t)delta | (uintptr_t)parts | (uintptr_t)w | (uintptr_t)a) % 16 == 0;
#define GN_LAUNCH(T, V)                                                                                                       \
    {                                                                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_group_rmsnorm_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return dk_launch(add_group_rmsnorm_kernel<T, V>, dim3(n_rows), dim3(GN_THREADS), smem, st, h, (const T*)delta, parts, n_parts, \
                         (size_t)part_stride, rows, w, eps, H, groups, (T*)a);                                                \
    }
    if (dtype == 0) {
        if (vec) GN_LAUNCH(float, true)
        GN_LAUNCH(float, false)
    }
    if (vec) GN_LAUNCH(bf16, true)
    GN_LAUNCH(bf16, false)
#undef GN_LAUNCH
}

DK_EXPORT int dk_gate_group_norm(int dtype, const float* o, const float* x, long long ldx, const float* skip, int hdv, const void* z,
                                 long long ldz, const float* w, float eps, float out_scale, void* out, long long ldo,
                                 int n_tok, int n, int groups, cudaStream_t st) {
    if (groups < 1 || n % groups || hdv < 1 || n % hdv) return (int)cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * (size_t)(n + groups);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(gate_group_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return dk_launch(gate_group_norm_kernel<float>, dim3(n_tok), dim3(GN_THREADS), smem, st, o, x, ldx, skip, hdv, (const float*)z,
                         ldz, w, eps, out_scale, (float*)out, ldo, n, groups);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(gate_group_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return dk_launch(gate_group_norm_kernel<bf16>, dim3(n_tok), dim3(GN_THREADS), smem, st, o, x, ldx, skip, hdv, (const bf16*)z, ldz, w,
                     eps, out_scale, (bf16*)out, ldo, n, groups);
}

DK_EXPORT int dk_diff_combine(int dtype, const void* a, long long lda, float lambda, float eps, float out_scale, void* out,
                              long long ldo, int n_tok, int nh, int hdv, cudaStream_t st) {
    if (hdv < 1 || hdv > 256) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)n_tok * nh;
    const dim3 grid((unsigned)((warps + 3) / 4)), block(128);
    if (dtype == 0)
        return dk_launch(diff_combine_kernel<float>, grid, block, 0, st, (const float*)a, lda, lambda, eps, out_scale,
                         (float*)out, ldo, n_tok, nh, hdv);
    return dk_launch(diff_combine_kernel<bf16>, grid, block, 0, st, (const bf16*)a, lda, lambda, eps, out_scale, (bf16*)out,
                     ldo, n_tok, nh, hdv);
}
