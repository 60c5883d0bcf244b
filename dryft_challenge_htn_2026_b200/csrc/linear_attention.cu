// Linear attention with a constant decay per head ("lightning attention"):
//   S_t = d_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   q, k, v = act(projection rows)
// with the state S [hd, hdv] of every (sequence, head) kept in float32 between steps, and the
// norm-and-gate step that follows it: all heads of a token together through a weighted RMS norm, times
// sigmoid(gate), times a constant. State, decay powers, scores and sums are float32; the projections
// come in the model's storage type and their activation is worked out in float32.
//
// The same kernel also runs gated linear attention: a decay per key channel and token instead of one per
// head, alpha_t = sigmoid(z_t + b)^(1/tau) from rows z of a low-rank projection, acting on the rows of
// the state, S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, with q times a constant and no activation. The
// decay is worked out in float32 as exp(log sigmoid(z) / tau).
//
// This file: the recurrence token by token, one block per (sequence, head), the state in registers; it
// serves single-token steps, short portions and every float32 step. Portions of many tokens in bfloat16
// run in blocks of 64 tokens on the tensor cores (linear_attention_bf16.cu).
#include "common.cuh"
#include <type_traits>

#define LA_THREADS 256
#define LA_TB 8   // tokens staged at a time by the step kernel

__device__ __forceinline__ float act_silu(float x) { return x / (1.f + expf(-x)); }

// Block (sequence s, head h, slice of up to cslice value columns: the columns of a state evolve independently,
// and a slice of 32 keeps a thread's share of the state at hd / 8 registers, so that several blocks fit an
// SM). Thread (rg, c): column c of the slice, rows rg, rg + R, ... (R row groups).
// cu_q == nullptr: one token per sequence (row s is sequence s). seq_pos0[s] < 0: a padding row.
// GATED: ``zrows`` [tokens, nh * hd] float32 and ``zbias`` [nh * hd] give the decay of every state row and token,
// exp(log sigmoid(z + b) * inv_tau); q is multiplied by q_scale and nothing goes through SiLU.
template <typename T, int EPT, bool GATED>
__global__ void __launch_bounds__(LA_THREADS)
linear_attention_step_kernel(const T* q, const T* k, const T* v, long long ld, float* out, float* state,
                             const int* cu_q, const int* seq_pos0, const int* seq_slot, const float* __restrict__ decay,
                             int nh, int hd, int hdv, int cols_pad, int cslice, const float* zrows,
                             const float* __restrict__ zbias, float inv_tau, float q_scale) {
    extern __shared__ float sm[];
    const int R = LA_THREADS / cols_pad;
    float* sq = sm;                              // [LA_TB][hd]
    float* sk = sq + LA_TB * hd;                 // [LA_TB][hd]
    float* sv = sk + LA_TB * hd;                 // [LA_TB][cslice]
    float* part = sv + LA_TB * cslice;           // [LA_TB][R][cols_pad]
    float* sd = part + LA_TB * LA_THREADS;       // [LA_TB][hd], GATED only
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cslice;
    const int cols = min(cslice, hdv - col0);            // value columns of this block: [col0, col0 + cols)
    const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
    const int tid = threadIdx.x, c = tid % cols_pad, rg = tid / cols_pad;
    const size_t ow = (size_t)nh * hdv;
    if (seq_pos0[s] < 0) {
        for (int t = r0; t < r1; t++)
            for (int i = tid; i < cols; i += LA_THREADS) out[(size_t)t * ow + (size_t)h * hdv + col0 + i] = 0.f;
        return;
    }
    const float d = GATED ? 0.f : decay[h];
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)hd * hdv + col0;
    float st[EPT];
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        const int row = rg + R * i;
        st[i] = (row < hd && c < cols) ? S[(size_t)row * hdv + c] : 0.f;
    }
    for (int t0 = r0; t0 < r1; t0 += LA_TB) {
        const int nt = min(LA_TB, r1 - t0);
        __syncthreads();
        for (int i = tid; i < nt * hd; i += LA_THREADS) {
            const size_t at = (size_t)(t0 + i / hd) * ld + (size_t)h * hd + i % hd;
            if (GATED) {
                sq[i] = to_f(q[at]) * q_scale;
                sk[i] = to_f(k[at]);
                const float z = zrows[(size_t)(t0 + i / hd) * nh * hd + (size_t)h * hd + i % hd] + zbias[h * hd + i % hd];
                sd[i] = expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau);   // sigmoid(z)^(1/tau)
            } else {
                sq[i] = act_silu(to_f(q[at]));
                sk[i] = act_silu(to_f(k[at]));
            }
        }
        for (int i = tid; i < nt * cols; i += LA_THREADS) {
            const float x = to_f(v[(size_t)(t0 + i / cols) * ld + (size_t)h * hdv + col0 + i % cols]);
            sv[i] = GATED ? x : act_silu(x);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float vc = c < cols ? sv[tt * cols + c] : 0.f;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < EPT; i++) {
                const int row = rg + R * i;
                if (row < hd) {
                    st[i] = fmaf(GATED ? sd[tt * hd + row] : d, st[i], sk[tt * hd + row] * vc);
                    o = fmaf(st[i], sq[tt * hd + row], o);
                }
            }
            part[(tt * R + rg) * cols_pad + c] = o;
        }
        __syncthreads();
        for (int i = tid; i < nt * cols; i += LA_THREADS) {
            const int tt = i / cols, cc = i % cols;
            float o = 0.f;
            for (int g = 0; g < R; g++) o += part[(tt * R + g) * cols_pad + cc];
            out[(size_t)(t0 + tt) * ow + (size_t)h * hdv + col0 + cc] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        const int row = rg + R * i;
        if (row < hd && c < cols) S[(size_t)row * hdv + c] = st[i];
    }
}

// ---------------------------------------------------------------------------------------------
// Gated linear attention, a warp per (sequence, head, 8 value columns): lane l keeps the state rows of key channels
// DPL * l .. DPL * l + DPL - 1 (DPL = hd / 32) for its 8 columns in registers, DPL * 8 numbers. A token costs the
// warp DPL * 16 multiply-adds and 9 shuffles (the 8 column sums over the lanes are folded by halves: 4, 2, 1
// exchanges, then two more on the one value left), no shared memory and no barrier; the state's own chain is one
// multiply-add a token, the loads of later tokens do not wait for it. The decays come as float32 rows
// (gla_decay_kernel makes them from the projection's rows, once for all column groups).
template <int N> __device__ __forceinline__ void ld_vec(const float* p, float (&f)[N], bool vec) {
    if (vec && N == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
    } else if (vec && N == 8) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < N; i++) f[i] = p[i];
    }
}
template <int N> __device__ __forceinline__ void ld_vec(const bf16* p, float (&f)[N], bool vec) {
    if (vec && N == 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x, f[2 * i + 1] = x.y;
        }
    } else if (vec && N == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x, f[2 * i + 1] = x.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; i++) f[i] = __bfloat162float(p[i]);
    }
}

// alpha = sigmoid(z + b)^(1/tau) = exp(log sigmoid(z + b) / tau), in place over the float32 rows z [rows, n]
__global__ void gla_decay_kernel(float* z, const float* __restrict__ bias, float inv_tau, size_t total, int n) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float x = z[i] + bias[i % n];
    z[i] = expf((fminf(x, 0.f) - log1pf(expf(-fabsf(x)))) * inv_tau);
}

template <typename T, int DPL>
__global__ void __launch_bounds__(128)
gla_warp_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                const float* __restrict__ alpha, float* __restrict__ out, float* state, const int* cu_q, const int* seq_pos0,
                const int* seq_slot, int nh, int hdv, float q_scale, int vec) {
    constexpr int HDK = 32 * DPL;
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = blockIdx.x, h = blockIdx.y;
    const int c0 = (blockIdx.z * 4 + warp) * 8;
    if (c0 >= hdv) return;
    const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
    const size_t ow = (size_t)nh * hdv;
    // after the folds lane l holds the sum of column 4 * bit4 + 2 * bit3 + bit2 of its number
    const int my_col = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if (seq_pos0[s] < 0) {        // a padding row: zeros out, state untouched
        if ((lane & 3) == 0)
            for (int t = r0; t < r1; t++) out[(size_t)t * ow + (size_t)h * hdv + c0 + my_col] = 0.f;
        return;
    }
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)HDK * hdv + (size_t)(DPL * lane) * hdv + c0;
    float st[DPL][8];
#pragma unroll
    for (int i = 0; i < DPL; i++) ld_vec<8>(S + (size_t)i * hdv, st[i], true);
    const size_t qk_at = (size_t)h * HDK + DPL * lane, v_at = (size_t)h * hdv + c0;
    const bool hi16 = lane & 16, hi8 = lane & 8, hi4 = lane & 4;
#pragma unroll 2
    for (int t = r0; t < r1; t++) {
        float qv[DPL], kv[DPL], av[DPL], vv[8];
        ld_vec<DPL>(q + (size_t)t * ld + qk_at, qv, vec);
        ld_vec<DPL>(k + (size_t)t * ld + qk_at, kv, vec);
        ld_vec<DPL>(alpha + (size_t)t * nh * HDK + qk_at, av, vec);
        ld_vec<8>(v + (size_t)t * ld + v_at, vv, vec);
        float o[8];
#pragma unroll
        for (int c = 0; c < 8; c++) o[c] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            const float qs = qv[i] * q_scale;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                st[i][c] = fmaf(av[i], st[i][c], kv[i] * vv[c]);
                o[c] = fmaf(st[i][c], qs, o[c]);
            }
        }
        float r4[4], r2[2], r;
#pragma unroll
        for (int c = 0; c < 4; c++) r4[c] = (hi16 ? o[4 + c] : o[c]) + __shfl_xor_sync(0xffffffffu, hi16 ? o[c] : o[4 + c], 16);
#pragma unroll
        for (int c = 0; c < 2; c++) r2[c] = (hi8 ? r4[2 + c] : r4[c]) + __shfl_xor_sync(0xffffffffu, hi8 ? r4[c] : r4[2 + c], 8);
        r = (hi4 ? r2[1] : r2[0]) + __shfl_xor_sync(0xffffffffu, hi4 ? r2[0] : r2[1], 4);
        r += __shfl_xor_sync(0xffffffffu, r, 2);
        r += __shfl_xor_sync(0xffffffffu, r, 1);
        if ((lane & 3) == 0) out[(size_t)t * ow + v_at + my_col] = r;
    }
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        *reinterpret_cast<float4*>(S + (size_t)i * hdv) = make_float4(st[i][0], st[i][1], st[i][2], st[i][3]);
        *reinterpret_cast<float4*>(S + (size_t)i * hdv + 4) = make_float4(st[i][4], st[i][5], st[i][6], st[i][7]);
    }
}

// The same with the rows staged: the block's warps share a head, so its q, k and decay rows (and the block's value
// columns) of 16 tokens at a time come into shared memory by cp.async, up to four stages in turn, and the warps read
// them from there: the loads of the next chunks run under the arithmetic of this one. A warp takes VC = 8, 4 or 2 value
// columns and a block BC = 32 or 16 of them: a single sequence of few heads is cut fine, so that every scheduler of
// every SM has a warp or two (one warp alone waits out every shuffle of its folds). Rows on 16-byte boundaries.
#define GLA_NT 16
__device__ __forceinline__ void gla_cp16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
// the VC column sums of the 32 lanes: halves are exchanged while more than one value is left, then plain sums; lane l
// ends with the sum of the column whose number is spelled by its top log2(VC) bits
template <int VC> __device__ __forceinline__ float fold_columns(const float (&o)[VC], int lane) {
    float r;
    if (VC == 8) {
        const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
        float r4[4], r2[2];
#pragma unroll
        for (int c = 0; c < 4; c++) r4[c] = (h16 ? o[(4 + c) % VC] : o[c % VC]) + __shfl_xor_sync(0xffffffffu, h16 ? o[c % VC] : o[(4 + c) % VC], 16);
#pragma unroll
        for (int c = 0; c < 2; c++) r2[c] = (h8 ? r4[2 + c] : r4[c]) + __shfl_xor_sync(0xffffffffu, h8 ? r4[c] : r4[2 + c], 8);
        r = (h4 ? r2[1] : r2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? r2[0] : r2[1], 4);
    } else if (VC == 4) {
        const bool h16 = lane & 16, h8 = lane & 8;
        float r2[2];
#pragma unroll
        for (int c = 0; c < 2; c++) r2[c] = (h16 ? o[(2 + c) % VC] : o[c % VC]) + __shfl_xor_sync(0xffffffffu, h16 ? o[c % VC] : o[(2 + c) % VC], 16);
        r = (h8 ? r2[1] : r2[0]) + __shfl_xor_sync(0xffffffffu, h8 ? r2[0] : r2[1], 8);
        r += __shfl_xor_sync(0xffffffffu, r, 4);
    } else {
        const bool h16 = lane & 16;
        r = (h16 ? o[1 % VC] : o[0]) + __shfl_xor_sync(0xffffffffu, h16 ? o[0] : o[1 % VC], 16);
        r += __shfl_xor_sync(0xffffffffu, r, 8);
        r += __shfl_xor_sync(0xffffffffu, r, 4);
    }
    r += __shfl_xor_sync(0xffffffffu, r, 2);
    r += __shfl_xor_sync(0xffffffffu, r, 1);
    return r;
}
template <typename T, int DPL, int VC>
__global__ void __launch_bounds__(512)
gla_warp_staged_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                       const float* __restrict__ alpha, float* __restrict__ out, float* state, const int* cu_q,
                       const int* seq_pos0, const int* seq_slot, int nh, int hdv, float q_scale, int BC, int n_stages) {
    constexpr int HDK = 32 * DPL;
    constexpr int QB = GLA_NT * HDK * (int)sizeof(T), AB = GLA_NT * HDK * 4, VB = GLA_NT * 32 * (int)sizeof(T);
    constexpr int STAGE = 2 * QB + AB + VB;
    constexpr int WRITERS = 32 / VC;                  // every WRITERS-th lane holds a column's sum
    extern __shared__ __align__(16) unsigned char gla_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, threads = blockDim.x;
    const int s = blockIdx.x, h = blockIdx.y;
    const int col0 = blockIdx.z * BC, c0 = col0 + warp * VC;
    const bool active = c0 < hdv;
    const int cols_here = min(BC, hdv - col0);
    const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
    const size_t ow = (size_t)nh * hdv;
    const int my_col = lane / WRITERS;
    if (seq_pos0[s] < 0) {
        if (active && lane % WRITERS == 0)
            for (int t = r0; t < r1; t++) out[(size_t)t * ow + (size_t)h * hdv + c0 + my_col] = 0.f;
        return;
    }
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)HDK * hdv + (size_t)(DPL * lane) * hdv + c0;
    float st[DPL][VC];
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        if (active) ld_vec<VC>(S + (size_t)i * hdv, st[i], VC >= 4);
        else
#pragma unroll
            for (int c = 0; c < VC; c++) st[i][c] = 0.f;
    }
    const int n_chunks = (r1 - r0 + GLA_NT - 1) / GLA_NT;
    constexpr int QP = HDK * (int)sizeof(T) / 16, AP = HDK * 4 / 16;         // 16-byte pieces a token
    const int VP = cols_here * (int)sizeof(T) / 16;
    auto issue = [&](int c) {
        if (c < n_chunks) {
            unsigned char* base = gla_smem + (c % n_stages) * STAGE;
            const int t0 = r0 + c * GLA_NT, nt = min(GLA_NT, r1 - t0);
            for (int i = tid; i < nt * QP; i += threads) {
                const int tt = i / QP, pc = i % QP;
                const size_t src = ((size_t)(t0 + tt) * ld + (size_t)h * HDK) * sizeof(T) + pc * 16;
                gla_cp16(base + tt * (HDK * sizeof(T)) + pc * 16, reinterpret_cast<const unsigned char*>(q) + src);
                gla_cp16(base + QB + tt * (HDK * sizeof(T)) + pc * 16, reinterpret_cast<const unsigned char*>(k) + src);
            }
            for (int i = tid; i < nt * AP; i += threads) {
                const int tt = i / AP, pc = i % AP;
                gla_cp16(base + 2 * QB + tt * (HDK * 4) + pc * 16,
                         reinterpret_cast<const unsigned char*>(alpha + (size_t)(t0 + tt) * nh * HDK + (size_t)h * HDK) + pc * 16);
            }
            for (int i = tid; i < nt * VP; i += threads) {
                const int tt = i / VP, pc = i % VP;
                gla_cp16(base + 2 * QB + AB + tt * (32 * sizeof(T)) + pc * 16,
                         reinterpret_cast<const unsigned char*>(v + (size_t)(t0 + tt) * ld + (size_t)h * hdv + col0) + pc * 16);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // n_stages - 1 chunks ahead: a chunk's arithmetic is shorter than a trip to memory (with one chunk ahead every
    // chunk waited out that trip: 3 us for 16 tokens, whatever the warps did)
    for (int c = 0; c < n_stages - 1; c++) issue(c);
    for (int c = 0; c < n_chunks; c++) {
        issue(c + n_stages - 1);
        if (n_stages == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
        else if (n_stages == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
        else asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const unsigned char* base = gla_smem + (c % n_stages) * STAGE;
        const T* sq = reinterpret_cast<const T*>(base);
        const T* sk = reinterpret_cast<const T*>(base + QB);
        const float* sa = reinterpret_cast<const float*>(base + 2 * QB);
        const T* sv = reinterpret_cast<const T*>(base + 2 * QB + AB);
        const int t0 = r0 + c * GLA_NT, nt = min(GLA_NT, r1 - t0);
        if (active) {
            // U tokens a turn: their state updates follow one another (one multiply-add each), their folds are
            // independent chains of five shuffles that run side by side (one token at a time, a warp alone on its
            // scheduler waited out every shuffle: the time did not depend on the columns a warp took)
            constexpr int U = DPL * VC <= 16 ? 4 : 2;
            auto turn = [&](int tt0, auto tail_c) {
                constexpr bool TAIL = decltype(tail_c)::value;    // the chunk's last turn may hold fewer than U tokens
                float o[U][VC];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int tt = TAIL ? min(tt0 + u, nt - 1) : tt0 + u;   // past the end: the last token again, its result unused
                    float qv[DPL], kv[DPL], av[DPL], vv[VC];
                    ld_vec<DPL>(sq + tt * HDK + DPL * lane, qv, true);
                    ld_vec<DPL>(sk + tt * HDK + DPL * lane, kv, true);
                    ld_vec<DPL>(sa + tt * HDK + DPL * lane, av, true);
                    ld_vec<VC>(sv + tt * 32 + warp * VC, vv, true);
                    const bool live = !TAIL || tt0 + u < nt;
#pragma unroll
                    for (int cc = 0; cc < VC; cc++) o[u][cc] = 0.f;
#pragma unroll
                    for (int i = 0; i < DPL; i++) {
                        const float qs = qv[i] * q_scale;
#pragma unroll
                        for (int cc = 0; cc < VC; cc++) {
                            const float nx = fmaf(av[i], st[i][cc], kv[i] * vv[cc]);
                            st[i][cc] = live ? nx : st[i][cc];
                            o[u][cc] = fmaf(nx, qs, o[u][cc]);
                        }
                    }
                }
                float r[U];
#pragma unroll
                for (int u = 0; u < U; u++) r[u] = fold_columns<VC>(o[u], lane);
#pragma unroll
                for (int u = 0; u < U; u++)
                    if ((!TAIL || tt0 + u < nt) && lane % WRITERS == 0)
                        out[(size_t)(t0 + tt0 + u) * ow + (size_t)h * hdv + c0 + my_col] = r[u];
            };
            int tt0 = 0;
            for (; tt0 + U <= nt; tt0 += U) turn(tt0, std::false_type{});
            if (tt0 < nt) turn(tt0, std::true_type{});
        }
        __syncthreads();              // the stage is free for the chunk after next
    }
    if (active) {
#pragma unroll
        for (int i = 0; i < DPL; i++)
#pragma unroll
            for (int c = 0; c < VC; c++) S[(size_t)i * hdv + c] = st[i][c];
    }
}

template <typename T>
static int launch_gla_warp(const void* q, const void* k, const void* v, long long ld, const float* alpha, float* out,
                           float* state, const int* cu_q, const int* seq_pos0, const int* seq_slot, int n_seq, int nh, int hd,
                           int hdv, float q_scale, int vec, long long n_tok_max, cudaStream_t st) {
    const dim3 grid(n_seq, nh, (hdv + 31) / 32), block(128);
#define GLA_WARP(D)                                                                                                    \
    if (hd == 32 * D)                                                                                                  \
        return dk_launch(gla_warp_kernel<T, D>, grid, block, 0, st, (const T*)q, (const T*)k, (const T*)v, ld, alpha, out, \
                         state, cu_q, seq_pos0, seq_slot, nh, hdv, q_scale, vec);
    if (vec && n_tok_max > 4) {      // portions: staged rows (single tokens have nothing to run ahead of)
        // columns a warp and a block: coarse when the sequences and heads alone fill the schedulers, finer when not
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long blocks32 = (long long)n_seq * nh * ((hdv + 31) / 32), scheds = 4LL * sms;
        int VCs = 8, BC = 32;
        if (blocks32 * 4 < 3 * scheds) VCs = 4;
        if (blocks32 * 8 < 3 * scheds) { VCs = 2; if (blocks32 < sms) BC = 16; }
        const dim3 sgrid(n_seq, nh, (hdv + BC - 1) / BC), sblock(32 * BC / VCs);
#define GLA_STAGED(D, V)                                                                                                   \
    if (hd == 32 * D && VCs == V) {                                                                                        \
        const size_t stage = 2 * GLA_NT * 32 * D * sizeof(T) + GLA_NT * 32 * D * 4 + GLA_NT * 32 * sizeof(T);              \
        const int n_stages = stage * 4 <= 160 * 1024 ? 4 : (stage * 3 <= 160 * 1024 ? 3 : 2);                              \
        const size_t smem = n_stages * stage;                                                                              \
        if (smem > 48 * 1024)                                                                                              \
            cudaFuncSetAttribute(gla_warp_staged_kernel<T, D, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return dk_launch(gla_warp_staged_kernel<T, D, V>, sgrid, sblock, smem, st, (const T*)q, (const T*)k, (const T*)v,  \
                         ld, alpha, out, state, cu_q, seq_pos0, seq_slot, nh, hdv, q_scale, BC, n_stages);                 \
    }
        GLA_STAGED(1, 8) GLA_STAGED(2, 8) GLA_STAGED(4, 8) GLA_STAGED(8, 8)
        GLA_STAGED(1, 4) GLA_STAGED(2, 4) GLA_STAGED(4, 4) GLA_STAGED(8, 4)
        GLA_STAGED(1, 2) GLA_STAGED(2, 2) GLA_STAGED(4, 2) GLA_STAGED(8, 2)
#undef GLA_STAGED
    }
    GLA_WARP(1) GLA_WARP(2) GLA_WARP(4) GLA_WARP(8)
#undef GLA_WARP
    return (int)cudaErrorInvalidValue;
}

// z [rows, nh * hd] float32 is overwritten by the decays. Head sizes: hd 32, 64, 128 or 256, hdv a multiple of 8.
DK_EXPORT int dk_gated_linear_attention_warp(int dtype, const void* q, const void* k, const void* v, long long ld, float* z,
                                             const float* zbias, float inv_tau, long long n_rows, float* out, float* state,
                                             const int* cu_q, const int* seq_pos0, const int* seq_slot, float q_scale, int n_seq,
                                             int nh, int hd, int hdv, cudaStream_t st) {
    const long long n_tok_max = cu_q ? n_rows : 1;      // the most tokens a sequence can bring: all rows, or one without cu_q
    if (hdv % 8 || hdv > 256 || (hd != 32 && hd != 64 && hd != 128 && hd != 256)) return (int)cudaErrorInvalidValue;
    const size_t total = (size_t)n_rows * nh * hd;
    int e = dk_launch(gla_decay_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, z, zbias, inv_tau, total, nh * hd);
    if (e) return e;
    // whole 16-byte pieces: rows of q, k, v that start on 16-byte boundaries
    const int esz = dtype == 0 ? 4 : 2;
    const int vec = ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 16 == 0 && (ld * esz) % 16 == 0 && (hd * esz) % 16 == 0 &&
                    (hdv * esz) % 16 == 0;
    if (dtype == 0)
        return launch_gla_warp<float>(q, k, v, ld, z, out, state, cu_q, seq_pos0, seq_slot, n_seq, nh, hd, hdv, q_scale, vec, n_tok_max, st);
    return launch_gla_warp<bf16>(q, k, v, ld, z, out, state, cu_q, seq_pos0, seq_slot, n_seq, nh, hd, hdv, q_scale, vec, n_tok_max, st);
}

// The same recurrence with the decays given (float32 [rows, nh * hd]) instead of made from z: for mixers that make their
// own decays, keys and queries (a forget gate with a lower bound, a state-space step). q, k, v of one row stride.
DK_EXPORT int dk_decayed_recurrence_warp(int dtype, const void* q, const void* k, const void* v, long long ld, const float* decay,
                                         long long n_rows, float* out, float* state, const int* cu_q, const int* seq_pos0,
                                         const int* seq_slot, int n_seq, int nh, int hd, int hdv, cudaStream_t st) {
    const long long n_tok_max = cu_q ? n_rows : 1;
    if (hdv % 8 || hdv > 256 || (hd != 32 && hd != 64 && hd != 128 && hd != 256)) return (int)cudaErrorInvalidValue;
    const int esz = dtype == 0 ? 4 : 2;
    const int vec = ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)decay) % 16 == 0 && (ld * esz) % 16 == 0 &&
                    (hd * esz) % 16 == 0 && (hdv * esz) % 16 == 0;
    if (dtype == 0)
        return launch_gla_warp<float>(q, k, v, ld, decay, out, state, cu_q, seq_pos0, seq_slot, n_seq, nh, hd, hdv, 1.f, vec, n_tok_max, st);
    return launch_gla_warp<bf16>(q, k, v, ld, decay, out, state, cu_q, seq_pos0, seq_slot, n_seq, nh, hd, hdv, 1.f, vec, n_tok_max, st);
}

// out[t] = rmsnorm(o[t]) * w * sigmoid(gate[t]) * out_scale, the norm over each group of ``group`` columns of
// the row (the whole row of all heads, width n, or one head at a time with a weight of the head's size,
// shared by the heads); gate_act 1: SiLU of the gate instead of its sigmoid. Block (token, group).
template <typename T>
__global__ void norm_gate_kernel(const float* o, const float* __restrict__ w, float eps, const T* gate, long long ldg,
                                 float out_scale, T* out, long long ldo, int n, int group, int gate_act) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    const int c0 = blockIdx.y * group;
    const float* orow = o + t * n + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) ss += orow[i] * orow[i];
    ss = block_sum(ss, red);
    const float rs = out_scale / sqrtf(ss / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        float v = orow[i] * rs * w[i];
        if (gate) {
            const float g = to_f(gate[t * ldg + c0 + i]);
            v *= (gate_act == 1 ? g : 1.f) / (1.f + expf(-g));
        }
        out[t * ldo + c0 + i] = from_f<T>(v);
    }
}

template <typename T, bool GATED>
static int launch_step(const void* q, const void* k, const void* v, long long ld, float* out, float* state,
                       const int* cu_q, const int* seq_pos0, const int* seq_slot, const float* decay, int n_seq, int nh,
                       int hd, int hdv, cudaStream_t st, const float* zrows = nullptr, const float* zbias = nullptr,
                       float inv_tau = 0.f, float q_scale = 1.f) {
    const int cslice = hdv < 32 ? hdv : 32;
    int cols_pad = 1;
    while (cols_pad < cslice) cols_pad <<= 1;
    const int R = LA_THREADS / cols_pad;
    const int ept = (hd + R - 1) / R;
    const size_t smem = sizeof(float) * (size_t)(LA_TB * ((GATED ? 3 : 2) * hd + cslice) + LA_TB * LA_THREADS);
    const dim3 grid(n_seq, nh, (hdv + cslice - 1) / cslice), block(LA_THREADS);
#define LA_STEP(E)                                                                                                       \
    if (ept <= E) {                                                                                                      \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(linear_attention_step_kernel<T, E, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return dk_launch(linear_attention_step_kernel<T, E, GATED>, grid, block, smem, st, (const T*)q, (const T*)k, (const T*)v, \
                         ld, out, state, cu_q, seq_pos0, seq_slot, decay, nh, hd, hdv, cols_pad, cslice, zrows, zbias,    \
                         inv_tau, q_scale);                                                                              \
    }
    LA_STEP(4) LA_STEP(8) LA_STEP(16) LA_STEP(32) LA_STEP(64) LA_STEP(128) LA_STEP(256)
#undef LA_STEP
    return (int)cudaErrorInvalidValue;
}

DK_EXPORT int dk_linear_attention_step(int dtype, const void* q, const void* k, const void* v, long long ld, float* out,
                                       float* state, const int* cu_q, const int* seq_pos0, const int* seq_slot,
                                       const float* decay, int n_seq, int nh, int hd, int hdv, cudaStream_t st) {
    if (hd > 256 || hdv > 256 || hd < 1 || hdv < 1) return (int)cudaErrorInvalidValue;
    if (dtype == 0)
        return launch_step<float, false>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, nh, hd, hdv, st);
    return launch_step<bf16, false>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, nh, hd, hdv, st);
}

DK_EXPORT int dk_gated_linear_attention_step(int dtype, const void* q, const void* k, const void* v, long long ld,
                                             float* out, float* state, const int* cu_q, const int* seq_pos0,
                                             const int* seq_slot, const float* zrows, const float* zbias, float inv_tau,
                                             float q_scale, int n_seq, int nh, int hd, int hdv, cudaStream_t st) {
    if (hd > 256 || hdv > 256 || hd < 1 || hdv < 1) return (int)cudaErrorInvalidValue;
    if (dtype == 0)
        return launch_step<float, true>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, nullptr, n_seq, nh, hd, hdv,
                                        st, zrows, zbias, inv_tau, q_scale);
    return launch_step<bf16, true>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, nullptr, n_seq, nh, hd, hdv, st,
                                   zrows, zbias, inv_tau, q_scale);
}

DK_EXPORT int dk_norm_gate(int dtype, const float* o, const float* w, float eps, const void* gate, long long ldg,
                           float out_scale, void* out, long long ldo, int n_tok, int n, int group, int gate_act,
                           cudaStream_t st) {
    if (group < 1 || n % group) return (int)cudaErrorInvalidValue;
    const int threads = group >= 2048 ? 512 : (group >= 512 ? 256 : (group >= 128 ? 128 : (group > 32 ? 64 : 32)));
    const dim3 grid(n_tok, n / group);
    if (dtype == 0)
        return dk_launch(norm_gate_kernel<float>, grid, dim3(threads), 0, st, o, w, eps, (const float*)gate, ldg,
                         out_scale, (float*)out, ldo, n, group, gate_act);
    return dk_launch(norm_gate_kernel<bf16>, grid, dim3(threads), 0, st, o, w, eps, (const bf16*)gate, ldg,
                     out_scale, (bf16*)out, ldo, n, group, gate_act);
}
