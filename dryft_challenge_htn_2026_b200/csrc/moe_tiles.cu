// The routed experts of a mixture of experts for many tokens at once, bfloat16, on mma.sync tensor cores.
//
// The (token, chosen expert) pairs are put in the order of their experts on the device (one block counts,
// scans and scatters; nothing goes through the host, so the step can be captured as a graph), cut into tiles
// of 64 pairs of one expert, and every tile is a small matrix product against that expert's matrices:
//   up:    mid[r] = act(W_gate[e] x_r) * (W_up[e] x_r)      rows gathered by token, both products in one pass
//   down:  y[r]   = W_down[e] mid[r]
//   sum:   out[t] = sum_j weight[t][j] * y[place of pair (t, j)] + gate[t] * shared[t]
// A row's sums run over its own elements in a fixed order, so a result does not depend on which other pairs
// share its tile. Grids are sized for the most tiles the pairs can make (pairs / 64 + experts); blocks
// beyond the tiles that exist leave at once.
#include "common.cuh"

#define MT_ROWS 64      // pairs a tile
#define MT_COLS 64      // output columns a block
#define MT_KC 32        // inner elements a stage
#define MT_STAGES 3
#define MT_STR (MT_KC + 8)

__device__ __forceinline__ void mt_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mt_ldsm(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mt_cp16(bf16* smem, const bf16* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void mt_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void mt_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One block. idx [P] = expert of every pair. Leaves perm [P] (pairs in expert order), inv [P] (a pair's place in
// that order) and for every tile its expert, first place and row count in tiles [max_tiles][3] (rows 0: no tile).
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* idx, int P, int E, int* perm, int* inv, int* tiles, int max_tiles) {
    __shared__ int cnt[256], off[257], tbase[257];
    pdl_wait();
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        off[0] = tbase[0] = 0;
        for (int e = 0; e < E; e++) {
            off[e + 1] = off[e] + cnt[e];
            tbase[e + 1] = tbase[e] + (cnt[e] + MT_ROWS - 1) / MT_ROWS;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        for (int k = 0; tbase[e] + k < tbase[e + 1]; k++) {
            int* t = tiles + 3 * (tbase[e] + k);
            t[0] = e, t[1] = off[e] + k * MT_ROWS, t[2] = min(MT_ROWS, cnt[e] - k * MT_ROWS);
        }
    }
    for (int t = tbase[E] + threadIdx.x; t < max_tiles; t += blockDim.x) tiles[3 * t] = 0, tiles[3 * t + 1] = 0, tiles[3 * t + 2] = 0;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = idx[p];
        const int at = off[e] + atomicAdd(&cnt[e], 1);
        perm[at] = p;
        inv[p] = at;
    }
}

// Block (tile, 64 columns of the output). GATED: B is an expert's [gate rows; up rows] (2 * N rows of K), the
// output act(gate) * up; A rows are gathered (row r of the tile is token perm[first + r] / top of x). Otherwise B is
// the expert's [N rows of K] and A the rows first + r of a dense matrix. K % 32 == 0; rows on 16-byte boundaries.
// Three stages of 32 inner elements in flight (cp.async), one block barrier a stage: 46 KB a block, four blocks an SM
// (stages of 64 left room for two blocks and ran 12 % slower).
template <bool GATED>
__global__ void __launch_bounds__(128)
moe_tile_product_kernel(const bf16* A, const bf16* __restrict__ B, const int* tiles, const int* perm, int top, bf16* out,
                        int N, int K, int act, const float* in_wt, float limit) {
    extern __shared__ __align__(16) bf16 mt_smem[];
    constexpr int A_ELEMS = MT_ROWS * MT_STR, B_ELEMS = (GATED ? 2 : 1) * MT_COLS * MT_STR;
    bf16* As = mt_smem;                              // [MT_STAGES][A_ELEMS]
    bf16* Bs = mt_smem + MT_STAGES * A_ELEMS;        // [MT_STAGES][B_ELEMS]
    __shared__ int arow[MT_ROWS];
    pdl_wait();
    pdl_launch_dependents();
    const int* tl = tiles + 3 * blockIdx.x;
    const int rows = tl[2];
    if (rows == 0) return;
    const int e = tl[0], first = tl[1];
    const int n0 = blockIdx.y * MT_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < MT_ROWS) arow[tid] = tid < rows ? (GATED ? perm[first + tid] / top : first + tid) : -1;
    for (int i = tid; i < MT_STAGES * (A_ELEMS + B_ELEMS) / 8; i += 128) reinterpret_cast<uint4*>(mt_smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const bf16* Be = B + (size_t)e * (GATED ? 2 : 1) * N * K;
    const int nk = K / MT_KC;
    constexpr int PCS = MT_KC / 8;                                  // 16-byte pieces a row and stage
    auto load = [&](int kc) {                                       // stage kc into buffer kc % MT_STAGES; past the end: an empty group
        if (kc < nk) {
            const int k0 = kc * MT_KC, buf = kc % MT_STAGES;
            for (int i = tid; i < MT_ROWS * PCS; i += 128) {
                const int r = i / PCS, c = (i % PCS) * 8;
                if (arow[r] >= 0) mt_cp16(As + buf * A_ELEMS + r * MT_STR + c, A + (size_t)arow[r] * K + k0 + c);
            }
            for (int i = tid; i < (GATED ? 2 : 1) * MT_COLS * PCS; i += 128) {
                const int r = i / PCS, c = (i % PCS) * 8;
                const int n = n0 + (r % MT_COLS);
                if (n < N) mt_cp16(Bs + buf * B_ELEMS + r * MT_STR + c, Be + ((size_t)(r / MT_COLS) * N + n) * K + k0 + c);
            }
        }
        mt_commit();
    };
    // four warps as 2 x 2: each owns 32 rows x 32 columns (two 16-row fragments of A against two 16-column fragments
    // of B: 6 ldmatrix for 16 mma a 16-wide step of the gated product, where 16 x 64 a warp needed 9)
    const int wm = warp >> 1, wn = warp & 1;
    float accg[2][4][4], accu[GATED ? 2 : 1][4][4];
#pragma unroll
    for (int m = 0; m < 2; m++)
#pragma unroll
        for (int i = 0; i < 4; i++) accg[m][i][0] = accg[m][i][1] = accg[m][i][2] = accg[m][i][3] = 0.f;
#pragma unroll
    for (int m = 0; m < (GATED ? 2 : 1); m++)
#pragma unroll
        for (int i = 0; i < 4; i++) accu[m][i][0] = accu[m][i][1] = accu[m][i][2] = accu[m][i][3] = 0.f;
    load(0);
    load(1);
    const int j = lane >> 3;
    for (int kc = 0; kc < nk; kc++) {
        const int buf = kc % MT_STAGES;
        mt_wait<1>();                 // stage kc has landed (one later group may still be on its way)
        __syncthreads();              // ... for every thread, and all are done with the buffer that stage kc + 2 goes to
        load(kc + 2);
        const bf16* Ab = As + buf * A_ELEMS;
        const bf16* Bb = Bs + buf * B_ELEMS;
#pragma unroll
        for (int kk = 0; kk < MT_KC / 16; kk++) {
            uint32_t a0[4], a1[4];
            mt_ldsm(a0, Ab + (wm * 32 + (lane & 15)) * MT_STR + kk * 16 + 8 * (lane >> 4));
            mt_ldsm(a1, Ab + (wm * 32 + 16 + (lane & 15)) * MT_STR + kk * 16 + 8 * (lane >> 4));
#pragma unroll
            for (int np = 0; np < 2; np++) {
                uint32_t b[4];
                mt_ldsm(b, Bb + (wn * 32 + np * 16 + (lane & 7) + 8 * (j >> 1)) * MT_STR + kk * 16 + 8 * (j & 1));
                mt_mma(accg[0][2 * np], a0, b[0], b[1]);
                mt_mma(accg[0][2 * np + 1], a0, b[2], b[3]);
                mt_mma(accg[1][2 * np], a1, b[0], b[1]);
                mt_mma(accg[1][2 * np + 1], a1, b[2], b[3]);
                if (GATED) {
                    mt_ldsm(b, Bb + (MT_COLS + wn * 32 + np * 16 + (lane & 7) + 8 * (j >> 1)) * MT_STR + kk * 16 + 8 * (j & 1));
                    mt_mma(accu[0][2 * np], a0, b[0], b[1]);
                    mt_mma(accu[0][2 * np + 1], a0, b[2], b[3]);
                    mt_mma(accu[1][2 * np], a1, b[0], b[1]);
                    mt_mma(accu[1][2 * np + 1], a1, b[2], b[3]);
                }
            }
        }
    }
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int m = 0; m < 2; m++)
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int r = wm * 32 + m * 16 + g + 8 * (c >> 1), n = n0 + wn * 32 + nt * 8 + 2 * t + (c & 1);
                if (r < rows && n < N) {
                    float v = accg[m][nt][c];
                    if (GATED) {
                        float u = accu[m][nt][c];
                        if (in_wt != nullptr) {      // the pair's weight on the expert's input: W (w x) = w (W x)
                            const float w = in_wt[perm[first + r]];
                            v *= w;
                            u *= w;
                        }
                        if (act == 2) {              // g' = min(g, limit), u' = clamp(u): g' sigmoid(1.702 g') (u' + 1)
                            v = fminf(v, limit);
                            u = fminf(fmaxf(u, -limit), limit);
                            v = v / (1.f + expf(-1.702f * v)) * (u + 1.f);
                        } else {
                            v = (act == 1 ? 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)))
                                          : v / (1.f + expf(-v))) * u;
                        }
                    }
                    out[(size_t)(first + r) * N + n] = __float2bfloat16_rn(v);
                }
            }
        }
}

// out[t][c] = sum_j wt[t][j] * y[inv[t * top + j]][c] + sgate[t] * shared[t][c]
__global__ void moe_sum_kernel(const bf16* y, const int* inv, const float* wt, const bf16* shared, const float* sgate, bf16* out,
                               int W, int top) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; j++) acc = fmaf(wt != nullptr ? wt[t * top + j] : 1.f, __bfloat162float(y[(size_t)inv[t * top + j] * W + c]), acc);
        if (shared != nullptr) acc = fmaf(sgate ? sgate[t] : 1.f, __bfloat162float(shared[t * W + c]), acc);
        out[t * W + c] = __float2bfloat16_rn(acc);
    }
}

DK_EXPORT int dk_moe_sort(const int* idx, int P, int E, int* perm, int* inv, int* tiles, int max_tiles, cudaStream_t st) {
    if (E < 1 || E > 256 || max_tiles < (P + MT_ROWS - 1) / MT_ROWS + E - 1) return (int)cudaErrorInvalidValue;
    return dk_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, st, idx, P, E, perm, inv, tiles, max_tiles);
}

DK_EXPORT int dk_moe_up_tiles(const void* x, const void* wgu, const int* tiles, int max_tiles, const int* perm, int top, void* mid,
                              int ff, int W, int act, const float* in_wt, float limit, cudaStream_t st) {
    if (W % MT_KC || ((uintptr_t)x | (uintptr_t)wgu) % 16) return (int)cudaErrorInvalidValue;
    constexpr size_t smem = sizeof(bf16) * MT_STAGES * (MT_ROWS + 2 * MT_COLS) * MT_STR;
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(moe_tile_product_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    return dk_launch(moe_tile_product_kernel<true>, dim3(max_tiles, (ff + MT_COLS - 1) / MT_COLS), dim3(128), smem, st, (const bf16*)x,
                     (const bf16*)wgu, tiles, perm, top, (bf16*)mid, ff, W, act, in_wt, limit);
}

DK_EXPORT int dk_moe_down_tiles(const void* mid, const void* wd, const int* tiles, int max_tiles, void* y, int W, int ff,
                                cudaStream_t st) {
    if (ff % MT_KC || ((uintptr_t)mid | (uintptr_t)wd) % 16) return (int)cudaErrorInvalidValue;
    constexpr size_t smem = sizeof(bf16) * MT_STAGES * (MT_ROWS + MT_COLS) * MT_STR;
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(moe_tile_product_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    return dk_launch(moe_tile_product_kernel<false>, dim3(max_tiles, (W + MT_COLS - 1) / MT_COLS), dim3(128), smem, st, (const bf16*)mid,
                     (const bf16*)wd, tiles, (const int*)nullptr, 1, (bf16*)y, W, ff, 0, (const float*)nullptr, 0.f);
}

DK_EXPORT int dk_moe_sum(const void* y, const int* inv, const float* wt, const void* shared, const float* sgate, void* out,
                         int n_tok, int W, int top, cudaStream_t st) {
    return dk_launch(moe_sum_kernel, dim3(n_tok), dim3(W >= 1024 ? 256 : 128), 0, st, (const bf16*)y, inv, wt, (const bf16*)shared,
                     sgate, (bf16*)out, W, top);
}
