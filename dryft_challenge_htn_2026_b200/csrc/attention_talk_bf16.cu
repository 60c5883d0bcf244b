// Attention with mixed head scores (see attention_talk.cu for the float32-arithmetic form) on mma.sync tensor cores, for
// bfloat16 with key and value sizes in steps of 16 (built per pair of sizes with -DHD= -DHDV=).
//
// A block takes 16 consecutive queries of one sequence (or one single token) with all their heads and walks the keys in
// runs of 32: the run's key and value rows of every kv head are staged in shared memory (cp.async); warp g makes the raw
// scores q_g . k of its 16 x 32 tile with mma.sync and leaves them in shared memory (float32); after a barrier warp h
// mixes them, s'_h = sum_g talk[h][g] s_g (float32, in the fragment layout of its own tile), masks, moves its rows'
// running maximum and sum on and adds P . V of its head with mma.sync. A block has min(heads, 16) warps; with more heads
// the output heads are dealt out over blockIdx.z and every block makes all raw scores. For single tokens the runs of
// keys are dealt out over blockIdx.y and a second kernel merges the parts.
#include "common.cuh"

#ifndef HD
#error "compile with -DHD=<key size> -DHDV=<value size>"
#endif
static_assert(HD % 16 == 0 && HDV % 16 == 0 && HD <= 256 && HDV <= 256, "head sizes in steps of 16 up to 256");

#define TK_KB 32                    // keys a run
#define TK_ROWS 16                  // queries a block
#define TK_MAX_WARPS 16
// rows of scores 40 floats apart: the 16 lanes of a half warp (4 rows x 4 pairs of columns) then read 16 different pairs of banks
constexpr int KSTR = HD + 8, VSTR = HDV + 8, SSTR = TK_KB + 8;

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void cp_async16(bf16* smem, const bf16* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// tiles (prompts): tiles[2i] = sequence, tiles[2i + 1] = first query of the tile within the sequence's rows of this step.
// tiles == nullptr (single tokens): block x is row x, its position row_pos[x], its page table row x.
template <bool QS>
__global__ void __launch_bounds__(32 * TK_MAX_WARPS)
attn_talk_kernel(const bf16* q, long long ldq, bf16* out, long long ldo, float out_scale, const bf16* k_store, const bf16* v_store,
                 const int* tiles, const int* cu_q, const int* seq_pos0, const int* row_pos, const int* page_table, int pt_stride,
                 int nh, int nkv, int window, float scale, const float* __restrict__ talk, int nsplit, float* ws_acc, float* ws_ml) {
    constexpr bool q_staged = QS;
    extern __shared__ __align__(16) unsigned char tk_smem[];
    bf16* Ks = reinterpret_cast<bf16*>(tk_smem);                                   // [nkv][TK_KB][KSTR]
    bf16* Vs = Ks + (size_t)nkv * TK_KB * KSTR;                                    // [nkv][TK_KB][VSTR]
    float* S = reinterpret_cast<float*>(Vs + (size_t)nkv * TK_KB * VSTR);          // [nh][TK_ROWS][SSTR]
    float* Tm = S + (size_t)nh * TK_ROWS * SSTR;                                   // [nh][nh] talk * scale * log2(e)
    bf16* Qs = reinterpret_cast<bf16*>(Tm + (((size_t)nh * nh + 3) & ~(size_t)3));  // [nh][TK_ROWS][KSTR], when q_staged
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, t4 = lane & 3;
    const int n_warps = blockDim.x >> 5, group = nh / nkv;
    int seq, row_first, rows_here, pos_first;
    if (tiles != nullptr) {
        seq = tiles[2 * blockIdx.x];
        const int q0 = tiles[2 * blockIdx.x + 1];
        row_first = cu_q[seq] + q0;
        rows_here = min(TK_ROWS, cu_q[seq + 1] - cu_q[seq] - q0);
        pos_first = seq_pos0[seq] + q0;
    } else {
        seq = blockIdx.x;
        row_first = blockIdx.x;
        rows_here = 1;
        pos_first = row_pos[blockIdx.x];
    }
    const int h = blockIdx.z * n_warps + warp;               // the output head of this warp
    const bool has_head = h < nh;
    if (pos_first < 0) {                                      // a padding row
        if (has_head && nsplit == 1)
            for (int d = lane; d < HDV; d += 32) out[(size_t)row_first * ldo + (size_t)h * HDV + d] = __float2bfloat16_rn(0.f);
        if (has_head && nsplit > 1 && lane == 0) {
            float* ml = ws_ml + (((size_t)row_first * nh + h) * nsplit + blockIdx.y) * 2;
            ml[0] = -INFINITY, ml[1] = 0.f;
        }
        return;
    }
    const int* pt = page_table + (size_t)seq * pt_stride;
    for (int i = tid; i < nh * nh; i += blockDim.x) Tm[i] = talk[i] * scale * 1.4426950408889634f;
    // rows gq and gq + 8 of the tile: positions and the first key each sees
    int hi[2], lo[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int rr = gq + 8 * r;
        hi[r] = rr < rows_here ? pos_first + rr : -1;
        lo[r] = window > 0 ? max(0, hi[r] - window + 1) : 0;
    }
    const int pos_last = pos_first + rows_here - 1;
    const int key_first = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int run_first = key_first / TK_KB, run_end = pos_last / TK_KB + 1;
    const int per = (run_end - run_first + nsplit - 1) / nsplit;
    const int run0 = run_first + blockIdx.y * per, run1 = min(run_end, run0 + per);
    const bf16* qrow[2] = {gq < rows_here ? q + (size_t)(row_first + gq) * ldq : nullptr,
                           gq + 8 < rows_here ? q + (size_t)(row_first + gq + 8) * ldq : nullptr};
    if (q_staged) {      // the tile's query rows of every head into shared memory once (zeros for rows past the end): read by ldmatrix in every run
        constexpr int QP = HD / 8;
        for (int i = tid; i < nh * TK_ROWS * QP; i += blockDim.x) {
            const int pc = i % QP, rr = (i / QP) % TK_ROWS, g = i / (QP * TK_ROWS);
            bf16* dst = Qs + ((size_t)g * TK_ROWS + rr) * KSTR + pc * 8;
            if (rr < rows_here) cp_async16(dst, q + (size_t)(row_first + rr) * ldq + (size_t)g * HD + pc * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");     // waited for with the first run's keys
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[HDV / 8][4];
#pragma unroll
    for (int i = 0; i < HDV / 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int j8 = lane >> 3;
    for (int run = run0; run < run1; run++) {
        const int j0 = run * TK_KB;
        const int page = pt[j0 / DK_PAGE], in_page = j0 % DK_PAGE;
        __syncthreads();                                      // the run before is done with Ks, Vs and S
        constexpr int KP = HD / 8, VP = HDV / 8;              // 16-byte pieces a row
        for (int i = tid; i < nkv * TK_KB * KP; i += blockDim.x) {
            const int pc = i % KP, jj = (i / KP) % TK_KB, g = i / (KP * TK_KB);
            cp_async16(Ks + ((size_t)g * TK_KB + jj) * KSTR + pc * 8, k_store + kv_offset(page, nkv, g, in_page + jj, HD) + pc * 8);
        }
        for (int i = tid; i < nkv * TK_KB * VP; i += blockDim.x) {
            const int pc = i % VP, jj = (i / VP) % TK_KB, g = i / (VP * TK_KB);
            cp_async16(Vs + ((size_t)g * TK_KB + jj) * VSTR + pc * 8, v_store + kv_offset(page, nkv, g, in_page + jj, HDV) + pc * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // raw scores: this warp's heads g = warp, warp + n_warps, ..: a 16 x 32 tile each, into shared memory
        for (int g = warp; g < nh; g += n_warps) {
            float s[TK_KB / 8][4];
#pragma unroll
            for (int i = 0; i < TK_KB / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            const bf16* Kg = Ks + (size_t)(g / group) * TK_KB * KSTR;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++) {
                const int c = g * HD + ks * 16 + 2 * t4;
                uint32_t a[4];
                if (q_staged) {
                    ldsm_x4(a, Qs + ((size_t)g * TK_ROWS + (lane & 15)) * KSTR + ks * 16 + 8 * (lane >> 4));
                } else {
                    a[0] = qrow[0] ? *reinterpret_cast<const uint32_t*>(qrow[0] + c) : 0u;
                    a[1] = qrow[1] ? *reinterpret_cast<const uint32_t*>(qrow[1] + c) : 0u;
                    a[2] = qrow[0] ? *reinterpret_cast<const uint32_t*>(qrow[0] + c + 8) : 0u;
                    a[3] = qrow[1] ? *reinterpret_cast<const uint32_t*>(qrow[1] + c + 8) : 0u;
                }
#pragma unroll
                for (int np = 0; np < TK_KB / 16; np++) {
                    uint32_t b[4];
                    ldsm_x4(b, Kg + (np * 16 + (lane & 7) + 8 * (j8 >> 1)) * KSTR + ks * 16 + 8 * (j8 & 1));
                    mma16816(s[2 * np], a, b[0], b[1]);
                    mma16816(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            float* Sg = S + (size_t)g * TK_ROWS * SSTR;
#pragma unroll
            for (int nt = 0; nt < TK_KB / 8; nt++) {
                *reinterpret_cast<float2*>(Sg + gq * SSTR + nt * 8 + 2 * t4) = make_float2(s[nt][0], s[nt][1]);
                *reinterpret_cast<float2*>(Sg + (gq + 8) * SSTR + nt * 8 + 2 * t4) = make_float2(s[nt][2], s[nt][3]);
            }
        }
        __syncthreads();
        if (!has_head) continue;
        // this warp's head: mixed scores in the fragment layout, masks, online softmax, P . V
        float x[TK_KB / 8][4];
#pragma unroll
        for (int i = 0; i < TK_KB / 8; i++) x[i][0] = x[i][1] = x[i][2] = x[i][3] = 0.f;
        for (int g = 0; g < nh && (hi[0] >= 0 || hi[1] >= 0); g++) {      // rows that do not exist (a single token has one) are masked anyway
            const float tg = Tm[h * nh + g];
            const float* Sg = S + (size_t)g * TK_ROWS * SSTR;
#pragma unroll
            for (int nt = 0; nt < TK_KB / 8; nt++) {
                const float2 u0 = *reinterpret_cast<const float2*>(Sg + gq * SSTR + nt * 8 + 2 * t4);
                const float2 u1 = *reinterpret_cast<const float2*>(Sg + (gq + 8) * SSTR + nt * 8 + 2 * t4);
                x[nt][0] = fmaf(tg, u0.x, x[nt][0]);
                x[nt][1] = fmaf(tg, u0.y, x[nt][1]);
                x[nt][2] = fmaf(tg, u1.x, x[nt][2]);
                x[nt][3] = fmaf(tg, u1.y, x[nt][3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < TK_KB / 8; nt++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int key = j0 + nt * 8 + 2 * t4 + (c & 1), r = c >> 1;
                const float v = key >= lo[r] && key <= hi[r] ? x[nt][c] : -INFINITY;
                x[nt][c] = v;
                mx[r] = fmaxf(mx[r], v);
            }
        float ms[2], alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            ms[r] = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = exp2f(m[r] - ms[r]);
            m[r] = m_new;
        }
#pragma unroll
        for (int nt = 0; nt < TK_KB / 8; nt++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float p = exp2f(x[nt][c] - ms[c >> 1]);
                x[nt][c] = p;
                sum[c >> 1] += p;
            }
        l[0] = l[0] * alpha[0] + sum[0];
        l[1] = l[1] * alpha[1] + sum[1];
#pragma unroll
        for (int i = 0; i < HDV / 8; i++) {
            acc[i][0] *= alpha[0];
            acc[i][1] *= alpha[0];
            acc[i][2] *= alpha[1];
            acc[i][3] *= alpha[1];
        }
        const bf16* Vg = Vs + (size_t)(h / group) * TK_KB * VSTR;
#pragma unroll
        for (int kk = 0; kk < TK_KB / 16; kk++) {
            uint32_t a[4];
            a[0] = pack_bf16(x[2 * kk][0], x[2 * kk][1]);
            a[1] = pack_bf16(x[2 * kk][2], x[2 * kk][3]);
            a[2] = pack_bf16(x[2 * kk + 1][0], x[2 * kk + 1][1]);
            a[3] = pack_bf16(x[2 * kk + 1][2], x[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HDV / 16; dp++) {
                uint32_t b[4];
                ldsm_x4_trans(b, Vg + (kk * 16 + (lane & 15)) * VSTR + dp * 16 + 8 * (lane >> 4));
                mma16816(acc[2 * dp], a, b[0], b[1]);
                mma16816(acc[2 * dp + 1], a, b[2], b[3]);
            }
        }
    }
    if (!has_head) return;
#pragma unroll
    for (int r = 0; r < 2; r++) {          // a row's sum is spread over the four lanes that hold its columns
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    if (nsplit == 1) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int rr = gq + 8 * r;
            if (rr >= rows_here) continue;
            const float inv = out_scale / l[r];
            bf16* o = out + (size_t)(row_first + rr) * ldo + (size_t)h * HDV;
#pragma unroll
            for (int i = 0; i < HDV / 8; i++)
                *reinterpret_cast<uint32_t*>(o + i * 8 + 2 * t4) = pack_bf16(acc[i][2 * r] * inv, acc[i][2 * r + 1] * inv);
        }
        return;
    }
    // single tokens, keys dealt out over blocks: this block's part of row 0 (maximum, sum, unnormalised P . V)
    if (gq == 0) {
        const size_t part = ((size_t)row_first * nh + h) * nsplit + blockIdx.y;
        if (t4 == 0) { ws_ml[part * 2] = m[0]; ws_ml[part * 2 + 1] = l[0]; }
#pragma unroll
        for (int i = 0; i < HDV / 8; i++)
            *reinterpret_cast<float2*>(ws_acc + part * HDV + i * 8 + 2 * t4) = make_float2(acc[i][0], acc[i][1]);
    }
}

// out[row][h] = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s * out_scale; a warp per (row, head)
__global__ void attn_talk_merge_kernel(const float* ws_acc, const float* ws_ml, bf16* out, long long ldo, float out_scale,
                                       const int* row_pos, int n_rows, int nh, int nsplit) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= n_rows * nh) return;
    const int b = wid / nh, h = wid % nh;
    bf16* o = out + (size_t)b * ldo + (size_t)h * HDV;
    if (row_pos[b] < 0) {
        for (int d = lane; d < HDV; d += 32) o[d] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* ml = ws_ml + ((size_t)b * nh + h) * nsplit * 2;
    const float* acc = ws_acc + ((size_t)b * nh + h) * nsplit * HDV;
    // lane s holds part s (nsplit <= 32): its maximum and sum in one trip, its weight 2^(m_s - M) handed round by shuffles
    const float m_s = lane < nsplit ? ml[2 * lane] : -INFINITY;
    const float l_s = lane < nsplit ? ml[2 * lane + 1] : 0.f;
    const float M = warp_max(m_s);
    const float w = l_s > 0.f ? exp2f(m_s - M) : 0.f;
    const float inv = out_scale / warp_sum(l_s * w);
    float v[HDV / 32 + 1];
#pragma unroll
    for (int i = 0; i < HDV / 32 + 1; i++) v[i] = 0.f;
    for (int s = 0; s < nsplit; s++) {
        const float ws = __shfl_sync(0xffffffffu, w, s);
#pragma unroll
        for (int i = 0; i < HDV / 32 + 1; i++) {
            const int d = lane + 32 * i;
            if (d < HDV) v[i] = fmaf(acc[(size_t)s * HDV + d], ws, v[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < HDV / 32 + 1; i++) {
        const int d = lane + 32 * i;
        if (d < HDV) o[d] = __float2bfloat16_rn(v[i] * inv);
    }
}

static size_t talk_smem(int nh, int nkv, bool q_staged) {
    return sizeof(bf16) * (size_t)nkv * TK_KB * (KSTR + VSTR) + sizeof(float) * ((size_t)nh * TK_ROWS * SSTR + (((size_t)nh * nh + 3) & ~(size_t)3)) +
           (q_staged ? sizeof(bf16) * (size_t)nh * TK_ROWS * KSTR : 0);
}

// n_tiles blocks of 16 queries (tiles) or n_tiles single tokens (tiles == nullptr, keys in nsplit runs with the merge)
DK_EXPORT int dk_attention_talk_bf16(const void* q, long long ldq, void* out, long long ldo, float out_scale, const void* k_store,
                                     const void* v_store, const int* tiles, int n_tiles, const int* cu_q, const int* seq_pos0,
                                     const int* row_pos, const int* page_table, int pt_stride, int nh, int nkv, int window,
                                     float scale, const float* talk, int nsplit, float* ws_acc, float* ws_ml, cudaStream_t st) {
    if (nh < 1 || nh > 64 || nkv < 1 || nh % nkv || nsplit < 1 || nsplit > 32 || (nsplit > 1 && (tiles != nullptr || ws_acc == nullptr || ws_ml == nullptr)))
        return (int)cudaErrorInvalidValue;
    // the query rows stay in shared memory where there is room (16-byte rows), else every run reads them from memory again
    // (a single token has one row: it is read from memory, and two blocks may share an SM)
    const bool q_staged = tiles != nullptr && talk_smem(nh, nkv, true) <= 220 * 1024 && (uintptr_t)q % 16 == 0 && (ldq * 2) % 16 == 0;
    const size_t smem = talk_smem(nh, nkv, q_staged);
    if (smem > 220 * 1024) return (int)cudaErrorInvalidValue;
    static size_t attr[2] = {0, 0};
    if (smem > 48 * 1024 && smem > attr[q_staged]) {
        cudaError_t e = q_staged ? cudaFuncSetAttribute(attn_talk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                 : cudaFuncSetAttribute(attn_talk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr[q_staged] = smem;
    }
    const int warps = nh < TK_MAX_WARPS ? nh : TK_MAX_WARPS;
    const dim3 grid(n_tiles, nsplit, (nh + warps - 1) / warps), block(32 * warps);
    int e = q_staged ? dk_launch(attn_talk_kernel<true>, grid, block, smem, st, (const bf16*)q, ldq, (bf16*)out, ldo, out_scale,
                                 (const bf16*)k_store, (const bf16*)v_store, tiles, cu_q, seq_pos0, row_pos, page_table, pt_stride, nh,
                                 nkv, window, scale, talk, nsplit, ws_acc, ws_ml)
                     : dk_launch(attn_talk_kernel<false>, grid, block, smem, st, (const bf16*)q, ldq, (bf16*)out, ldo, out_scale,
                                 (const bf16*)k_store, (const bf16*)v_store, tiles, cu_q, seq_pos0, row_pos, page_table, pt_stride, nh,
                                 nkv, window, scale, talk, nsplit, ws_acc, ws_ml);
    if (e || nsplit == 1) return e;
    const int warps_m = n_tiles * nh;
    return dk_launch(attn_talk_merge_kernel, dim3((warps_m + 3) / 4), dim3(128), 0, st, (const float*)ws_acc, (const float*)ws_ml,
                     (bf16*)out, ldo, out_scale, row_pos, n_tiles, nh, nsplit);
}
