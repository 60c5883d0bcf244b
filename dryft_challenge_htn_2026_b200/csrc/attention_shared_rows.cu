// bfloat16 attention over cached rows that are key and value at once: a key is the whole row (HD numbers), its value
// the row's first HDV numbers, and the query heads of a group all read the same rows. That is attention through
// low-rank latents with the keys' up projection moved to the query's side: rows of [latent | rotated part], hundreds
// of numbers wide, far beyond what a warp can hold as fragments. Built once per pair of sizes with -DHD= -DHDV=
// (HD a multiple of 16 up to 640, HDV a multiple of 32 up to 512 and at most HD). A chunk mask or a window bounds
// the keys; scores, softmax and sums are float32, P is rounded to bfloat16 before P.V.
//
// A block of 8 warps owns 64 rows of the (query, head of the group) plane of one sequence and one key/value head:
// with G heads in a group, 64 / G consecutive queries with all their heads (G >= 64: one query and 64 of its heads).
// It keeps its 64 query rows in shared memory and walks the keys in half pages of 32, staged by cp.async (three stages:
// the half page whose scores are taken, the one before it, whose P.V runs side by side with them, and the one on its way):
//   scores : warp (r, c) takes rows 16 r .. 16 r + 15 against keys 16 c .. 16 c + 15 of the half page, query and key
//            fragments by ldmatrix, mma.sync m16n8k16; the two warps of a row block meet their row maxima in shared
//            memory and leave P there;
//   P.V    : warp (r, c) holds the output of its 16 rows for the value columns c HDV / 2 .. (c + 1) HDV / 2 - 1 in
//            registers and adds P (16 x 32) times those columns of the staged rows.
// One kernel serves prompts (tiles from the host's work list) and single tokens (a block per token and 64 heads; the
// keys of a token may be dealt out to several blocks, whose parts a second kernel puts together).
#include "common.cuh"

#if !defined(HD) || !defined(HDV)
#error "compile with -DHD=<row size> -DHDV=<value size>"
#endif
static_assert(HD % 16 == 0 && HD >= 32 && HD <= 640, "row size must be a multiple of 16 up to 640");
static_assert(HDV % 32 == 0 && HDV >= 32 && HDV <= 512 && HDV <= HD, "value size must be a multiple of 32 up to 512, at most the row size");

constexpr int SR_ROWS = 64;                 // rows of the (query, head) plane a block owns
constexpr int SR_KEYS = 32;                 // keys a turn
constexpr int SR_THREADS = 256;
constexpr int SR_STR = HD + 8;              // shared-memory stride of query and key rows (elements): 16 B of padding
constexpr int SR_PSTR = SR_KEYS + 8;
constexpr int SR_Q_ELEMS = SR_ROWS * SR_STR;
constexpr int SR_K_ELEMS = SR_KEYS * SR_STR;
constexpr int SR_P_ELEMS = SR_ROWS * SR_PSTR;
constexpr int SR_STAGES = 3;
constexpr size_t SR_SMEM_BYTES = (size_t)(SR_Q_ELEMS + SR_STAGES * SR_K_ELEMS + SR_P_ELEMS) * sizeof(bf16) + 4 * SR_ROWS * sizeof(float);
constexpr int SR_HALF = HDV / 2;            // value columns a warp holds

__device__ __forceinline__ void sr_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sr_ldsm(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sr_ldsm_trans(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sr_cp16(bf16* smem, const bf16* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void sr_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void sr_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t sr_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ int sr_first_key(int pos, int window, int chunk) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    return lo;
}

// half page ``kt`` (keys 32 kt .. 32 kt + 31 of the sequence) of one key/value head into a stage
__device__ __forceinline__ void sr_stage_keys(bf16* stage, const bf16* k_store, const int* pt, int kt, int nkv, int kvh) {
    const size_t off = kv_offset(pt[kt / (DK_PAGE / SR_KEYS)], nkv, kvh, (kt % (DK_PAGE / SR_KEYS)) * SR_KEYS, HD);
    constexpr int CK = HD / 8;
    for (int c = threadIdx.x; c < SR_KEYS * CK; c += SR_THREADS) {
        const int row = c / CK, col = (c % CK) * 8;
        sr_cp16(stage + row * SR_STR + col, k_store + off + (size_t)row * HD + col);
    }
}

// The products of a turn, the two kinds step by step in turn so that neither waits for its own loads: SCORES: s +=
// (16 query rows at qa) x (16 keys at kc) over the row's length, in two chains of sums (even and odd steps); PV: acc +=
// (P of 16 rows x 32 keys at pa) x (this warp's value columns of those 32 rows at vp).
template <bool SCORES, bool PV>
__device__ __forceinline__ void sr_products(const bf16* qa, const bf16* kc, const bf16* pa, const bf16* vp, float (&s)[2][4],
                                            float (&acc)[SR_HALF / 8][4]) {
    constexpr int DPN = SR_HALF / 16;
    constexpr int N1 = SCORES ? HD / 16 : 0, N2 = PV ? (SR_KEYS / 16) * DPN : 0;
    float s2[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++) s2[i][0] = s2[i][1] = s2[i][2] = s2[i][3] = 0.f;
    uint32_t pf[4];
#pragma unroll
    for (int i = 0; i < (N1 > N2 ? N1 : N2); i++) {
        if (i < N1) {
            uint32_t a[4], b[4];
            sr_ldsm(a, qa + i * 16);
            sr_ldsm(b, kc + i * 16);
            if (i & 1) {
                sr_mma(s2[0], a, b[0], b[1]);
                sr_mma(s2[1], a, b[2], b[3]);
            } else {
                sr_mma(s[0], a, b[0], b[1]);
                sr_mma(s[1], a, b[2], b[3]);
            }
        }
        if (i < N2) {
            const int kk = i / DPN, dp = i % DPN;
            if (dp == 0) sr_ldsm(pf, pa + kk * 16);
            uint32_t b[4];
            sr_ldsm_trans(b, vp + kk * 16 * SR_STR + dp * 16);
            sr_mma(acc[2 * dp], pf, b[0], b[1]);
            sr_mma(acc[2 * dp + 1], pf, b[2], b[3]);
        }
    }
    if (SCORES) {
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int c = 0; c < 4; c++) s[i][c] += s2[i][c];
    }
}

// grid (work items, nkv * head blocks, nsplit). Prompts (``tiles`` given): item i = (sequence tiles[2i], first query
// tiles[2i+1] of the step's portion), 64 / G queries a block; cu_q: first flat row of each portion; seq_pos0: tokens
// cached before it. Single tokens (``tiles`` null): item i = row i at position row_pos[i] (negative: padding, zeros
// out), page table row i. The step's own keys are in the cache when this runs. q and out are rows of wider matrices.
// nsplit > 1: the half pages a block's rows can see are dealt out in runs to nsplit blocks, each of which leaves its
// part (maximum and sum in ws_ml [rows, nh, nsplit, 2], unnormalised P.V in ws_acc [rows, nh, nsplit, HDV]).
__global__ void __launch_bounds__(SR_THREADS, 1)
attn_shared_rows_kernel(const bf16* q, long long ldq, bf16* out, long long ldo, float out_scale, const bf16* k_store,
                        const int* tiles, const int* cu_q, const int* seq_pos0, const int* row_pos, const int* page_table,
                        int pt_stride, int nh, int nkv, int window, int chunk, float sl2, int nsplit, float* ws_acc,
                        float* ws_ml) {
    extern __shared__ __align__(16) bf16 smem[];
    bf16* Qs = smem;
    bf16* Ks = Qs + SR_Q_ELEMS;
    bf16* Ps = Ks + SR_STAGES * SR_K_ELEMS;
    float* smax = reinterpret_cast<float*>(Ps + SR_P_ELEMS);      // [2][64]: a row's maximum over each half of the turn's keys
    float* ssum = smax + 2 * SR_ROWS;                             // [2][64]: a row's sum over the keys of each warp column
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int wr = warp & 3, wc = warp >> 2, split = blockIdx.z;
    const int G = nh / nkv, GB = min(G, SR_ROWS), HB = (G + SR_ROWS - 1) / SR_ROWS;
    const int kvh = blockIdx.y / HB, hb = blockIdx.y % HB;
    int seq, nq, pos_first, flat_first;
    if (tiles != nullptr) {
        seq = tiles[2 * blockIdx.x];
        const int q0 = tiles[2 * blockIdx.x + 1];
        nq = min(max(1, SR_ROWS / GB), cu_q[seq + 1] - cu_q[seq] - q0);
        pos_first = seq_pos0[seq] + q0;
        flat_first = cu_q[seq] + q0;
    } else {
        seq = blockIdx.x;
        pos_first = row_pos[seq];
        nq = pos_first < 0 ? 0 : 1;
        flat_first = seq;
    }
    // this thread's two rows of the block: (query, head) and the keys it may see
    int lo[2], hi[2], head[2];
    size_t flat[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int R = wr * 16 + g + 8 * r, qi = R / GB, hh = hb * SR_ROWS + R % GB;
        const bool ok = qi < nq && hh < G;
        head[r] = ok ? kvh * G + hh : -1;
        flat[r] = (size_t)(flat_first + qi);
        hi[r] = ok ? pos_first + qi : -1;
        lo[r] = ok ? sr_first_key(hi[r], window, chunk) : 0;
    }
    const int kt_lo = nq > 0 ? sr_first_key(pos_first, window, chunk) / SR_KEYS : 0;
    const int kt_hi = nq > 0 ? (pos_first + nq - 1) / SR_KEYS : -1;
    const int per = (kt_hi - kt_lo + 1 + nsplit - 1) / nsplit;
    const int ka = kt_lo + split * per, kb = min(kt_hi, ka + per - 1);
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[SR_HALF / 8][4];
#pragma unroll
    for (int i = 0; i < SR_HALF / 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    if (ka <= kb) {
        const int* pt = page_table + (size_t)seq * pt_stride;
        sr_stage_keys(Ks, k_store, pt, ka, nkv, kvh);
        constexpr int CQ = HD / 8;
        for (int c = tid; c < SR_ROWS * CQ; c += SR_THREADS) {
            const int R = c / CQ, col = (c % CQ) * 8, qi = R / GB, hh = hb * SR_ROWS + R % GB;
            bf16* dst = Qs + R * SR_STR + col;
            if (qi < nq && hh < G)
                sr_cp16(dst, q + (size_t)(flat_first + qi) * ldq + (size_t)(kvh * G + hh) * HD + col);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        sr_commit();
        const bf16* qa = Qs + (wr * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * SR_STR + 8 * (lane >> 4);
        const bf16* pa = Ps + (wr * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * SR_PSTR + 8 * (lane >> 4);
        const int k_lane = (wc * 16 + (lane & 7) + 8 * (lane >> 4)) * SR_STR + 8 * ((lane >> 3) & 1);
        const int v_lane = (lane & 15) * SR_STR + wc * SR_HALF + 8 * (lane >> 4);
        // Turn kt takes the scores of half page kt and, side by side with them, P.V of half page kt - 1 (whose P the turn
        // before left in shared memory): two independent streams of products for every warp. One more turn ends it.
        for (int kt = ka; kt <= kb + 1; kt++) {
            sr_wait<0>();
            __syncthreads();       // half page kt is there; every warp has left the turn before, so the stage of kt - 2 is free
            if (kt + 1 <= kb) sr_stage_keys(Ks + ((kt + 1 - ka) % SR_STAGES) * SR_K_ELEMS, k_store, pt, kt + 1, nkv, kvh);
            sr_commit();
            const bf16* Kc = Ks + ((kt - ka) % SR_STAGES) * SR_K_ELEMS;
            const bf16* Kp = Ks + ((kt - ka + SR_STAGES - 1) % SR_STAGES) * SR_K_ELEMS;
            const bool scores = kt <= kb;
            float s[2][4];
#pragma unroll
            for (int i = 0; i < 2; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            if (scores && kt > ka) sr_products<true, true>(qa, Kc + k_lane, pa, Kp + v_lane, s, acc);
            else if (scores) sr_products<true, false>(qa, Kc + k_lane, pa, Kp + v_lane, s, acc);
            else sr_products<false, true>(qa, Kc + k_lane, pa, Kp + v_lane, s, acc);
            float mx[2] = {-INFINITY, -INFINITY};
            if (scores) {
                const int key0 = kt * SR_KEYS + wc * 16;
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const int key = key0 + nt * 8 + 2 * t + (c & 1), r = c >> 1;
                        const float v = (key >= lo[r] && key <= hi[r]) ? s[nt][c] * sl2 : -INFINITY;
                        s[nt][c] = v;
                        mx[r] = fmaxf(mx[r], v);
                    }
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    if (t == 0) smax[wc * SR_ROWS + wr * 16 + g + 8 * r] = mx[r];
                }
            }
            __syncthreads();       // the maxima of both warp columns are there; P of the turn before has been read
            if (!scores) break;
            float ms[2], alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const float other = smax[(wc ^ 1) * SR_ROWS + wr * 16 + g + 8 * r];
                const float m_new = fmaxf(m[r], fmaxf(mx[r], other));
                ms[r] = m_new == -INFINITY ? 0.f : m_new;
                alpha[r] = exp2f(m[r] - ms[r]);
                m[r] = m_new;
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const float p = exp2f(s[nt][c] - ms[c >> 1]);
                    s[nt][c] = p;
                    sum[c >> 1] += p;
                }
#pragma unroll
                for (int r = 0; r < 2; r++)
                    *reinterpret_cast<uint32_t*>(Ps + (wr * 16 + g + 8 * r) * SR_PSTR + wc * 16 + nt * 8 + 2 * t) =
                        sr_pack(s[nt][2 * r], s[nt][2 * r + 1]);
            }
            l[0] = l[0] * alpha[0] + sum[0];
            l[1] = l[1] * alpha[1] + sum[1];
#pragma unroll
            for (int i = 0; i < SR_HALF / 8; i++) {
                acc[i][0] *= alpha[0];
                acc[i][1] *= alpha[0];
                acc[i][2] *= alpha[1];
                acc[i][3] *= alpha[1];
            }
        }
    }
    // the row sums of the two warp columns meet
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (t == 0) ssum[wc * SR_ROWS + wr * 16 + g + 8 * r] = l[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = wr * 16 + g + 8 * r;
        const float lt = ssum[row] + ssum[SR_ROWS + row];
        if (nsplit > 1) {
            if (head[r] < 0) continue;
            const size_t part = (flat[r] * nh + head[r]) * nsplit + split;
            if (wc == 0 && t == 0) ws_ml[part * 2] = m[r], ws_ml[part * 2 + 1] = lt;
#pragma unroll
            for (int nt = 0; nt < SR_HALF / 8; nt++)
                *reinterpret_cast<float2*>(ws_acc + part * HDV + wc * SR_HALF + nt * 8 + 2 * t) =
                    make_float2(acc[nt][2 * r], acc[nt][2 * r + 1]);
            continue;
        }
        if (head[r] < 0) continue;
        const float inv = lt > 0.f ? out_scale / lt : 0.f;
        bf16* o = out + flat[r] * ldo + (size_t)head[r] * HDV + wc * SR_HALF + 2 * t;
#pragma unroll
        for (int nt = 0; nt < SR_HALF / 8; nt++)
            *reinterpret_cast<uint32_t*>(o + nt * 8) = sr_pack(acc[nt][2 * r] * inv, acc[nt][2 * r + 1] * inv);
    }
    // a padding row of a single-token step (no position): zeros out, or a part that counts for nothing
    if (tiles == nullptr && nq == 0) {
        for (int i = tid; i < GB * HDV; i += SR_THREADS) {
            const int hh = hb * SR_ROWS + i / HDV;
            if (hh >= G) continue;
            const size_t hd = (size_t)flat_first * nh + kvh * G + hh;
            if (nsplit > 1) {
                ws_acc[(hd * nsplit + split) * HDV + i % HDV] = 0.f;
                if (i % HDV == 0) ws_ml[(hd * nsplit + split) * 2] = -INFINITY, ws_ml[(hd * nsplit + split) * 2 + 1] = 0.f;
            } else {
                out[(size_t)flat_first * ldo + (size_t)(kvh * G + hh) * HDV + i % HDV] = __float2bfloat16_rn(0.f);
            }
        }
    }
}

// The parts of a split step put together: a block per (row, head), a thread per four value columns. M = the parts'
// largest maximum, w_s = 2^(m_s - M), L = sum_s l_s w_s, out = sum_s acc_s w_s / L * out_scale (maxima in the log2 domain).
constexpr int SR_MAX_SPLITS = 16;
__global__ void __launch_bounds__(HDV / 4)
attn_shared_rows_merge_kernel(const float* __restrict__ ws_acc, const float* __restrict__ ws_ml, bf16* out, long long ldo,
                              float out_scale, int nh, int nsplit) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.x / nh, h = blockIdx.x % nh;
    const float* ml = ws_ml + (size_t)blockIdx.x * nsplit * 2;
    const float4* acc = reinterpret_cast<const float4*>(ws_acc + (size_t)blockIdx.x * nsplit * HDV) + threadIdx.x;
    float w[SR_MAX_SPLITS];
    float M = -INFINITY, L = 0.f;
#pragma unroll
    for (int s = 0; s < SR_MAX_SPLITS; s++)
        if (s < nsplit) M = fmaxf(M, ml[2 * s]);
#pragma unroll
    for (int s = 0; s < SR_MAX_SPLITS; s++) {
        w[s] = (s < nsplit && M != -INFINITY) ? exp2f(ml[2 * s] - M) : 0.f;
        if (s < nsplit) L += ml[2 * s + 1] * w[s];
    }
    const float inv = L > 0.f ? out_scale / L : 0.f;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < SR_MAX_SPLITS; s++)
        if (s < nsplit) {
            const float4 v = acc[(size_t)s * (HDV / 4)];
            a.x = fmaf(v.x, w[s], a.x), a.y = fmaf(v.y, w[s], a.y), a.z = fmaf(v.z, w[s], a.z), a.w = fmaf(v.w, w[s], a.w);
        }
    uint2 o;
    o.x = sr_pack(a.x * inv, a.y * inv), o.y = sr_pack(a.z * inv, a.w * inv);
    bf16* dst = out + (size_t)b * ldo + (size_t)h * HDV + 4 * threadIdx.x;
    *reinterpret_cast<uint32_t*>(dst) = o.x;
    *reinterpret_cast<uint32_t*>(dst + 2) = o.y;
}

// tiles (or null for a single-token step of n_items rows), n_items: tiles or rows. nsplit > 1 only for single tokens.
DK_EXPORT int dk_attn_shared_rows_bf16(const void* q, long long ldq, void* out, long long ldo, float out_scale,
                                       const void* k_store, const int* tiles, int n_items, const int* cu_q,
                                       const int* seq_pos0, const int* row_pos, const int* page_table, int pt_stride,
                                       int nh, int nkv, int window, int chunk, float scale, int nsplit, float* ws_acc,
                                       float* ws_ml, cudaStream_t st) {
    if (nh % nkv != 0 || nsplit < 1 || nsplit > SR_MAX_SPLITS || (nsplit > 1 && (tiles != nullptr || ws_acc == nullptr || ws_ml == nullptr)))
        return (int)cudaErrorInvalidValue;
    if (ldq % 8 != 0 || ldo % 2 != 0 || ((uintptr_t)q & 15) != 0 || ((uintptr_t)out & 3) != 0) return (int)cudaErrorInvalidValue;
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(attn_shared_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SR_SMEM_BYTES);
        attr = true;
    }
    const int G = nh / nkv, HB = (G + SR_ROWS - 1) / SR_ROWS;
    int e = dk_launch(attn_shared_rows_kernel, dim3(n_items, nkv * HB, nsplit), dim3(SR_THREADS), SR_SMEM_BYTES, st,
                      (const bf16*)q, ldq, (bf16*)out, ldo, out_scale, (const bf16*)k_store, tiles, cu_q, seq_pos0, row_pos,
                      page_table, pt_stride, nh, nkv, window, chunk, scale * 1.4426950408889634f, nsplit, ws_acc, ws_ml);
    if (e != 0 || nsplit == 1) return e;
    return dk_launch(attn_shared_rows_merge_kernel, dim3(n_items * nh), dim3(HDV / 4), 0, st, (const float*)ws_acc,
                     (const float*)ws_ml, (bf16*)out, ldo, out_scale, nh, nsplit);
}

DK_EXPORT int dk_attn_shared_rows_tile_queries(int group) { return max(1, SR_ROWS / min(group, SR_ROWS)); }
