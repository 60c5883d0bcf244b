// bfloat16 attention with a chunk mask or window, logarithmic distance bias, sink and output gate (see
// attention_masked.cu for the float32-arithmetic form of the same options) on the tensor cores:
// mma.sync m16n8k16 with float32 scores, softmax and accumulators. Built once per pair of head sizes
// with -DHD=<key size> -DHDV=<value size>, both multiples of 16 up to 256.
//
//  * prefill: ragged batch of query portions; a block owns 64 consecutive queries of one sequence and one
//    query head (4 warps x 16 rows) and walks the key pages from the first one any of its rows may see
//    (the start of the chunk of its first row, or of its window) up to its diagonal. Pages are staged by
//    cp.async, two stages deep. The bias is taken off every score in the log2 domain:
//    r1 * ln(1 + r2 d) * log2(e) = r1 * log2(1 + r2 d). P is rounded to bfloat16 before P.V; row sums use
//    the unrounded values. The sink joins the denominator after the last page; the gate and the constant
//    factor are applied to the float32 result before it is stored.
//  * decode: one query token per sequence; a block owns the query heads that share a kv head: scores of
//    all visible keys into shared memory (a thread per key), softmax with the sink over them, then P.V with
//    eight output columns and every 16th (or so) key a thread, the partial sums meeting in shared memory. A
//    chunk or window bounds the keys, so there is no split over blocks.
#include "attention_mma.cuh"

#ifndef HDV
#error "compile with -DHDV=<value head size>"
#endif
static_assert(HDV % 16 == 0 && HDV >= 16 && HDV <= 256, "value head size must be a multiple of 16 up to 256");

constexpr int VSTR = HDV + 8;
constexpr int KTILE = DK_PAGE * KSTR, VTILE = DK_PAGE * VSTR;
constexpr int MSTAGE = KTILE + VTILE;
constexpr size_t MSMEM_BYTES = 2 * MSTAGE * sizeof(bf16);

__device__ __forceinline__ void stage_page_kv(bf16* stage, const bf16* k_store, const bf16* v_store, int page, int nkv,
                                              int kvh) {
    const size_t koff = kv_offset(page, nkv, kvh, 0, HD), voff = kv_offset(page, nkv, kvh, 0, HDV);
    constexpr int CK = HD / 8, CV = HDV / 8;
    for (int c = threadIdx.x; c < DK_PAGE * CK; c += blockDim.x) {
        const int row = c / CK, col = (c % CK) * 8;
        cp_async16(stage + row * KSTR + col, k_store + koff + (size_t)row * HD + col);
    }
    // without a store of values (v_store null) a value row is the first HDV numbers of its key row
    for (int c = threadIdx.x; c < DK_PAGE * CV; c += blockDim.x) {
        const int row = c / CV, col = (c % CV) * 8;
        cp_async16(stage + KTILE + row * VSTR + col,
                   v_store != nullptr ? v_store + voff + (size_t)row * HDV + col : k_store + koff + (size_t)row * HD + col);
    }
}

// One warp: 16 query rows against the 64 staged keys of a page. Row r (0: lane group g, 1: g+8) sits at
// position hi[r] and may see keys lo[r] <= position <= hi[r]. Scores in the log2 domain.
__device__ __forceinline__ void warp_attend_masked(const uint32_t (&qf)[HD / 16][4], const bf16* Ks, const bf16* Vs,
                                                   int key0, const int (&lo)[2], const int (&hi)[2], float sl2, float b1,
                                                   float b2, float (&m)[2], float (&l)[2], float (&acc)[HDV / 8][4]) {
    constexpr int NKEYS = DK_PAGE;
    const int lane = threadIdx.x & 31, t = lane & 3;
    float s[NKEYS / 8][4];
#pragma unroll
    for (int i = 0; i < NKEYS / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const int j = lane >> 3;
#pragma unroll
    for (int np = 0; np < NKEYS / 16; np++) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t b[4];
            ldsm_x4(b, Ks + (np * 16 + (lane & 7) + 8 * (j >> 1)) * KSTR + ks * 16 + 8 * (j & 1));
            mma16816(s[2 * np], qf[ks], b[0], b[1]);
            mma16816(s[2 * np + 1], qf[ks], b[2], b[3]);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NKEYS / 8; nt++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int key = key0 + nt * 8 + 2 * t + (c & 1), r = c >> 1;
            float v = -INFINITY;
            if (key >= lo[r] && key <= hi[r]) {
                v = s[nt][c] * sl2;
                if (b1 != 0.f) v -= b1 * __log2f(fmaf(b2, (float)(hi[r] - key), 1.f));
            }
            s[nt][c] = v;
            mx[r] = fmaxf(mx[r], v);
        }
    }
    float ms[2], alpha[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        ms[r] = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = exp2f(m[r] - ms[r]);
        m[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NKEYS / 8; nt++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const float p = exp2f(s[nt][c] - ms[c >> 1]);
            s[nt][c] = p;
            sum[c >> 1] += p;
        }
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
#pragma unroll
    for (int kk = 0; kk < NKEYS / 16; kk++) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < HDV / 16; dp++) {
            uint32_t b[4];
            ldsm_x4_trans(b, Vs + (kk * 16 + (lane & 15)) * VSTR + dp * 16 + 8 * (lane >> 4));
            mma16816(acc[2 * dp], a, b[0], b[1]);
            mma16816(acc[2 * dp + 1], a, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ int first_key(int pos, int window, int chunk) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    return lo;
}

// grid (nh, tiles). tiles[2i] = sequence, tiles[2i+1] = first query of the tile within the sequence's
// portion. cu_q: first flat row of each portion; seq_pos0: tokens cached before it (the portion's own
// keys are in the cache when this runs). q, gate and out are rows of wider matrices (ldq, ldg, ldo).
__global__ void __launch_bounds__(128)
attn_masked_prefill_kernel(const bf16* q, long long ldq, bf16* out, long long ldo, const bf16* gate, long long ldg,
                           float out_scale, const bf16* k_store, const bf16* v_store, const int* tiles, const int* cu_q,
                           const int* seq_pos0, const int* page_table, int pt_stride, int nh, int nkv, int window,
                           int chunk, float sl2, const float* __restrict__ r1, const float* __restrict__ r2,
                           const float* __restrict__ sink) {
    extern __shared__ __align__(16) bf16 smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int seq = tiles[2 * blockIdx.y], q0 = tiles[2 * blockIdx.y + 1];
    const int h = blockIdx.x, kvh = h / (nh / nkv);
    const int q_len = cu_q[seq + 1] - cu_q[seq];
    const int pos0 = seq_pos0[seq];
    const int rows_here = min(64, q_len - q0);
    const int* pt = page_table + (size_t)seq * pt_stride;
    const float b1 = r1 ? r1[h] : 0.f, b2 = r1 ? r2[h] : 0.f;

    const int r0 = q0 + warp * 16 + g, r1w = r0 + 8;  // rows within the portion
    const bool ok0 = r0 < q_len, ok1 = r1w < q_len;
    const size_t flat0 = (size_t)(cu_q[seq] + r0), flat1 = (size_t)(cu_q[seq] + r1w);
    uint32_t qf[HD / 16][4];
    load_q_frags(qf, ok0 ? q + flat0 * ldq + (size_t)h * HD : nullptr, ok1 ? q + flat1 * ldq + (size_t)h * HD : nullptr);
    int lo[2], hi[2];
    hi[0] = ok0 ? pos0 + r0 : -1;
    hi[1] = ok1 ? pos0 + r1w : -1;
    lo[0] = ok0 ? first_key(hi[0], window, chunk) : 0;
    lo[1] = ok1 ? first_key(hi[1], window, chunk) : 0;
    // keys this warp's 16 rows can see at all (the first key a row sees never moves back as the position grows)
    const int w_first = pos0 + q0 + warp * 16;
    const int w_hi = min(w_first + 15, pos0 + q_len - 1);
    const int w_lo = first_key(w_first, window, chunk);

    const int max_pos = pos0 + q0 + rows_here - 1;
    const int min_pos = pos0 + q0;
    const int jt_hi = max_pos / DK_PAGE;
    const int jt_lo = first_key(min_pos, window, chunk) / DK_PAGE;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[HDV / 8][4];
#pragma unroll
    for (int i = 0; i < HDV / 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    stage_page_kv(smem, k_store, v_store, pt[jt_lo], nkv, kvh);
    cp_async_commit();
    for (int jt = jt_lo; jt <= jt_hi; jt++) {
        const int cur = (jt - jt_lo) & 1;
        if (jt < jt_hi) stage_page_kv(smem + (cur ^ 1) * MSTAGE, k_store, v_store, pt[jt + 1], nkv, kvh);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = jt * DK_PAGE;
        if (key0 <= w_hi && key0 + DK_PAGE - 1 >= w_lo && warp * 16 < rows_here) {
            const bf16* Ks = smem + cur * MSTAGE;
            warp_attend_masked(qf, Ks, Ks + KTILE, key0, lo, hi, sl2, b1, b2, m, l, acc);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    float inv[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        float a = 1.f;
        if (sink) {  // one more term of the denominator, in the log2 domain like the scores
            const float s2 = sink[h] * 1.4426950408889634f;
            const float m_new = fmaxf(m[r], s2);
            a = exp2f(m[r] - m_new);
            l[r] = l[r] * a + exp2f(s2 - m_new);
        }
        inv[r] = a / l[r] * out_scale;
    }
#pragma unroll
    for (int nt = 0; nt < HDV / 8; nt++) {
        const int d = nt * 8 + 2 * t;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            if (!(r ? ok1 : ok0)) continue;
            const size_t flat = r ? flat1 : flat0;
            float v0 = acc[nt][2 * r] * inv[r], v1 = acc[nt][2 * r + 1] * inv[r];
            if (gate) {
                const __nv_bfloat162 gg = *reinterpret_cast<const __nv_bfloat162*>(gate + flat * ldg + (size_t)h * HDV + d);
                v0 *= 1.f / (1.f + __expf(-__bfloat162float(gg.x)));
                v1 *= 1.f / (1.f + __expf(-__bfloat162float(gg.y)));
            }
            *reinterpret_cast<uint32_t*>(out + flat * ldo + (size_t)h * HDV + d) = pack_bf16(v0, v1);
        }
    }
}

// -------------------------------------------------------------------------------------- decode
// grid (nkv, rows). Block: the G query heads of one kv head for one row (sequence); 256 threads.
// Shared memory: q [G][HD] float, scores [G][span] float with span = the most keys a row can see, and
// 32 KB in which the threads' partial sums of P.V meet.
constexpr int MD_THREADS = 256;
constexpr int MD_RED_FLOATS = MD_THREADS * 4 * 8;

__global__ void __launch_bounds__(MD_THREADS)
attn_masked_decode_kernel(const bf16* q, long long ldq, bf16* out, long long ldo, const bf16* gate, long long ldg,
                          float out_scale, const bf16* k_store, const bf16* v_store, const int* row_pos,
                          const int* page_table, int pt_stride, int nh, int nkv, int window, int chunk, float scale,
                          const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink,
                          int span, const bf16* k_new, const bf16* v_new, long long ldkv, bf16* k_out, bf16* v_out,
                          int nsplit, float* ws_acc, float* ws_ml) {
    extern __shared__ __align__(16) float fsm[];
    const int G = nh / nkv, kvh = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, split = blockIdx.z;
    float* red = fsm;                       // [key split][4 heads][HDV]
    float* qs = fsm + MD_RED_FLOATS;        // [G][HD]
    float* sc = qs + G * HD;                // [G][span]
    pdl_wait();
    pdl_launch_dependents();
    const int pos = row_pos[b];
    if (pos < 0) {
        for (int i = tid; i < G * HDV; i += MD_THREADS) out[(size_t)b * ldo + (size_t)kvh * G * HDV + i] = __float2bfloat16_rn(0.f);
        return;
    }
    // With nsplit > 1 the visible keys are dealt out to nsplit blocks in equal runs; each leaves its part of the
    // softmax (maximum, sum, unnormalised P.V) for the merge kernel. The run that ends at the token's own position
    // belongs to the block that also stores the token's key and value.
    const int lo_all = first_key(pos, window, chunk), n_all = pos - lo_all + 1;
    const int per = (n_all + nsplit - 1) / nsplit;
    const int lo = lo_all + split * per, n = max(0, min(per, n_all - split * per));
    const int* pt = page_table + (size_t)b * pt_stride;
    if (nsplit > 1 && n == 0) {                   // nothing for this block: a part that counts for nothing
        for (int i = tid; i < G; i += MD_THREADS) {
            float* ml = ws_ml + (((size_t)b * nh + kvh * G + i) * nsplit + split) * 2;
            ml[0] = -INFINITY, ml[1] = 0.f;
        }
        for (int i = tid; i < G * HDV; i += MD_THREADS)
            ws_acc[(((size_t)b * nh + kvh * G + i / HDV) * nsplit + split) * HDV + i % HDV] = 0.f;
        return;
    }
    if (k_new != nullptr && lo + n - 1 == pos) {   // the token's own key and value go into the cache here, by the block that reads them
        const int page = pt[pos / DK_PAGE];
        for (int i = tid; i < HD; i += MD_THREADS)
            k_out[kv_offset(page, nkv, kvh, pos % DK_PAGE, HD) + i] = k_new[(size_t)b * ldkv + (size_t)kvh * HD + i];
        if (v_out != nullptr)
            for (int i = tid; i < HDV; i += MD_THREADS)
                v_out[kv_offset(page, nkv, kvh, pos % DK_PAGE, HDV) + i] = v_new[(size_t)b * ldkv + (size_t)kvh * HDV + i];
    }
    for (int i = tid; i < G * HD; i += MD_THREADS) qs[i] = __bfloat162float(q[(size_t)b * ldq + (size_t)kvh * G * HD + i]);
    __syncthreads();
    // scores: a thread per key, the key row read in 16-byte pieces, four heads from one read
    for (int jj = tid; jj < n; jj += MD_THREADS) {
        const int j = lo + jj;
        const bf16* kr = k_store + kv_offset(pt[j / DK_PAGE], nkv, kvh, j % DK_PAGE, HD);
        float dot[4];
        for (int g0 = 0; g0 < G; g0 += 4) {       // later passes over the key row hit the L1
            const int gn = min(4, G - g0);
            dot[0] = dot[1] = dot[2] = dot[3] = 0.f;
#pragma unroll 4
            for (int c = 0; c < HD; c += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(kr + c);
                const bf16* kv8 = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const float kf = __bfloat162float(kv8[e]);
#pragma unroll
                    for (int gg = 0; gg < 4; gg++)
                        if (gg < gn) dot[gg] = fmaf(qs[(g0 + gg) * HD + c + e], kf, dot[gg]);
                }
            }
#pragma unroll
            for (int gg = 0; gg < 4; gg++)
                if (gg < gn) {
                    const int h = kvh * G + g0 + gg;
                    float s = dot[gg] * scale;
                    if (r1) s -= r1[h] * log1pf(r2[h] * (float)(pos - j));
                    sc[(g0 + gg) * span + jj] = s;
                }
        }
    }
    __syncthreads();
    // softmax with the sink, head by head: a warp per head at a time; the weights leave normalised
    const int lane = tid & 31, warp = tid >> 5;
    for (int gq = warp; gq < G; gq += MD_THREADS / 32) {
        const int h = kvh * G + gq;
        float mx = (sink && nsplit == 1) ? sink[h] : -INFINITY;
        for (int jj = lane; jj < n; jj += 32) mx = fmaxf(mx, sc[gq * span + jj]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int jj = lane; jj < n; jj += 32) {
            const float p = expf(sc[gq * span + jj] - mx);
            sc[gq * span + jj] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        if (nsplit > 1) {                         // the part's maximum and sum; its weights stay unnormalised
            if (lane == 0) {
                float* ml = ws_ml + (((size_t)b * nh + h) * nsplit + split) * 2;
                ml[0] = mx, ml[1] = sum;
            }
            continue;
        }
        if (sink) sum += expf(sink[h] - mx);
        const float inv = out_scale / sum;
        for (int jj = lane; jj < n; jj += 32) sc[gq * span + jj] *= inv;
    }
    __syncthreads();
    // P.V: a thread takes 8 output columns and every KS-th key, for four heads at a time from one read of the value
    // row; the KS partial sums of a column meet in shared memory
    constexpr int CGN = HDV / 8, KS = MD_THREADS / CGN;
    const int cgp = tid % CGN, ks = tid / CGN;
    for (int g0 = 0; g0 < G; g0 += 4) {
        const int gn = min(4, G - g0);
        float acc[4][8];
#pragma unroll
        for (int gg = 0; gg < 4; gg++)
#pragma unroll
            for (int e = 0; e < 8; e++) acc[gg][e] = 0.f;
        if (ks < KS) {
#pragma unroll 4
            for (int jj = ks; jj < n; jj += KS) {
                const int j = lo + jj;
                const uint4 raw = *reinterpret_cast<const uint4*>(
                    (v_store != nullptr ? v_store + kv_offset(pt[j / DK_PAGE], nkv, kvh, j % DK_PAGE, HDV)
                                        : k_store + kv_offset(pt[j / DK_PAGE], nkv, kvh, j % DK_PAGE, HD)) + cgp * 8);
                const bf16* v8 = reinterpret_cast<const bf16*>(&raw);
                float vf[8];
#pragma unroll
                for (int e = 0; e < 8; e++) vf[e] = __bfloat162float(v8[e]);
#pragma unroll
                for (int gg = 0; gg < 4; gg++)
                    if (gg < gn) {
                        const float p = sc[(g0 + gg) * span + jj];
#pragma unroll
                        for (int e = 0; e < 8; e++) acc[gg][e] = fmaf(p, vf[e], acc[gg][e]);
                    }
            }
#pragma unroll
            for (int gg = 0; gg < 4; gg++)
#pragma unroll
                for (int e = 0; e < 8; e++) red[(ks * 4 + gg) * HDV + cgp * 8 + e] = acc[gg][e];
        }
        __syncthreads();
        for (int i = tid; i < gn * HDV; i += MD_THREADS) {
            const int gg = i / HDV, d = i % HDV;
            float a = 0.f;
            for (int kk = 0; kk < KS; kk++) a += red[(kk * 4 + gg) * HDV + d];
            const size_t col = (size_t)(kvh * G + g0 + gg) * HDV + d;
            if (nsplit > 1) {
                ws_acc[(((size_t)b * nh + kvh * G + g0 + gg) * nsplit + split) * HDV + d] = a;
                continue;
            }
            if (gate) a *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)b * ldg + col])));
            out[(size_t)b * ldo + col] = __float2bfloat16_rn(a);
        }
        __syncthreads();
    }
}

// The parts of a split single-token attention put together: a warp per (row, head). M = max(sink, the parts'
// maxima), L = e^(sink - M) + sum_s l_s e^(m_s - M), out = sum_s acc_s e^(m_s - M) / L * sigmoid(gate) * out_scale.
__global__ void attn_masked_merge_kernel(const float* ws_acc, const float* ws_ml, bf16* out, long long ldo, const bf16* gate,
                                         long long ldg, float out_scale, const float* __restrict__ sink, const int* row_pos,
                                         int n_rows, int nh, int nsplit) {
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
    float M = sink ? sink[h] : -INFINITY;
    for (int s = 0; s < nsplit; s++) M = fmaxf(M, ml[2 * s]);
    float L = sink ? expf(sink[h] - M) : 0.f;
    for (int s = 0; s < nsplit; s++) L += ml[2 * s + 1] * expf(ml[2 * s] - M);
    const float inv = out_scale / L;
    for (int d = lane; d < HDV; d += 32) {
        float a = 0.f;
        for (int s = 0; s < nsplit; s++) a = fmaf(acc[(size_t)s * HDV + d], expf(ml[2 * s] - M), a);
        a *= inv;
        if (gate) a *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)b * ldg + (size_t)h * HDV + d])));
        o[d] = __float2bfloat16_rn(a);
    }
}

DK_EXPORT int dk_attn_masked_prefill_bf16(const void* q, long long ldq, void* out, long long ldo, const void* gate,
                                          long long ldg, float out_scale, const void* k_store, const void* v_store,
                                          const int* tiles, int n_tiles, const int* cu_q, const int* seq_pos0,
                                          const int* page_table, int pt_stride, int nh, int nkv, int window, int chunk,
                                          float scale, const float* r1, const float* r2, const float* sink,
                                          cudaStream_t st) {
    if (nh % nkv != 0) return (int)cudaErrorInvalidValue;
    static bool attr = false;
    if (!attr && MSMEM_BYTES > 48 * 1024) {
        cudaFuncSetAttribute(attn_masked_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MSMEM_BYTES);
        attr = true;
    }
    return dk_launch(attn_masked_prefill_kernel, dim3(nh, n_tiles), dim3(128), MSMEM_BYTES, st, (const bf16*)q, ldq,
                     (bf16*)out, ldo, (const bf16*)gate, ldg, out_scale, (const bf16*)k_store, (const bf16*)v_store, tiles,
                     cu_q, seq_pos0, page_table, pt_stride, nh, nkv, window, chunk, scale * 1.4426950408889634f, r1, r2,
                     sink);
}

// k_new, v_new (or null): rows [n_rows, nkv*HD] / [n_rows, nkv*HDV] of the step's projection, ldkv elements apart,
// which the kernel stores at each row's position before it reads the cache (no separate cache-write launch).
// nsplit > 1: the keys of a row in nsplit runs, a block each, then the merge kernel; ws_acc [rows, nh, nsplit, HDV]
// and ws_ml [rows, nh, nsplit, 2] float32 scratch; span is then the most keys of a run.
// span: the most keys any row sees (the chunk, the window, or the longest sequence's length, rounded up by the caller)
DK_EXPORT int dk_attn_masked_decode_bf16(const void* q, long long ldq, void* out, long long ldo, const void* gate,
                                         long long ldg, float out_scale, const void* k_store, const void* v_store,
                                         const int* row_pos, const int* page_table, int pt_stride, int n_rows, int nh,
                                         int nkv, int window, int chunk, float scale, const float* r1, const float* r2,
                                         const float* sink, int span, const void* k_new, const void* v_new, long long ldkv,
                                         int nsplit, float* ws_acc, float* ws_ml, cudaStream_t st) {
    if (nh % nkv != 0 || nsplit < 1 || (nsplit > 1 && (ws_acc == nullptr || ws_ml == nullptr))) return (int)cudaErrorInvalidValue;
    const int G = nh / nkv;
    const size_t smem = sizeof(float) * ((size_t)MD_RED_FLOATS + (size_t)G * HD + (size_t)G * span);
    if (smem > 224 * 1024) return (int)cudaErrorInvalidValue;
    static size_t attr = 48 * 1024;
    if (smem > attr) {
        cudaFuncSetAttribute(attn_masked_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr = smem;
    }
    int e = dk_launch(attn_masked_decode_kernel, dim3(nkv, n_rows, nsplit), dim3(MD_THREADS), smem, st, (const bf16*)q, ldq,
                      (bf16*)out, ldo, (const bf16*)gate, ldg, out_scale, (const bf16*)k_store, (const bf16*)v_store, row_pos,
                      page_table, pt_stride, nh, nkv, window, chunk, scale, r1, r2, sink, span, (const bf16*)k_new,
                      (const bf16*)v_new, ldkv, (bf16*)k_store, (bf16*)v_store, nsplit, ws_acc, ws_ml);
    if (e != 0 || nsplit == 1) return e;
    return dk_launch(attn_masked_merge_kernel, dim3((n_rows * nh + 3) / 4), dim3(128), 0, st, (const float*)ws_acc,
                     (const float*)ws_ml, (bf16*)out, ldo, (const bf16*)gate, ldg, out_scale, sink, row_pos, n_rows, nh, nsplit);
}
