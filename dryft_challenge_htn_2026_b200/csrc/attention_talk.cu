// Grouped-query softmax attention over the paged cache in which the heads' scores are mixed before the softmax:
//     s_g(i, j) = q_g(i) . k_kv(g)(j) * scale,    s'_h(i, j) = sum_g talk[h][g] s_g(i, j),    p_h = softmax_j s'_h,
//     o_h(i) = sum_j p_h(i, j) v_kv(h)(j),
// causal, optionally inside a sliding window (position i sees j with 0 <= i - j < window). A query needs the scores
// of all its heads for a key at once, so a block takes one token row with all its heads and walks the row's keys in
// runs of up to 32: the run's key and value rows of every kv head are staged in shared memory (float32), every
// (head, key) pair gets its score, the scores are mixed, each head's running maximum and sum move on (online softmax),
// and every (head, value column) adds its part. All arithmetic is float32 whatever the storage type; q and the output
// are rows of wider matrices. Every phase (whole prompts, continued portions, single tokens; rows with position < 0
// are padding).
#include "common.cuh"

#define AT_THREADS 256
#define AT_WARPS (AT_THREADS / 32)
#define AT_MAX_OUT 16              // (head, value column) pairs a thread may own

template <typename T>
__global__ void __launch_bounds__(AT_THREADS)
attention_talk_kernel(const T* q, long long ldq, T* out, long long ldo, float out_scale, const T* k_store, const T* v_store,
                      const int* row_pos, const int* row_seq, const int* page_table, int pt_stride, int nh, int nkv, int hd,
                      int hdv, int window, float scale, const float* __restrict__ talk, int KC) {
    extern __shared__ float at_smem[];
    const int hdp = hd + 1;                              // rows of keys one float apart from a multiple of the banks
    float* qs = at_smem;                                 // [nh][hd]
    float* tk = qs + nh * hd;                            // [nh][nh], times scale
    float* ks = tk + nh * nh;                            // [nkv][KC][hd + 1]
    float* vs = ks + (size_t)nkv * KC * hdp;             // [nkv][KC][hdv]
    float* sc = vs + (size_t)nkv * KC * hdv;             // [nh][KC] raw scores, then the weights
    float* run_m = sc + nh * KC;                         // [nh] running maximum
    float* run_l = run_m + nh;                           // [nh] running sum
    float* run_f = run_l + nh;                           // [nh] factor of this run on what was gathered before
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = row_pos[t];
    const int n_out = nh * hdv;
    if (pos < 0) {
        for (int i = tid; i < n_out; i += AT_THREADS) out[(size_t)t * ldo + i] = from_f<T>(0.f);
        return;
    }
    const int group = nh / nkv;
    const int* pt = page_table + (size_t)row_seq[t] * pt_stride;
    for (int i = tid; i < nh * hd; i += AT_THREADS) qs[i] = to_f(q[(size_t)t * ldq + i]);
    for (int i = tid; i < nh * nh; i += AT_THREADS) tk[i] = talk[i] * scale;
    for (int i = tid; i < nh; i += AT_THREADS) { run_m[i] = -INFINITY; run_l[i] = 0.f; }
    float acc[AT_MAX_OUT];
#pragma unroll
    for (int i = 0; i < AT_MAX_OUT; i++) acc[i] = 0.f;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    for (int j0 = lo; j0 <= pos; j0 += KC) {
        const int nk = min(KC, pos - j0 + 1);
        __syncthreads();                                 // the run before is done with ks, vs and sc
        for (int i = tid; i < nkv * nk * hd; i += AT_THREADS) {
            const int d = i % hd, jj = (i / hd) % nk, g = i / (hd * nk);
            const int j = j0 + jj;
            ks[((size_t)g * KC + jj) * hdp + d] = to_f(k_store[kv_offset(pt[j / DK_PAGE], nkv, g, j % DK_PAGE, hd) + d]);
        }
        for (int i = tid; i < nkv * nk * hdv; i += AT_THREADS) {
            const int d = i % hdv, jj = (i / hdv) % nk, g = i / (hdv * nk);
            const int j = j0 + jj;
            vs[((size_t)g * KC + jj) * hdv + d] = to_f(v_store[kv_offset(pt[j / DK_PAGE], nkv, g, j % DK_PAGE, hdv) + d]);
        }
        __syncthreads();
        // raw scores of every (head, key) pair of the run
        for (int i = tid; i < nh * nk; i += AT_THREADS) {
            const int jj = i % nk, g = i / nk;
            const float* qr = qs + g * hd;
            const float* kr = ks + ((size_t)(g / group) * KC + jj) * hdp;
            float dot = 0.f;
            for (int d = 0; d < hd; d++) dot = fmaf(qr[d], kr[d], dot);
            sc[g * KC + jj] = dot;
        }
        __syncthreads();
        // mixed scores and the online softmax: a warp a head, a lane a key; the mixed scores stay in registers until
        // every warp has read the raw ones
        float mixed[(64 + AT_WARPS - 1) / AT_WARPS];
        {
            int n = 0;
            for (int h = warp; h < nh; h += AT_WARPS, n++) {
                float s = -INFINITY;
                if (lane < nk) {
                    s = 0.f;
                    for (int g = 0; g < nh; g++) s = fmaf(tk[h * nh + g], sc[g * KC + lane], s);
                }
                mixed[n] = s;
            }
        }
        __syncthreads();
        {
            int n = 0;
            for (int h = warp; h < nh; h += AT_WARPS, n++) {
                const float s = mixed[n];
                const float m_old = run_m[h];
                const float m_new = fmaxf(m_old, warp_max(s));
                const float p = lane < nk ? expf(s - m_new) : 0.f;
                const float f = expf(m_old - m_new);          // 0 on the first run: m_old = -inf
                const float l = run_l[h] * f + warp_sum(p);
                if (lane < KC) sc[h * KC + lane] = p;
                __syncwarp();
                if (lane == 0) { run_m[h] = m_new; run_l[h] = l; run_f[h] = f; }
            }
        }
        __syncthreads();
        // every (head, value column) takes the run's weighted values
#pragma unroll
        for (int n = 0; n < AT_MAX_OUT; n++) {
            const int i = tid + n * AT_THREADS;
            if (i < n_out) {
                const int h = i / hdv, c = i % hdv;
                const float* pr = sc + h * KC;
                const float* vr = vs + (size_t)(h / group) * KC * hdv + c;
                float a = acc[n] * run_f[h];
                for (int jj = 0; jj < nk; jj++) a = fmaf(pr[jj], vr[(size_t)jj * hdv], a);
                acc[n] = a;
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < AT_MAX_OUT; n++) {
        const int i = tid + n * AT_THREADS;
        if (i < n_out) out[(size_t)t * ldo + i] = from_f<T>(acc[n] / run_l[i / hdv] * out_scale);
    }
}

// shared memory of a block for runs of KC keys
static size_t talk_smem(int nh, int nkv, int hd, int hdv, int KC) {
    return sizeof(float) * ((size_t)nh * hd + (size_t)nh * nh + (size_t)nkv * KC * (hd + 1) + (size_t)nkv * KC * hdv +
                            (size_t)nh * KC + 3 * (size_t)nh);
}

DK_EXPORT int dk_attention_talk(int dtype, const void* q, long long ldq, void* out, long long ldo, float out_scale,
                                const void* k_store, const void* v_store, const int* row_pos, const int* row_seq,
                                const int* page_table, int pt_stride, int n_tok, int nh, int nkv, int hd, int hdv, int window,
                                float scale, const float* talk, cudaStream_t st) {
    if (nh < 1 || nh > 64 || nkv < 1 || nh % nkv || hd < 1 || hdv < 1 || nh * hdv > AT_MAX_OUT * AT_THREADS || talk == nullptr)
        return (int)cudaErrorInvalidValue;
    int KC = 32;
    while (KC > 4 && talk_smem(nh, nkv, hd, hdv, KC) > 96 * 1024) KC >>= 1;     // two blocks an SM where the heads allow
    const size_t smem = talk_smem(nh, nkv, hd, hdv, KC);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_talk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return dk_launch(attention_talk_kernel<float>, dim3(n_tok), dim3(AT_THREADS), smem, st, (const float*)q, ldq, (float*)out, ldo,
                         out_scale, (const float*)k_store, (const float*)v_store, row_pos, row_seq, page_table, pt_stride, nh, nkv,
                         hd, hdv, window, scale, talk, KC);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(attention_talk_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return dk_launch(attention_talk_kernel<bf16>, dim3(n_tok), dim3(AT_THREADS), smem, st, (const bf16*)q, ldq, (bf16*)out, ldo,
                     out_scale, (const bf16*)k_store, (const bf16*)v_store, row_pos, row_seq, page_table, pt_stride, nh, nkv, hd,
                     hdv, window, scale, talk, KC);
}
