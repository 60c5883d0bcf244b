// Grouped-query softmax attention over the paged cache with the options a mixer may switch on:
//   * key and value heads of different sizes (hd, hdv), kept in two stores of their own,
//   * a chunk mask (a query at position i sees j <= i with floor(j / chunk) == floor(i / chunk)) and/or
//     a sliding window,
//   * a distance bias taken off the score: r1_h * ln(1 + r2_h * (i - j)),
//   * a sink: exp(sink_h) joins the softmax's denominator and nothing else,
//   * a cap on the score, cap * tanh(score / cap), before the masks,
//   * first tokens that a window keeps: key j < keep_first stays in sight of every later query,
//   * an output gate: the head's output times sigmoid of a gate row, and a constant factor.
// One warp per (token, query head), every phase (whole prompts, continued portions, single tokens);
// all arithmetic in float32 whatever the storage type. q, the gate and the output are rows of wider
// matrices (a fused projection, a buffer shared with another mixer), so each comes with a row stride.
#include "common.cuh"

// k and v heads of a fused projection row into each token's place in the paged stores
// k_store [pages, nkv, PAGE, hd], v_store [pages, nkv, PAGE, hdv]. Rows with position < 0 are skipped.
template <typename T>
__global__ void kv_write_kernel(const T* k, const T* v, long long ld, T* k_store, T* v_store, const int* row_pos,
                                const int* row_seq, const int* page_table, int pt_stride, int n_tok, int nkv, int hd,
                                int hdv) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = row_pos[t];
    if (pos < 0) return;
    const int page = page_table[(size_t)row_seq[t] * pt_stride + pos / DK_PAGE];
    if (page < 0) return;
    const int in_page = pos % DK_PAGE;
    for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x)
        k_store[kv_offset(page, nkv, i / hd, in_page, hd) + i % hd] = k[(size_t)t * ld + i];
    if (v_store == nullptr) return;        // values are the key rows' first numbers: nothing of their own to store
    for (int i = threadIdx.x; i < nkv * hdv; i += blockDim.x)
        v_store[kv_offset(page, nkv, i / hdv, in_page, hdv) + i % hdv] = v[(size_t)t * ld + i];
}

// NR: coordinates of a head that a lane holds (head sizes up to 32 * NR)
template <typename T, int NR>
__global__ void attention_masked_kernel(const T* q, long long ldq, T* out, long long ldo, const T* gate, long long ldg,
                                        float out_scale, const T* k_store, const T* v_store, const int* row_pos,
                                        const int* row_seq, const int* page_table, int pt_stride, int n_tok, int nh,
                                        int nkv, int hd, int hdv, int window, int chunk, float scale,
                                        const float* __restrict__ r1, const float* __restrict__ r2,
                                        const float* __restrict__ sink, float softcap, int keep_first) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (long long)n_tok * nh) return;
    const int t = (int)(wid / nh), h = (int)(wid % nh);
    T* o = out + (size_t)t * ldo + (size_t)h * hdv;
    const int pos = row_pos[t];
    if (pos < 0) {  // padding row
        for (int d = lane; d < hdv; d += 32) o[d] = from_f<T>(0.f);
        return;
    }
    const int kvh = h / (nh / nkv);
    const int* pt = page_table + (size_t)row_seq[t] * pt_stride;
    const T* qr = q + (size_t)t * ldq + (size_t)h * hd;
    float qv[NR], acc[NR];
#pragma unroll
    for (int i = 0; i < NR; i++) {
        const int d = lane + 32 * i;
        qv[i] = d < hd ? to_f(qr[d]) : 0.f;
        acc[i] = 0.f;
    }
    const float b1 = r1 ? r1[h] : 0.f, b2 = r1 ? r2[h] : 0.f;
    float m = -INFINITY, l = 0.f;
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    // the kept first tokens that the window has left behind, then the window (or chunk) itself
    const int kept = min(keep_first, lo);
    for (int jj = lo - kept; jj <= pos; jj++) {
        const int j = jj < lo ? jj - (lo - kept) : jj;
        const int page = pt[j / DK_PAGE];
        const T* kr = k_store + kv_offset(page, nkv, kvh, j % DK_PAGE, hd);
        const T* vr = v_store != nullptr ? v_store + kv_offset(page, nkv, kvh, j % DK_PAGE, hdv) : kr;   // no store of values: the key row's start
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < NR; i++) {
            const int d = lane + 32 * i;
            if (d < hd) dot += qv[i] * to_f(kr[d]);
        }
        float s = warp_sum(dot) * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        if (r1) s -= b1 * log1pf(b2 * (float)(pos - j));
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);  // m = -inf on the first key: alpha = 0
        const float p = expf(s - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < NR; i++) {
            const int d = lane + 32 * i;
            if (d < hdv) acc[i] = acc[i] * alpha + p * to_f(vr[d]);
        }
        m = m_new;
    }
    float alpha = 1.f;
    if (sink) {  // one more term of the denominator, without a value
        const float m_new = fmaxf(m, sink[h]);
        alpha = expf(m - m_new);
        l = l * alpha + expf(sink[h] - m_new);
    }
    const float inv = alpha / l * out_scale;
    const T* gr = gate ? gate + (size_t)t * ldg + (size_t)h * hdv : nullptr;
#pragma unroll
    for (int i = 0; i < NR; i++) {
        const int d = lane + 32 * i;
        if (d < hdv) {
            float v = acc[i] * inv;
            if (gr) v *= 1.f / (1.f + expf(-to_f(gr[d])));
            o[d] = from_f<T>(v);
        }
    }
}

DK_EXPORT int dk_kv_write(int dtype, const void* k, const void* v, long long ld, void* k_store, void* v_store,
                          const int* row_pos, const int* row_seq, const int* page_table, int pt_stride, int n_tok,
                          int nkv, int hd, int hdv, cudaStream_t st) {
    if (dtype == 0)
        return dk_launch(kv_write_kernel<float>, dim3(n_tok), dim3(128), 0, st, (const float*)k, (const float*)v, ld,
                         (float*)k_store, (float*)v_store, row_pos, row_seq, page_table, pt_stride, n_tok, nkv, hd, hdv);
    return dk_launch(kv_write_kernel<bf16>, dim3(n_tok), dim3(128), 0, st, (const bf16*)k, (const bf16*)v, ld,
                     (bf16*)k_store, (bf16*)v_store, row_pos, row_seq, page_table, pt_stride, n_tok, nkv, hd, hdv);
}

DK_EXPORT int dk_attention_masked(int dtype, const void* q, long long ldq, void* out, long long ldo, const void* gate,
                                  long long ldg, float out_scale, const void* k_store, const void* v_store,
                                  const int* row_pos, const int* row_seq, const int* page_table, int pt_stride,
                                  int n_tok, int nh, int nkv, int hd, int hdv, int window, int chunk, float scale,
                                  const float* r1, const float* r2, const float* sink, float softcap, int keep_first,
                                  cudaStream_t st) {
    if (hd > 640 || hdv > 640 || nh % nkv != 0) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)n_tok * nh;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    const bool wide = hd > 256 || hdv > 256;       // heads beyond 256 coordinates: 20 a lane instead of 8
#define AM_LAUNCH(T, NR)                                                                                              \
    return dk_launch(attention_masked_kernel<T, NR>, dim3(blocks), dim3(128), 0, st, (const T*)q, ldq, (T*)out, ldo,   \
                     (const T*)gate, ldg, out_scale, (const T*)k_store, (const T*)v_store, row_pos, row_seq, page_table, \
                     pt_stride, n_tok, nh, nkv, hd, hdv, window, chunk, scale, r1, r2, sink, softcap, keep_first)
    if (dtype == 0) {
        if (wide) AM_LAUNCH(float, 20);
        AM_LAUNCH(float, 8);
    }
    if (wide) AM_LAUNCH(bf16, 20);
    AM_LAUNCH(bf16, 8);
#undef AM_LAUNCH
}
