// Row kernels of attention through low-rank latents. With x a token's input to the mixer, the fused down
// projection leaves a row [a | b | r]: a (q_rank numbers) becomes the query latent, b (kv_rank) the key/value
// latent, r (rot_dim) the one rotated key part that all heads share.
//   latent_norm_rope_write : c_q = rmsnorm(a) * w_q -> dense rows; c = rmsnorm(b) * w_kv and r rotated by pairs
//                            -> the token's place in the paged cache: key row [c | r] (one kv head), whose first kv_rank
//                            numbers are the value row (a cache with a store of values gets c there as well).
//   latent_query           : per (token, head) the query of the up projection [plain (dim) | rot (rot_dim)] becomes
//                            [W_uk_h^T plain (kv_rank) | rot rotated by pairs]: the plain key's up projection moved to
//                            the query's side, so that scores are taken against the cached latent itself.
//   latent_value           : per (token, head) the attention's output over latents (kv_rank) becomes W_uv_h times it (vdim).
// Norms, angles, rotations and sums are float32 whatever the storage type. Rotation by pairs: coordinates
// (2i, 2i+1) of the first rot_dims of the rotated part turn by the angle table's entry [position, i].
#include "common.cuh"

#define LT_THREADS 128

template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
latent_norm_rope_write_kernel(const T* proj, long long ld, T* cq_out, long long ldq, const float* __restrict__ wq,
                              const float* __restrict__ wkv, float eps, const float* __restrict__ cosv,
                              const float* __restrict__ sinv, int rot_dims, const int* row_pos, const int* row_seq,
                              int q_rank, int kv_rank, int rot_dim, T* k_store, T* v_store, const int* page_table,
                              int pt_stride) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = row_pos[t];
    if (pos < 0) return;
    const T* row = proj + (size_t)t * ld;
    if (blockIdx.y == 0) {                    // the query latent
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += LT_THREADS) {
            const float v = to_f(row[i]);
            ss += v * v;
        }
        ss = block_sum(ss, red);
        const float rs = 1.f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += LT_THREADS)
            cq_out[(size_t)t * ldq + i] = from_f<T>(to_f(row[i]) * rs * wq[i]);
        return;
    }
    if (k_store == nullptr) return;
    const int page = page_table[(size_t)row_seq[t] * pt_stride + pos / DK_PAGE];
    if (page < 0) return;
    const T* b = row + q_rank;
    float ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += LT_THREADS) {
        const float v = to_f(b[i]);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = 1.f / sqrtf(ss / (float)kv_rank + eps);
    T* kr = k_store + kv_offset(page, 1, 0, pos % DK_PAGE, kv_rank + rot_dim);
    T* vr = v_store != nullptr ? v_store + kv_offset(page, 1, 0, pos % DK_PAGE, kv_rank) : nullptr;   // a store of values, if the cache keeps one
    for (int i = threadIdx.x; i < kv_rank; i += LT_THREADS) {
        const T c = from_f<T>(to_f(b[i]) * rs * wkv[i]);
        kr[i] = c;
        if (vr != nullptr) vr[i] = c;
    }
    const T* r = b + kv_rank;
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < rot_dim; i += LT_THREADS) {
        float y = to_f(r[i]);
        if (i < rot_dims) {
            const float c = cosv[(size_t)pos * half + i / 2], sn = sinv[(size_t)pos * half + i / 2];
            y = (i & 1) ? y * c + to_f(r[i - 1]) * sn : y * c - to_f(r[i + 1]) * sn;
        }
        kr[kv_rank + i] = from_f<T>(y);
    }
}

// One block per (token, head); threads over the kv_rank outputs read W_uk's rows of the head side by side.
template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
latent_query_kernel(const T* q, long long ldq, const T* __restrict__ w_uk, T* out, long long ldo,
                    const float* __restrict__ cosv, const float* __restrict__ sinv, int rot_dims, const int* row_pos,
                    int dim, int rot_dim, int kv_rank) {
    extern __shared__ float qs[];             // dim + rot_dim
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y;
    const int pos = row_pos[t];
    T* o = out + (size_t)t * ldo + (size_t)h * (kv_rank + rot_dim);
    if (pos < 0) {
        for (int i = threadIdx.x; i < kv_rank + rot_dim; i += LT_THREADS) o[i] = from_f<T>(0.f);
        return;
    }
    const T* qr = q + (size_t)t * ldq + (size_t)h * (dim + rot_dim);
    for (int i = threadIdx.x; i < dim + rot_dim; i += LT_THREADS) qs[i] = to_f(qr[i]);
    __syncthreads();
    const T* w = w_uk + (size_t)h * dim * kv_rank;
    for (int r = threadIdx.x; r < kv_rank; r += LT_THREADS) {
        float acc = 0.f;
        for (int d = 0; d < dim; d++) acc = fmaf(qs[d], to_f(w[(size_t)d * kv_rank + r]), acc);
        o[r] = from_f<T>(acc);
    }
    const int half = rot_dims / 2;
    const float* rq = qs + dim;
    for (int i = threadIdx.x; i < rot_dim; i += LT_THREADS) {
        float y = rq[i];
        if (i < rot_dims) {
            const float c = cosv[(size_t)pos * half + i / 2], sn = sinv[(size_t)pos * half + i / 2];
            y = (i & 1) ? y * c + rq[i - 1] * sn : y * c - rq[i + 1] * sn;
        }
        o[kv_rank + i] = from_f<T>(y);
    }
}

// The rotation alone, in place, on the rotated part of every head of q [tokens, heads * (dim + rot_dim)]: for
// steps whose plain parts go through a library product instead of latent_query.
template <typename T>
__global__ void latent_rotate_kernel(const T* q, long long ldq, T* out, long long ldo, const float* __restrict__ cosv,
                                     const float* __restrict__ sinv, int rot_dims, const int* row_pos, int n_tok, int n_heads,
                                     int dim, int rot_dim, int kv_rank) {
    pdl_wait();
    pdl_launch_dependents();
    // a thread per (token, head, two neighbouring coordinates of the rotated part; a last single one if rot_dim is odd)
    const int per_head = (rot_dim + 1) / 2;
    const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (long long)n_tok * n_heads * per_head) return;
    const int i = 2 * (int)(item % per_head), h = (int)(item / per_head % n_heads), t = (int)(item / per_head / n_heads);
    const int pos = row_pos[t];
    const T* rq = q + (size_t)t * ldq + (size_t)h * (dim + rot_dim) + dim;
    T* o = out + (size_t)t * ldo + (size_t)h * (kv_rank + rot_dim) + kv_rank;
    const bool two = i + 1 < rot_dim;
    float u = pos < 0 ? 0.f : to_f(rq[i]), v = (pos < 0 || !two) ? 0.f : to_f(rq[i + 1]);
    if (pos >= 0 && i + 1 < rot_dims) {
        const int half = rot_dims / 2;
        const float c = cosv[(size_t)pos * half + i / 2], sn = sinv[(size_t)pos * half + i / 2];
        const float u2 = u * c - v * sn;
        v = v * c + u * sn;
        u = u2;
    }
    o[i] = from_f<T>(u);
    if (two) o[i + 1] = from_f<T>(v);
}

// One block per (token, head); a warp per output: W_uv's row of kv_rank numbers times the latent output.
template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
latent_value_kernel(const T* o_lat, long long ldi, const T* __restrict__ w_uv, T* out, long long ldo, int kv_rank,
                    int vdim) {
    extern __shared__ float os[];             // kv_rank
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y;
    const T* src = o_lat + (size_t)t * ldi + (size_t)h * kv_rank;
    for (int i = threadIdx.x; i < kv_rank; i += LT_THREADS) os[i] = to_f(src[i]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = warp; j < vdim; j += LT_THREADS / 32) {
        const T* w = w_uv + ((size_t)h * vdim + j) * kv_rank;
        float acc = 0.f;
        for (int r = lane; r < kv_rank; r += 32) acc = fmaf(os[r], to_f(w[r]), acc);
        acc = warp_sum(acc);
        if (lane == 0) out[(size_t)t * ldo + (size_t)h * vdim + j] = from_f<T>(acc);
    }
}

#define LT_DISPATCH(dtype, ...)                         \
    if ((dtype) == 0) { typedef float T; __VA_ARGS__; } \
    else { typedef bf16 T; __VA_ARGS__; }

DK_EXPORT int dk_latent_norm_rope_write(int dtype, const void* proj, long long ld, void* cq_out, long long ldq,
                                        const float* wq, const float* wkv, float eps, const float* cosv,
                                        const float* sinv, int rot_dims, const int* row_pos, const int* row_seq, int n_tok,
                                        int q_rank, int kv_rank, int rot_dim, void* k_store, void* v_store,
                                        const int* page_table, int pt_stride, cudaStream_t st) {
    if (rot_dims % 2 || rot_dims > rot_dim) return (int)cudaErrorInvalidValue;
    LT_DISPATCH(dtype, return dk_launch(latent_norm_rope_write_kernel<T>, dim3(n_tok, 2), dim3(LT_THREADS), 0, st,
                                        (const T*)proj, ld, (T*)cq_out, ldq, wq, wkv, eps, cosv, sinv, rot_dims, row_pos,
                                        row_seq, q_rank, kv_rank, rot_dim, (T*)k_store, (T*)v_store, page_table, pt_stride));
}

DK_EXPORT int dk_latent_query(int dtype, const void* q, long long ldq, const void* w_uk, void* out, long long ldo,
                              const float* cosv, const float* sinv, int rot_dims, const int* row_pos, int n_tok,
                              int n_heads, int dim, int rot_dim, int kv_rank, int plain, cudaStream_t st) {
    if (rot_dims % 2 || rot_dims > rot_dim) return (int)cudaErrorInvalidValue;
    if (!plain) {
        const long long items = (long long)n_tok * n_heads * ((rot_dim + 1) / 2);
        LT_DISPATCH(dtype, return dk_launch(latent_rotate_kernel<T>, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, st,
                                            (const T*)q, ldq, (T*)out, ldo, cosv, sinv, rot_dims, row_pos, n_tok, n_heads, dim,
                                            rot_dim, kv_rank));
    }
    const size_t smem = (size_t)(dim + rot_dim) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    LT_DISPATCH(dtype, return dk_launch(latent_query_kernel<T>, dim3(n_tok, n_heads), dim3(LT_THREADS), smem, st,
                                        (const T*)q, ldq, (const T*)w_uk, (T*)out, ldo, cosv, sinv, rot_dims, row_pos, dim,
                                        rot_dim, kv_rank));
}

DK_EXPORT int dk_latent_value(int dtype, const void* o_lat, long long ldi, const void* w_uv, void* out, long long ldo,
                              int n_tok, int n_heads, int kv_rank, int vdim, cudaStream_t st) {
    const size_t smem = (size_t)kv_rank * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    LT_DISPATCH(dtype, return dk_launch(latent_value_kernel<T>, dim3(n_tok, n_heads), dim3(LT_THREADS), smem, st,
                                        (const T*)o_lat, ldi, (const T*)w_uv, (T*)out, ldo, kv_rank, vdim));
}
