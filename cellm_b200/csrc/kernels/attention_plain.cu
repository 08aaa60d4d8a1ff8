// Plain attention over the paged cache: one block per (token, head), every
// earlier key of the request (or the last `window` of them) read through the
// block table. It serves the 32-bit path and is the reference for the faster
// attention kernels.
//
// For head h the key/value head is h / (nh / nkv); scores are q.k * scale;
// softmax takes the maximum off first; all of it in 32-bit
// (crates/cellm-cache/src/kvcache.rs:753-787, :1206-1227). Keys are walked in
// chunks that start at multiples of the chunk size counted from key 0, so the
// order of every sum depends only on the token's position, never on how the
// sequence was cut into steps or what else is in the batch.
//
// Cache layout of one layer: [page][kv_head][slot in page][head_dim].
#include "common.cuh"

#define ATTN_PLAIN_THREADS 128
#define ATTN_PLAIN_MAX_HD 512

template <typename TA>
__global__ void __launch_bounds__(ATTN_PLAIN_THREADS)
attention_plain_kernel(TA* __restrict__ out, const TA* __restrict__ q, const TA* __restrict__ k_pool,
                       const TA* __restrict__ v_pool, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                       int bt_stride, int num_pages, int page_size, int nh, int nkv, int hd, float scale,
                       int window, int* __restrict__ err) {
    constexpr int CH = ATTN_PLAIN_THREADS;
    extern __shared__ float smem[];
    float* qs = smem;             // [hd]
    float* sc = smem + hd;        // [CH]
    int* pg = (int*)(sc + CH);    // [CH] page of each key in the chunk
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x / nh, h = blockIdx.x % nh;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int b = seq_of_token[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < hd; i += CH) qs[i] = to_float(q[(size_t)t * nh * hd + (size_t)h * hd + i]) * scale;
    float m = -INFINITY, l = 0.f;
    float acc[ATTN_PLAIN_MAX_HD / CH];
#pragma unroll
    for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) acc[r] = 0.f;
    const size_t page_elems = (size_t)nkv * page_size * hd;
    for (int c0 = (lo / CH) * CH; c0 <= pos; c0 += CH) {
        __syncthreads();
        {   // page of key c0 + tid
            const int j = c0 + threadIdx.x;
            int p = -1;
            if (j >= lo && j <= pos) {
                p = block_table[(size_t)b * bt_stride + j / page_size];
                if (p < 0 || p >= num_pages) { atomicOr(err, CELLM_DEV_BAD_PAGE); p = -1; }
            }
            pg[threadIdx.x] = p;
        }
        __syncthreads();
        for (int jj = warp; jj < CH; jj += CH / 32) {
            const int p = pg[jj];
            float s = -INFINITY;
            if (p >= 0) {
                const int j = c0 + jj;
                const TA* kr = k_pool + (size_t)p * page_elems + ((size_t)kvh * page_size + j % page_size) * hd;
                float d = 0.f;
                for (int i = lane; i < hd; i += 32) d += qs[i] * to_float(kr[i]);
                s = warp_sum(d);
            }
            if (lane == 0) sc[jj] = s;
        }
        __syncthreads();
        const float cmax = block_max(sc[threadIdx.x], scratch);
        const float m_new = fmaxf(m, cmax);
        const float s = sc[threadIdx.x];
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float psum = block_sum(p, scratch);
        __syncthreads();
        sc[threadIdx.x] = p;
        __syncthreads();
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + psum;
        m = m_new;
#pragma unroll
        for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) {
            const int d = threadIdx.x + r * CH;
            if (d < hd) {
                float a = acc[r] * corr;
                for (int jj = 0; jj < CH; ++jj) {
                    const int pgj = pg[jj];
                    if (pgj < 0) continue;
                    const int j = c0 + jj;
                    a += sc[jj] * to_float(v_pool[(size_t)pgj * page_elems + ((size_t)kvh * page_size + j % page_size) * hd + d]);
                }
                acc[r] = a;
            }
        }
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) {
        const int d = threadIdx.x + r * CH;
        if (d < hd) out[(size_t)t * nh * hd + (size_t)h * hd + d] = from_float<TA>(acc[r] * inv);
    }
}

// out, q: [T, nh*hd]; pools: one layer's keys and values; positions[t] is the
// token's place in its request (keys 0..positions[t] are read; the token's own
// key must already be in the cache).
CELLM_API int cellm_attention_plain(void* out, const void* q, const void* k_pool, const void* v_pool,
                                    const int* positions, const int* seq_of_token, const int* block_table,
                                    int bt_stride, int num_pages, int page_size, int T, int nh, int nkv,
                                    int hd, float scale, int window, int dtype, int* err,
                                    cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (hd > ATTN_PLAIN_MAX_HD || hd <= 0 || nkv <= 0 || nh % nkv) return CELLM_ERR_SIZE;
    const size_t smem = (size_t)(hd + 2 * ATTN_PLAIN_THREADS) * sizeof(float);
    const unsigned grid = (unsigned)T * (unsigned)nh;
    if (dtype == CELLM_F32)
        CELLM_RUN(attention_plain_kernel<float>, grid, ATTN_PLAIN_THREADS, smem, stream,
            (float*)out, (const float*)q, (const float*)k_pool, (const float*)v_pool, positions, seq_of_token,
            block_table, bt_stride, num_pages, page_size, nh, nkv, hd, scale, window, err);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(attention_plain_kernel<__nv_bfloat16>, grid, ATTN_PLAIN_THREADS, smem, stream,
            (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, positions, seq_of_token, block_table, bt_stride, num_pages,
            page_size, nh, nkv, hd, scale, window, err);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
