// Per-head RMSNorm of queries and keys, rotary position encoding, and the
// write of keys and values into the paged cache, in one pass over the
// projected rows.
//
// The reference normalises each head of q and k over head_dim with one eps
// (crates/cellm-model/src/lfm.rs:486-543), rotates pairs (i, i + rot/2) by
// pos * theta^(-2i/rot) (crates/cellm-kernels/src/cpu_kernels.rs:264-277; the
// interleaved pairing (2i, 2i+1) of :279-292 is the other layout), and writes
// k and v for the token's position (crates/cellm-model/src/lfm.rs:563-566).
// Values are not normalised. The host computes the inverse frequencies in 64-bit
// and passes each as a pair of floats (high part, remainder); the angle
// pos * inv_freq is formed as a float plus its exact rounding error, and that
// error enters cos/sin through the first terms of the addition formulas, so the
// rotation carries no error that grows with the position.
//
// Cache layout of one layer: [page][kv_head][slot in page][head_dim].
#include "common.cuh"

template <typename TA, typename TW>
__global__ void qk_norm_rope_kernel(TA* __restrict__ q_out, const TA* __restrict__ qkv, long long row_stride,
                                    const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ block_table, int bt_stride,
                                    TA* __restrict__ k_pool, TA* __restrict__ v_pool, int num_pages,
                                    int page_size, int nh, int nkv, int hd, int rot, int interleaved,
                                    const float* __restrict__ inv_freq, int* __restrict__ err) {
    extern __shared__ float smem[];
    float* cs = smem;                    // [rot/2] cos
    float* sn = smem + rot / 2;          // [rot/2] sin
    const int nwarps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = smem + rot + warp * hd; // one head per warp
    const int n_heads_all = nh + 2 * nkv;
    // blockIdx.y selects a run of heads, so that a token's heads are spread over several blocks
    const int heads_per_block = (n_heads_all + gridDim.y - 1) / gridDim.y;
    const int h_begin = blockIdx.y * heads_per_block, h_end = min(n_heads_all, h_begin + heads_per_block);
    pdl_trigger();
    // Positions, block table and frequencies are the step's inputs, not the work of the kernel before this one:
    // the cosines, sines and the page look-up are done before the wait on it; only the rows of qkv come after.
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int p = threadIdx.x; p < rot / 2; p += blockDim.x) {
        const float hi = inv_freq[2 * p], lo = inv_freq[2 * p + 1], fp = (float)pos;
        const float a = fp * hi;                              // angle, rounded
        const float e = fmaf(fp, hi, -a) + fp * lo;           // what the rounding dropped, plus the remainder's share
        float s, c, se, ce;
        sincosf(a, &s, &c);
        sincosf(e, &se, &ce);                                 // e is small (at most a few hundredths far out)
        cs[p] = c * ce - s * se;                              // cos(a + e)
        sn[p] = s * ce + c * se;                              // sin(a + e)
    }
    long long page_base = -1;
    if (nkv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(size_t)b * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_PAGE);
        } else {
            page_base = (long long)page * nkv * page_size * hd + (long long)(pos % page_size) * hd;
        }
    }
    __syncthreads();
    pdl_wait();
    const TA* row = qkv + (size_t)t * row_stride;
    for (int hh = h_begin + warp; hh < h_end; hh += nwarps) {
        const TA* src = row + (size_t)hh * hd;
        if (hh >= nh + nkv) {  // value head: copy
            if (page_base >= 0) {
                TA* dst = v_pool + page_base + (long long)(hh - nh - nkv) * page_size * hd;
                for (int i = lane; i < hd; i += 32) dst[i] = src[i];
            }
            continue;
        }
        const bool is_q = hh < nh;
        const TW* w = is_q ? q_w : k_w;
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) {
            const float v = to_float(src[i]);
            buf[i] = v;
            ss += v * v;
        }
        if (w) {
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
            for (int i = lane; i < hd; i += 32) buf[i] = buf[i] * inv * to_float(w[i]);
        }
        __syncwarp();
        TA* dst;
        if (is_q) dst = q_out + (size_t)t * nh * hd + (size_t)hh * hd;
        else if (page_base >= 0) dst = k_pool + page_base + (long long)(hh - nh) * page_size * hd;
        else { __syncwarp(); continue; }
        for (int p = lane; p < rot / 2; p += 32) {
            const int i0 = interleaved ? 2 * p : p;
            const int i1 = interleaved ? 2 * p + 1 : p + rot / 2;
            const float a = buf[i0], b = buf[i1];
            dst[i0] = from_float<TA>(a * cs[p] - b * sn[p]);
            dst[i1] = from_float<TA>(b * cs[p] + a * sn[p]);
        }
        for (int i = rot + lane; i < hd; i += 32) dst[i] = from_float<TA>(buf[i]);
        __syncwarp();
    }
}

// Fast form for long batches of bfloat16 rows with 64-wide heads turned whole in the
// "half" layout. One warp takes one token and a run of its heads (query, key and
// value heads alike), four heads at a time: a lane holds eight neighbouring values
// of a head (one 16-byte load and store), eight lanes a head. The token's 32
// cosines and sines are computed once per warp (lane l: frequency l) and passed
// through shared memory; a head's sum of squares takes three shuffles, and the
// rotation partners (+-32 values) sit four lanes away.
template <typename TW>
__global__ void __launch_bounds__(128)
qk_norm_rope_hd64_kernel(__nv_bfloat16* __restrict__ q_out, const __nv_bfloat16* __restrict__ qkv, long long row_stride,
                         const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                         const int* __restrict__ block_table, int bt_stride, __nv_bfloat16* __restrict__ k_pool,
                         __nv_bfloat16* __restrict__ v_pool, int num_pages, int page_size, int T, int nh, int nkv,
                         const float* __restrict__ inv_freq, int* __restrict__ err) {
    __shared__ float trig[4][64];            // per warp: 32 cosines, 32 sines
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    // The token's values are asked for first (the launcher gives a block at most sixteen heads: four rounds of four), so
    // that they travel while the cosines, the weights and the page are looked up.
    const int chunk = lane & 7;              // values 8 * chunk .. 8 * chunk + 7 of the head
    const __nv_bfloat16* row = qkv + (size_t)t * row_stride;
    // blockIdx.y takes a run of the token's heads: queries, then keys, then values
    const int all = nh + 2 * nkv;
    const int per = ((all + gridDim.y - 1) / gridDim.y + 3) / 4 * 4;
    const int h_begin = blockIdx.y * per, h_end = min(all, h_begin + per);
    uint4 ahead[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int hh = h_begin + 4 * r + (lane >> 3);
        ahead[r] = make_uint4(0, 0, 0, 0);
        if (hh < h_end) ahead[r] = *reinterpret_cast<const uint4*>(row + (size_t)hh * 64 + chunk * 8);
    }
    const int pos = positions[t];
    {
        const float hi = inv_freq[2 * lane], lo = inv_freq[2 * lane + 1], fp = (float)pos;
        const float a = fp * hi;
        const float e = fmaf(fp, hi, -a) + fp * lo;
        float s, c, se, ce;
        sincosf(a, &s, &c);
        sincosf(e, &se, &ce);
        trig[warp][lane] = c * ce - s * se;
        trig[warp][32 + lane] = s * ce + c * se;
    }
    __syncwarp();
    const int f0 = (chunk & 3) * 8;          // their frequencies (value i turns with frequency i mod 32)
    float cs[8], sn[8], wq[8], wk[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        cs[j] = trig[warp][f0 + j];
        sn[j] = trig[warp][32 + f0 + j];
        wq[j] = q_w ? to_float(q_w[chunk * 8 + j]) : 1.f;
        wk[j] = k_w ? to_float(k_w[chunk * 8 + j]) : 1.f;
    }
    const float sign = chunk < 4 ? -1.f : 1.f;     // first half: x0 cos - x1 sin; second half: x1 cos + x0 sin
    long long page_base = -1;
    if (nkv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(size_t)b * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) { if (lane == 0) atomicOr(err, CELLM_DEV_BAD_PAGE); }
        else page_base = (long long)page * nkv * page_size * 64 + (long long)(pos % page_size) * 64;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int h0 = h_begin + 4 * r;
        if (h0 >= h_end) break;
        const int hh = h0 + (lane >> 3);
        const bool on = hh < h_end;
        const uint4 raw = ahead[r];
        const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
        float v[8];
        {
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(p2[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
        }
        if (q_w) {                          // (all lanes shuffle; value heads drop the result)
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            ss += __shfl_xor_sync(0xffffffffu, ss, 4);
            const float inv = 1.0f / sqrtf(ss / 64.f + eps);
            if (is_q || is_k) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = v[j] * inv * (is_q ? wq[j] : wk[j]);
            }
        }
        uint4 outw;
        {
            uint32_t* ow = reinterpret_cast<uint32_t*>(&outw);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const float p0 = __shfl_xor_sync(0xffffffffu, v[j], 4), p1 = __shfl_xor_sync(0xffffffffu, v[j + 1], 4);
                const __nv_bfloat162 o = (is_q || is_k)
                    ? __floats2bfloat162_rn(v[j] * cs[j] + sign * p0 * sn[j], v[j + 1] * cs[j + 1] + sign * p1 * sn[j + 1])
                    : __floats2bfloat162_rn(v[j], v[j + 1]);
                ow[j >> 1] = *reinterpret_cast<const uint32_t*>(&o);
            }
        }
        if (!on) continue;
        if (is_q) *reinterpret_cast<uint4*>(q_out + (size_t)t * nh * 64 + (size_t)hh * 64 + chunk * 8) = outw;
        else if (page_base >= 0) {
            __nv_bfloat16* pool = is_k ? k_pool : v_pool;
            const int kvh = is_k ? hh - nh : hh - nh - nkv;
            *reinterpret_cast<uint4*>(pool + page_base + (long long)kvh * page_size * 64 + chunk * 8) = is_k ? outw : raw;
        }
    }
}

// qkv: [T, row_stride] rows holding nh query heads, then nkv key heads, then nkv
// value heads (nkv = 0: queries only, nothing is written to the cache).
// q_w, k_w: [hd] norm weights or null (no norm). inv_freq: [rot/2] pairs of floats
// (high part, remainder) of the 64-bit inverse frequencies.
CELLM_API int cellm_qk_norm_rope(void* q_out, const void* qkv, long long row_stride, const void* q_w,
                                 const void* k_w, int w_dtype, float eps, const int* positions,
                                 const int* seq_of_token, const int* block_table, int bt_stride,
                                 void* k_pool, void* v_pool, int num_pages, int page_size, int T, int nh,
                                 int nkv, int hd, int rot, int interleaved, const float* inv_freq,
                                 int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (rot < 0 || rot > hd || (rot & 1)) return CELLM_ERR_SIZE;
    if ((q_w == nullptr) != (k_w == nullptr)) return CELLM_ERR_ARG;
    if (act_dtype == CELLM_BF16 && hd == 64 && rot == 64 && !interleaved && T >= 256 && (row_stride & 7) == 0 &&
        (((uintptr_t)q_out | (uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0) {
        // heads in runs of sixteen: enough warps to keep loads in flight, few repeats of a token's cosines and sines
        const dim3 blocks((unsigned)((T + 3) / 4), (unsigned)((nh + 2 * nkv + 15) / 16));
        if (w_dtype == CELLM_BF16 || q_w == nullptr)
            CELLM_RUN(qk_norm_rope_hd64_kernel<__nv_bfloat16>, blocks, 128, 0, stream, (__nv_bfloat16*)q_out,
                      (const __nv_bfloat16*)qkv, row_stride, (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, eps,
                      positions, seq_of_token, block_table, bt_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                      num_pages, page_size, T, nh, nkv, inv_freq, err);
        else if (w_dtype == CELLM_F32)
            CELLM_RUN(qk_norm_rope_hd64_kernel<float>, blocks, 128, 0, stream, (__nv_bfloat16*)q_out,
                      (const __nv_bfloat16*)qkv, row_stride, (const float*)q_w, (const float*)k_w, eps, positions,
                      seq_of_token, block_table, bt_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, num_pages,
                      page_size, T, nh, nkv, inv_freq, err);
        else return CELLM_ERR_DTYPE;
        return CELLM_OK;
    }
    const int threads = 128;
    // few tokens: spread each token's heads over blocks of four (one per warp); many tokens: one block each
    const int heads_all = nh + 2 * nkv;
    const unsigned gy = T >= 1024 ? 1u : (unsigned)((heads_all + 3) / 4);
    dim3 grid((unsigned)T, gy > 65535u ? 65535u : gy);
    const size_t smem = (size_t)(rot + (threads / 32) * hd) * sizeof(float);
    if (smem > 48 * 1024) return CELLM_ERR_SIZE;
#define LAUNCH(TA, TW)                                                                               \
    CELLM_RUN((qk_norm_rope_kernel<TA, TW>), grid, threads, smem, stream,                            \
        (TA*)q_out, (const TA*)qkv, row_stride, (const TW*)q_w, (const TW*)k_w, eps, positions,      \
        seq_of_token, block_table, bt_stride, (TA*)k_pool, (TA*)v_pool, num_pages, page_size, nh,    \
        nkv, hd, rot, interleaved, inv_freq, err)
    if (act_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float);
    else if (act_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}
