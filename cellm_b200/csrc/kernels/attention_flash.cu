// Flash-style attention over the paged cache for bfloat16, on the tensor cores
// (mma.sync m16n8k16), for prompt portions and decoded tokens alike.
//
// All query heads that share a key/value head are packed into one tile: for
// key/value head g of request b the tile's rows are (token, head in group)
// pairs, row r = token * G + head (G = heads per key/value head). A CTA takes
// 16 rows per warp; keys are walked in blocks of 64 through the request's
// block table, with K and V blocks brought in by cp.async, double-buffered.
// Scores q.k * scale, causal mask (key <= the token's position), optional
// window, online softmax in 32-bit with the running maximum taken off
// (crates/cellm-cache/src/kvcache.rs:753-787, :1206-1227 is the reference's
// single-token loop). Probabilities are rounded to bfloat16 for the P.V
// product; sums and outputs stay 32-bit until the final store.
//
// A token with a long context can be split over gridDim.z CTAs, each taking a
// run of key blocks; the pieces (unnormalised output, maximum, sum) go to a
// workspace and a second kernel merges them in the order of the pieces.
//
// Cache layout of one layer: [page][kv_head][slot in page][head_dim].
#include <mma.h>

#include <mutex>

#include "common.cuh"
#include "attention_flash_noalloc.h"
#include "mma_tiles.cuh"

namespace {

template <int HD, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32, (HD <= 64 && NWARPS == 4) ? 4 : 1)
attention_flash_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                       const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                       const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ ctx_lens, const int* __restrict__ block_table, int bt_stride,
                       int B, int T, int num_pages, int page_size, int nh, int nkv, float scale_log2e, int window,
                       int* __restrict__ err) {
    constexpr int BM = 16 * NWARPS, BN = FA_BN, CH = HD / 8, NT = HD / 8, THREADS = NWARPS * 32;
    extern __shared__ __align__(128) uint8_t fa_smem[];
    uint8_t* q_s = fa_smem;                              // [BM][HD]
    uint8_t* k_s = q_s + BM * HD * 2;                    // [2][BN][HD]
    uint8_t* v_s = k_s + 2 * BN * HD * 2;                // [2][BN][HD]
    const int G = nh / nkv;
    const int kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();

    // which request this tile belongs to; tiles are taken from the last to the first, so
    // that the tiles with the most keys (the latest rows of a prompt) start first
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;
    int b = 0, base = 0;
    for (; b < B; ++b) {
        const int nt = ((cu_seqlens[b + 1] - cu_seqlens[b]) * G + BM - 1) / BM;
        if (tile < base + nt) break;
        base += nt;
    }
    if (b == B) return;
    const int t_base = cu_seqlens[b], q_len = cu_seqlens[b + 1] - t_base, rows = q_len * G;
    const int ctx = ctx_lens[b];
    const int r0 = (tile - base) * BM;
    const int t_lo = r0 / G, t_hi = min(r0 + BM - 1, rows - 1) / G;
    const int key_end = ctx + t_hi + 1;
    const int key_begin = window > 0 ? max(0, ctx + t_lo - window + 1) : 0;
    const int kb_begin = key_begin / BN, kb_end = (key_end + BN - 1) / BN;
    const int per = (kb_end - kb_begin + nsplit - 1) / nsplit;
    const int my_begin = kb_begin + split * per, my_end = min(kb_end, my_begin + per);
    const int* bt = block_table + (size_t)b * bt_stride;
    const size_t page_elems = (size_t)nkv * page_size * HD;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;   // -1: not a power of two
    auto page_of = [&](int j) { return page_shift >= 0 ? (j >> page_shift) : (j / page_size); };
    auto slot_of = [&](int j) { return page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size); };

    // Q tile
    for (int i = threadIdx.x; i < BM * CH; i += THREADS) {
        const int row = i / CH, chunk = i % CH, r = r0 + row;
        const bool ok = r < rows;
        const __nv_bfloat16* src = q + (size_t)(t_base + (ok ? r / G : 0)) * nh * HD + (size_t)(kvh * G + (ok ? r % G : 0)) * HD + chunk * 8;
        cp_async16(q_s + tile_offset<HD>(row, chunk), src, ok ? 16 : 0);
    }
    // The pages of a block's keys are looked up first, all at once, so that the
    // copies that follow do not each wait for a load of the block table.
    constexpr int KV_ITERS = (BN * CH + THREADS - 1) / THREADS;
    auto load_kv = [&](int kb, int stage) {
        uint8_t* ks = k_s + stage * BN * HD * 2;
        uint8_t* vs = v_s + stage * BN * HD * 2;
        int pages[KV_ITERS];
#pragma unroll
        for (int it = 0; it < KV_ITERS; ++it) {
            const int i = threadIdx.x + it * THREADS, j = kb * BN + i / CH;
            pages[it] = (i < BN * CH && j >= key_begin && j < key_end) ? bt[page_of(j)] : -1;
        }
#pragma unroll
        for (int it = 0; it < KV_ITERS; ++it) {
            const int i = threadIdx.x + it * THREADS;
            if (i >= BN * CH) break;
            const int row = i / CH, chunk = i % CH, j = kb * BN + row;
            int page = pages[it];
            if (j >= key_begin && j < key_end && (page < 0 || page >= num_pages)) { atomicOr(err, CELLM_DEV_BAD_PAGE); page = -1; }
            const size_t off = page >= 0 ? (size_t)page * page_elems + ((size_t)kvh * page_size + slot_of(j)) * HD + chunk * 8 : 0;
            cp_async16(ks + tile_offset<HD>(row, chunk), k_pool + off, page >= 0 ? 16 : 0);
            cp_async16(vs + tile_offset<HD>(row, chunk), v_pool + off, page >= 0 ? 16 : 0);
        }
    };
    if (my_begin < my_end) load_kv(my_begin, 0);
    cp_async_commit();

    // per-thread rows: g = lane / 4 and g + 8 of this warp's 16
    const int row_a = r0 + warp * 16 + (lane >> 2), row_b = row_a + 8;
    const int pos_a = row_a < rows ? ctx + row_a / G : -1, pos_b = row_b < rows ? ctx + row_b / G : -1;
    const int lo_a = window > 0 ? pos_a - window + 1 : 0, lo_b = window > 0 ? pos_b - window + 1 : 0;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    uint32_t qf[HD / 16][4];
    bool q_loaded = false;

    for (int kb = my_begin, it = 0; kb < my_end; ++kb, ++it) {
        const int stage = it & 1;
        if (kb + 1 < my_end) load_kv(kb + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (!q_loaded) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                ldmatrix_x4(qf[ks], q_s + tile_offset<HD>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
            q_loaded = true;
        }
        const uint8_t* ks_ = k_s + stage * BN * HD * 2;
        const uint8_t* vs_ = v_s + stage * BN * HD * 2;
        // S = Q K^T for 64 keys
        float s[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < BN / 16; ++n2) {
                uint32_t kf[4];
                ldmatrix_x4(kf, ks_ + tile_offset<HD>(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * n2], qf[ks], kf[0], kf[1]);
                mma_bf16(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
            }
        }
        // mask, online softmax. A block whose keys every row of this warp may read
        // (all below the diagonal, all inside the window) needs no mask.
        const int j0 = kb * BN + (lane & 3) * 2;
        float mx_a = -INFINITY, mx_b = -INFINITY;
        const int w_row0 = r0 + warp * 16, w_row1 = min(w_row0 + 15, rows - 1);
        const bool open_block = w_row0 + 15 < rows && kb * BN + BN - 1 <= ctx + w_row0 / G &&
                                (window <= 0 || kb * BN >= ctx + w_row1 / G - window + 1);
        if (open_block) {
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
                mx_a = fmaxf(mx_a, fmaxf(s[n][0], s[n][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[n][2], s[n][3]));
            }
        } else {
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = j0 + n * 8 + e;
                    const float va = (j <= pos_a && j >= lo_a) ? s[n][e] : -INFINITY;
                    const float vb = (j <= pos_b && j >= lo_b) ? s[n][2 + e] : -INFINITY;
                    s[n][e] = va;
                    s[n][2 + e] = vb;
                    mx_a = fmaxf(mx_a, va);
                    mx_b = fmaxf(mx_b, vb);
                }
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        // scores stay raw; the scale (positive) enters with the subtraction of the maximum: 2^(s*c - m)
        const float mn_a = fmaxf(m_a, mx_a * scale_log2e), mn_b = fmaxf(m_b, mx_b * scale_log2e);
        const float use_a = mn_a == -INFINITY ? 0.f : mn_a, use_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float corr_a = fast_exp2(m_a - use_a), corr_b = fast_exp2(m_b - use_b);
        m_a = mn_a;
        m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pf[BN / 16][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            const float p0 = fast_exp2(fmaf(s[n][0], scale_log2e, -use_a)), p1 = fast_exp2(fmaf(s[n][1], scale_log2e, -use_a));
            const float p2 = fast_exp2(fmaf(s[n][2], scale_log2e, -use_b)), p3 = fast_exp2(fmaf(s[n][3], scale_log2e, -use_b));
            sum_a += p0 + p1;
            sum_b += p2 + p3;
            pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_a = l_a * corr_a + sum_a;
        l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int n = 0; n < NT; ++n) { o[n][0] *= corr_a; o[n][1] *= corr_a; o[n][2] *= corr_b; o[n][3] *= corr_b; }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vs_ + tile_offset<HD>(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), n2 * 2 + (lane >> 4)));
                mma_bf16(o[2 * n2], pf[kk], vf[0], vf[1]);
                mma_bf16(o[2 * n2 + 1], pf[kk], vf[2], vf[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const int col = (lane & 3) * 2;
    if (nsplit == 1) {
        const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
        if (row_a < rows) {
            __nv_bfloat16* dst = out + (size_t)(t_base + row_a / G) * nh * HD + (size_t)(kvh * G + row_a % G) * HD + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][0] * inv_a, o[n][1] * inv_a);
        }
        if (row_b < rows) {
            __nv_bfloat16* dst = out + (size_t)(t_base + row_b / G) * nh * HD + (size_t)(kvh * G + row_b % G) * HD + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][2] * inv_b, o[n][3] * inv_b);
        }
    } else {
        const size_t n_rows = (size_t)T * nh;
        if (row_a < rows) {
            const size_t gr = (size_t)(t_base + row_a / G) * nh + kvh * G + row_a % G;
            float* dst = part_o + ((size_t)split * n_rows + gr) * HD + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][0], o[n][1]);
            if ((lane & 3) == 0) { part_ml[((size_t)split * n_rows + gr) * 2] = m_a; part_ml[((size_t)split * n_rows + gr) * 2 + 1] = l_a; }
        }
        if (row_b < rows) {
            const size_t gr = (size_t)(t_base + row_b / G) * nh + kvh * G + row_b % G;
            float* dst = part_o + ((size_t)split * n_rows + gr) * HD + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2], o[n][3]);
            if ((lane & 3) == 0) { part_ml[((size_t)split * n_rows + gr) * 2] = m_b; part_ml[((size_t)split * n_rows + gr) * 2 + 1] = l_b; }
        }
    }
}

// out[row] = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s, pieces in order.
__global__ void attention_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                       const float* __restrict__ part_ml, size_t n_rows, int hd, int nsplit) {
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[((size_t)s * n_rows + row) * 2]);
    const float use = m == -INFINITY ? 0.f : m;
    float l = 0.f;
    for (int s = 0; s < nsplit; ++s)
        l += exp2f(part_ml[((size_t)s * n_rows + row) * 2] - use) * part_ml[((size_t)s * n_rows + row) * 2 + 1];
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float w = exp2f(part_ml[((size_t)s * n_rows + row) * 2] - use);
            if (w != 0.f) acc += w * part_o[((size_t)s * n_rows + row) * hd + d];
        }
        out[row * hd + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int HD, int NWARPS>
int launch_flash(__nv_bfloat16* out, float* part_o, float* part_ml, const __nv_bfloat16* q, const __nv_bfloat16* k_pool,
                 const __nv_bfloat16* v_pool, const int* cu, const int* ctx, const int* bt, int bt_stride, int B, int T,
                 int n_tiles, int num_pages, int page_size, int nh, int nkv, float scale, int window, int nsplit,
                 int* err, cudaStream_t stream) {
    constexpr int BM = 16 * NWARPS;
    const size_t smem = (size_t)(BM + 4 * FA_BN) * HD * 2;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_flash_kernel<HD, NWARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((unsigned)n_tiles, (unsigned)nkv, (unsigned)nsplit);
    CELLM_RUN((attention_flash_kernel<HD, NWARPS>), grid, NWARPS * 32, smem, stream,
              out, part_o, part_ml, q, k_pool, v_pool, cu, ctx, bt, bt_stride, B, T, num_pages, page_size, nh, nkv,
              scale * 1.4426950408889634f, window, err);
    return CELLM_OK;
}

}  // namespace

// Head sizes the tensor-core kernel is built for.
CELLM_API int cellm_attention_flash_supports(int hd) { return hd == 32 || hd == 64 || hd == 128; }

// out, q: [T, nh*hd] bf16. n_tiles: sum over requests of ceil(q_len * (nh/nkv) / rows_per_cta),
// rows_per_cta = 64 (wide = 1) or 16 (wide = 0). nsplit > 1 needs part_o
// [nsplit, T*nh, hd] and part_ml [nsplit, T*nh, 2] floats.
CELLM_API int cellm_attention_flash(void* out, float* part_o, float* part_ml, const void* q, const void* k_pool,
                                    const void* v_pool, const int* cu_seqlens, const int* ctx_lens,
                                    const int* block_table, int bt_stride, int B, int T, int n_tiles, int num_pages,
                                    int page_size, int nh, int nkv, int hd, float scale, int window, int wide,
                                    int nsplit, int* err, cudaStream_t stream) {
    if (T <= 0 || n_tiles <= 0) return CELLM_OK;
    if (nkv <= 0 || nh % nkv) return CELLM_ERR_SIZE;
    if (nsplit < 1 || (nsplit > 1 && (!part_o || !part_ml))) return CELLM_ERR_ARG;
    if (nkv > 65535 || nsplit > 65535) return CELLM_ERR_SIZE;
    int rc;
#define GO(HD_)                                                                                                   \
    rc = wide ? launch_flash<HD_, 4>((__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q,               \
                                     (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, cu_seqlens,      \
                                     ctx_lens, block_table, bt_stride, B, T, n_tiles, num_pages, page_size, nh,   \
                                     nkv, scale, window, nsplit, err, stream)                                     \
              : launch_flash<HD_, 1>((__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q,               \
                                     (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, cu_seqlens,      \
                                     ctx_lens, block_table, bt_stride, B, T, n_tiles, num_pages, page_size, nh,   \
                                     nkv, scale, window, nsplit, err, stream)
    if (hd == 32) GO(32);
    else if (hd == 64) GO(64);
    else if (hd == 128) GO(128);
    else return CELLM_ERR_SIZE;
#undef GO
    if (rc != CELLM_OK) return rc;
    if (nsplit > 1) {
        CELLM_RUN(attention_merge_kernel, (unsigned)((size_t)T * nh), hd >= 64 ? 64 : 32, 0, stream,
                  (__nv_bfloat16*)out, (const float*)part_o, (const float*)part_ml, (size_t)T * nh, hd, nsplit);
    }
    return CELLM_OK;
}

// ---------------------------------------------------------------------------
// Entry point that allocates nothing (declared in attention_flash_noalloc.h).
//
// Who it is for: code that drives the GPU from a place where device memory
// cannot be asked for — a host callback or a real-time thread that must not
// block inside the driver, a plugin that was handed a fixed arena and may not
// grow the process's footprint, a caller between graph replays that has to keep
// every pointer stable. The regular entry point above leaves the split pieces
// (unnormalised outputs, maxima, sums) to a workspace its caller allocates; this
// one keeps them in the fixed array below, which lives in the library's image:
// every GPU that loads the library holds these bytes until the process exits.
//
// Limits and rules:
//   * nsplit * T * nh * (hd + 2) floats must fit NOALLOC_SCRATCH_FLOATS (8 MiB);
//     larger calls are refused with CELLM_ERR_SCRATCH and nothing is launched.
//   * The first call on a device looks the array's device address up
//     (cudaGetSymbolAddress with that device current). Make that first call
//     outside any stream capture.
//   * T must be the number of tokens the call brings, cu_seqlens[B]: the merge reads the pieces of all T * nh
//     rows, and rows beyond cu_seqlens[B] were written by no kernel of this call.
//   * All calls share the one array. It keeps the previous call's contents;
//     nothing in it has to start at zero, because every (piece, row) the merge
//     reads is written by this call's first kernel. Two calls whose kernels
//     overlap on the GPU (different streams, or graphs replayed side by side)
//     race on it: serialise them.
//   * No cudaMalloc, cudaFree or allocating library call is made.
#define NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) float noalloc_scratch[NOALLOC_SCRATCH_FLOATS];

namespace {
float* noalloc_scratch_ptr[NOALLOC_MAX_DEVICES];   // device address of the array, per device; null until looked up
std::mutex noalloc_mutex;
}  // namespace

enum { CELLM_ERR_SCRATCH = -5, CELLM_ERR_DEVICE = -6 };

CELLM_API const char* cellm_attention_flash_noalloc_error(int code) {
    switch (code) {
        case CELLM_OK: return "ok";
        case CELLM_ERR_SCRATCH: return "nsplit * T * nh * (hd + 2) floats exceed the built-in scratch of 2097152 floats (8 MiB); use fewer pieces or fewer tokens per call";
        case CELLM_ERR_DEVICE: return "the current device could not be determined, or its index is beyond the 64 this entry point keeps addresses for";
        case CELLM_ERR_SIZE: return "a size the kernel does not take (head size must be 32, 64 or 128; heads a multiple of key/value heads)";
        case CELLM_ERR_ARG: return "nsplit must be at least 1";
        default: return code > 0 ? "a CUDA error (the code is a cudaError_t)" : "unknown error";
    }
}

CELLM_API long long cellm_attention_flash_noalloc_capacity() { return NOALLOC_SCRATCH_FLOATS; }

// Same arguments and result as cellm_attention_flash without the two workspace
// pointers. Inputs and the output are the caller's; the split pieces go to the
// library's own fixed array.
CELLM_API int cellm_attention_flash_noalloc(void* out, const void* q, const void* k_pool, const void* v_pool,
                                            const int* cu_seqlens, const int* ctx_lens, const int* block_table,
                                            int bt_stride, int B, int T, int n_tiles, int num_pages, int page_size,
                                            int nh, int nkv, int hd, float scale, int window, int wide, int nsplit,
                                            int* err, cudaStream_t stream) {
    if (nsplit < 1) return CELLM_ERR_ARG;
    // the sizes the kernel takes, before the question whether the pieces fit (so that a bad head size reads as one)
    if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || (hd != 32 && hd != 64 && hd != 128)) return CELLM_ERR_SIZE;
    if (T <= 0 || n_tiles <= 0) return CELLM_OK;
    const long long need = (long long)nsplit * T * nh * (hd + 2);
    if (nsplit > 1 && need > (long long)NOALLOC_SCRATCH_FLOATS) return CELLM_ERR_SCRATCH;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return CELLM_ERR_DEVICE;
    float* base;
    {
        std::lock_guard<std::mutex> lock(noalloc_mutex);
        if (noalloc_scratch_ptr[dev] == nullptr) {
            // In host code `noalloc_scratch` is only a handle for the symbol, not a device address.
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, noalloc_scratch);
            if (e != cudaSuccess) return (int)e;
            noalloc_scratch_ptr[dev] = static_cast<float*>(p);
        }
        base = noalloc_scratch_ptr[dev];
    }
    float* part_o = base;
    float* part_ml = base + (size_t)nsplit * T * nh * hd;
    return cellm_attention_flash(out, nsplit > 1 ? part_o : nullptr, nsplit > 1 ? part_ml : nullptr, q, k_pool, v_pool,
                                 cu_seqlens, ctx_lens, block_table, bt_stride, B, T, n_tiles, num_pages, page_size, nh,
                                 nkv, hd, scale, window, wide, nsplit, err, stream);
}
