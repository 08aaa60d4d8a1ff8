// Attention for prompt portions on the 5th-generation tensor cores (tcgen05),
// over the paged cache: bfloat16, heads of 64, causal, optional window.
//
// One CTA takes two tiles of 128 rows, the rows being (token, query head) pairs of
// the heads that share one key/value head (row r = token * G + head, G heads per
// key/value head, G a divisor of 128; the second tile holds the next 128 / G
// tokens), and walks the request's keys in blocks of 128; both tiles use each block
// of K and V, which is brought in once:
//   warp 0      TMA: the Q tiles once (3-D boxes over [token][head][64]), then per
//               block the K and V pages through the block table (one box per page),
//               into rings of three stages each, 128-byte swizzle;
//   warp 1      MMA: per tile S = Q.K^T (M 128, N 128, K 64) into the tile's score
//               columns of tensor memory, and O += P.V (M 128, N 64, K 128) with P read
//               from tensor memory and V as it lies in its pages (MN-major);
//   warps 2..5  softmax of the first tile, warps 6..9 of the second, one row per
//               thread: the 128 scores from tensor memory into registers (the next
//               block's product may then overwrite them), mask, running maximum and sum
//               in 32-bit, P = 2^(s*c - m) rounded to bfloat16 into tensor memory, two keys
//               a column, where the MMA reads it as its A operand (shared memory carries
//               only Q, K and V: its bandwidth is what the tensor cores' operands need).
//               Two threads a row (eight warps a tile) were measured slower: the loads
//               from tensor memory and the exponentials of four warps a scheduler collide.
// While one tile's softmax runs, the tensor cores work on the other tile. The output
// accumulators stay in tensor memory; one is rescaled (read, multiplied, written
// back) only when a row's maximum has grown by more than 2^8 since the last rescale,
// so most blocks skip that pass; the stale maximum only scales P.
//
// Every wait on an mbarrier is bounded, as in gemm_tcgen05.cu: a role that gives up
// sets CELLM_DEV_WAIT_TIMEOUT and an abort flag; the CTA frees its tensor memory and
// returns. Scores (q.k * scale), mask and softmax follow
// crates/cellm-cache/src/kvcache.rs:753-787, :1206-1227.
//
// Cache layout of one layer: [page][kv_head][slot in page][64].
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int TM = 128;          // rows of a tile
constexpr int TN = 128;          // keys of a block
constexpr int HD = 64;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;
constexpr float RESCALE_STEP = 8.0f;   // in log2 units

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Descriptor of a tile with 128-byte rows under the 128-byte swizzle, eight rows
// per 1024 bytes. The same bits describe a K-major operand (rows = M or N, the 128
// bytes run along K) and an MN-major one (rows = K, the 128 bytes run along N);
// which of the two is meant is said by the instruction descriptor.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D float, A and B bfloat16; b_mn: B is MN-major (bit 16).
__device__ __forceinline__ uint32_t umma_idesc(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with A read from tensor memory (row = lane, two bfloat16 of K in a column)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// 128 columns of one lane quarter, issued back to back and awaited once
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

constexpr int KV_STAGES = 3;
constexpr int TMEM_TN = 512;       // scores of tile 0 and 1 in columns 0 and 128, their outputs in 256 and 320,
constexpr int O_COL = 256;           // their P (bfloat16, two keys a column) in 384 and 448
constexpr int P_COL = 384;
constexpr int THREADS = 320;         // warp 0 TMA, warp 1 MMA, warps 2..5 softmax of tile 0, warps 6..9 of tile 1

// 128 KB and a few words: one CTA per SM (it holds all 512 columns of tensor memory).
struct TcSmem {                                  // starts on a 1024-byte boundary (checked in the kernel)
    uint8_t q[2][TM * HD * 2];                   // 16 KB each
    uint8_t k[KV_STAGES][TN * HD * 2];           // 16 KB each
    uint8_t v[KV_STAGES][TN * HD * 2];
    uint64_t q_full;
    uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
    uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[2], s_empty[2], p_full[2], pv_done[2];
    uint32_t tmem_base;
    int abort_flag;
};

// The key blocks one tile of 128 rows needs: [lo, hi) in units of TN keys, and its rows' tokens.
struct TileRange {
    int tok0;        // first token of the tile within the portion
    int lo, hi;      // key blocks
    bool has;        // the tile holds at least one token
};

// Launched with 320 threads. A scheduler holds three of the ten warps and 16384 registers: 168 a thread at
// most, which the bound of 384 threads makes the compiler keep.
__global__ void __launch_bounds__(384, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens,
                    const int* __restrict__ block_table, int bt_stride, int B, int num_pages, int page_size, int nh,
                    int nkv, float scale_log2e, int window, int* __restrict__ err) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    TcSmem& sm = *reinterpret_cast<TcSmem*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = nh / nkv, kvh = blockIdx.y;
    const int tok_per_tile = TM / G, tok_per_cta = 2 * tok_per_tile;
    if (smem_u32(smem_raw) & 1023u) {            // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_LAYOUT);
        return;
    }

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&sm.k_full[i], 1); mbar_init(&sm.k_empty[i], 1);
            mbar_init(&sm.v_full[i], 1); mbar_init(&sm.v_empty[i], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&sm.s_full[t], 1);  mbar_init(&sm.s_empty[t], 128);
            mbar_init(&sm.p_full[t], 128); mbar_init(&sm.pv_done[t], 1);
        }
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    // V stages start as zeros: rows that are never loaded must not carry NaN bits into P.V (0 * NaN);
    // what K rows hold there does not matter, their scores are masked
    for (int i = threadIdx.x; i < (int)sizeof(sm.v) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(sm.v)[i] = make_uint4(0, 0, 0, 0);
    proxy_fence();
    if (warp == 1) tmem_alloc(&sm.tmem_base, TMEM_TN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_trigger();
    pdl_wait();
    const uint32_t tmem = sm.tmem_base;
    volatile int* abort_flag = &sm.abort_flag;

    // which request this pair of tiles belongs to (from the last to the first: longest first)
    const int item = (int)gridDim.x - 1 - (int)blockIdx.x;
    int b = 0, base = 0;
    for (; b < B; ++b) {
        const int nt = (cu_seqlens[b + 1] - cu_seqlens[b] + tok_per_cta - 1) / tok_per_cta;
        if (item < base + nt) break;
        base += nt;
    }
    const bool live = b < B;
    int t_base = 0, q_len = 0, ctx = 0;
    TileRange tr[2] = {{0, 0, 0, false}, {0, 0, 0, false}};
    int kb0 = 0, nblk = 0, key_begin = 0, key_end = 0;
    if (live) {
        t_base = cu_seqlens[b];
        q_len = cu_seqlens[b + 1] - t_base;
        ctx = ctx_lens[b];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            tr[t].tok0 = (item - base) * tok_per_cta + t * tok_per_tile;
            tr[t].has = tr[t].tok0 < q_len;
            if (tr[t].has) {
                const int tok1 = min(tr[t].tok0 + tok_per_tile, q_len) - 1;
                const int kb = window > 0 ? max(0, ctx + tr[t].tok0 - window + 1) : 0;
                tr[t].lo = kb / TN;
                tr[t].hi = (ctx + tok1 + 1 + TN - 1) / TN;
                if (t == 0) key_begin = kb;
                key_end = ctx + tok1 + 1;
            }
        }
        // tile 1 holds later tokens: its blocks start and end no earlier than tile 0's
        kb0 = tr[0].lo;
        nblk = (tr[1].has ? tr[1].hi : tr[0].hi) - kb0;
    }
    const int* bt = block_table + (size_t)(live ? b : 0) * bt_stride;
    const int pages_per_block = TN / page_size;
    auto active = [&](int t, int j) { return tr[t].has && kb0 + j >= tr[t].lo && kb0 + j < tr[t].hi; };

    if (warp == 0) {
        if (live) {
            if (lane == 0) {
                mbar_expect_tx(&sm.q_full, (tr[1].has ? 2 : 1) * TM * HD * 2);
                tma_load_3d(sm.q[0], &map_q, 0, kvh * G, t_base + tr[0].tok0, &sm.q_full);
                if (tr[1].has) tma_load_3d(sm.q[1], &map_q, 0, kvh * G, t_base + tr[1].tok0, &sm.q_full);
            }
            for (int j = 0; j < nblk; ++j) {
                const int st = j % KV_STAGES;
                const uint32_t ph = (uint32_t)(j / KV_STAGES) & 1u;
                // lane i brings page i of the block
                const int key0 = (kb0 + j) * TN + lane * page_size;
                int page = -1;
                if (lane < pages_per_block && key0 < key_end && key0 + page_size > key_begin) {
                    page = bt[key0 / page_size];
                    if (page < 0 || page >= num_pages) { atomicOr(err, CELLM_DEV_BAD_PAGE); page = -1; }
                }
                const unsigned have = __ballot_sync(0xffffffffu, page >= 0);
                const uint32_t bytes = (uint32_t)__popc(have) * (uint32_t)page_size * HD * 2;
                const int row = (page * nkv + kvh) * page_size;
                bool ok = true;
                if (lane == 0) ok = mbar_wait(&sm.k_empty[st], ph ^ 1u, abort_flag);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) { if (lane == 0) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); } break; }
                if (lane == 0) mbar_expect_tx(&sm.k_full[st], bytes);
                __syncwarp();
                if (page >= 0) tma_load_2d(sm.k[st] + (size_t)lane * page_size * HD * 2, &map_k, 0, row, &sm.k_full[st]);
                if (lane == 0) ok = mbar_wait(&sm.v_empty[st], ph ^ 1u, abort_flag);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) { if (lane == 0) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); } break; }
                if (lane == 0) mbar_expect_tx(&sm.v_full[st], bytes);
                __syncwarp();
                if (page >= 0) tma_load_2d(sm.v[st] + (size_t)lane * page_size * HD * 2, &map_v, 0, row, &sm.v_full[st]);
            }
        }
    } else if (warp == 1) {
        if (live && lane == 0) {
            const uint32_t idesc_s = umma_idesc(TM, TN, false);      // S[128 x 128] = Q (K-major) . K^T (K-major)
            const uint32_t idesc_o = umma_idesc(TM, HD, true);       // O[128 x 64] += P (K-major) . V (MN-major)
            int n_s[2] = {0, 0}, n_pv[2] = {0, 0};                   // products issued so far, per tile
            bool ok = mbar_wait(&sm.q_full, 0, abort_flag);
            // scores of block j for the tiles that need it; the softmax warps of a tile must have taken
            // the tile's last scores out of tensor memory first
            auto issue_s = [&](int j) -> bool {
                const int st = j % KV_STAGES;
                if (!mbar_wait(&sm.k_full[st], (uint32_t)(j / KV_STAGES) & 1u, abort_flag)) return false;
                const uint64_t dk = umma_desc(smem_u32(sm.k[st]));
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (!active(t, j)) continue;
                    if (n_s[t] > 0 && !mbar_wait(&sm.s_empty[t], (uint32_t)(n_s[t] - 1) & 1u, abort_flag)) return false;
                    tc_fence_after();
                    const uint64_t dq = umma_desc(smem_u32(sm.q[t]));
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks)
                        umma_bf16(tmem + (uint32_t)(t * TN), dq + (uint64_t)(ks * 2), dk + (uint64_t)(ks * 2), idesc_s, ks != 0 ? 1u : 0u);
                    umma_commit(&sm.s_full[t]);
                    ++n_s[t];
                }
                umma_commit(&sm.k_empty[st]);
                return true;
            };
            if (ok && nblk > 0) ok = issue_s(0);
            for (int j = 0; ok && j < nblk; ++j) {
                const int st = j % KV_STAGES;
                if (j + 1 < nblk) { ok = issue_s(j + 1); if (!ok) break; }
                ok = mbar_wait(&sm.v_full[st], (uint32_t)(j / KV_STAGES) & 1u, abort_flag);
                if (!ok) break;
                const uint64_t dv = umma_desc(smem_u32(sm.v[st]));
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (!active(t, j)) continue;
                    ok = mbar_wait(&sm.p_full[t], (uint32_t)n_pv[t] & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < TN / 16; ++ks) {
                        const uint32_t pa = tmem + (uint32_t)(P_COL + t * (TN / 2) + ks * 8);     // 16 keys = 8 columns of P
                        const uint64_t db = dv + (uint64_t)(ks * 16 * HD * 2 / 16);               // 16 keys = 16 rows of V
                        umma_bf16_ts(tmem + (uint32_t)(O_COL + t * HD), pa, db, idesc_o, (n_pv[t] | ks) != 0 ? 1u : 0u);
                    }
                    umma_commit(&sm.pv_done[t]);
                    ++n_pv[t];
                }
                if (!ok) break;
                umma_commit(&sm.v_empty[st]);
            }
            if (!ok) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); }
        }
    } else if (live && tr[(warp - 2) >> 2].has) {
        const int t = (warp - 2) >> 2;                                // which tile
        const int qt = warp & 3;                                      // quarter of the tile's rows = of tensor memory's lanes
        const int r = qt * 32 + lane;                                 // row of the tile = lane of tensor memory
        const int tok = tr[t].tok0 + r / G;                           // token within the portion
        const bool row_ok = tok < q_len;
        const int pos = row_ok ? ctx + tok : -1;
        const int lo = window > 0 ? pos - window + 1 : 0;
        const uint32_t lane_base = tmem + ((uint32_t)(qt * 32) << 16);
        const uint32_t s_col = (uint32_t)(t * TN);
        const uint32_t o_col = (uint32_t)(O_COL + t * HD);
        const uint32_t p_col = (uint32_t)(P_COL + t * (TN / 2));
        const int n_blocks = tr[t].hi - tr[t].lo;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_blocks; ++it) {
            ok = mbar_wait(&sm.s_full[t], (uint32_t)it & 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t s[TN];
#pragma unroll
            for (int c = 0; c < TN / 32; ++c) tmem_ld32_nowait(lane_base + s_col + (uint32_t)(c * 32), s + c * 32);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&sm.s_empty[t]);                              // the scores are in registers now
            const int jbase = (tr[t].lo + it) * TN;
            const bool open_block = row_ok && jbase + TN - 1 <= pos && (window <= 0 || jbase >= lo);
            if (!open_block) {
#pragma unroll
                for (int i = 0; i < TN; ++i) {
                    const int key = jbase + i;
                    if (!(key <= pos && key >= lo)) s[i] = 0xff800000u;            // -inf
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < TN; i += 4) {
                mx0 = fmaxf(mx0, __uint_as_float(s[i]));     mx1 = fmaxf(mx1, __uint_as_float(s[i + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(s[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(s[i + 3]));
            }
            const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2e);
            // rescale O only when the maximum has grown much (or nothing has been accumulated with it yet);
            // the accumulator (and below, P) is free once the last block's P.V is done
            const bool want = m_new > m + RESCALE_STEP || (m == -INFINITY && m_new != -INFINITY);
            bool pv_seen = it == 0;
            if (__any_sync(0xffffffffu, want)) {
                if (it > 0) {
                    ok = mbar_wait(&sm.pv_done[t], (uint32_t)(it - 1) & 1u, abort_flag);
                    if (!ok) break;
                    pv_seen = true;
                    tc_fence_after();
                    const float corr = want ? (m == -INFINITY ? 0.f : fast_exp2(m - m_new)) : 1.0f;
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + o_col + (uint32_t)(c * 32), o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st32(lane_base + o_col + (uint32_t)(c * 32), o);
                    }
                    if (want) l *= corr;
                }
                if (want) m = m_new;
            }
            // P = 2^(s*c - m) in place (-inf gives 0), then rounded to bfloat16 pairs (in place again)
            const float neg_use = m == -INFINITY ? 0.f : -m;
#pragma unroll
            for (int i = 0; i < TN; ++i) s[i] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(s[i]), scale_log2e, neg_use)));
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
            for (int i = 0; i < TN / 2; i += 2) {
                const float a0 = __uint_as_float(s[2 * i]), a1 = __uint_as_float(s[2 * i + 1]);
                const float a2 = __uint_as_float(s[2 * i + 2]), a3 = __uint_as_float(s[2 * i + 3]);
                sum0 += a0; sum1 += a1; sum2 += a2; sum3 += a3;
                s[i] = pack_bf16(a0, a1);
                s[i + 1] = pack_bf16(a2, a3);
            }
            l += (sum0 + sum1) + (sum2 + sum3);
            if (!pv_seen) {
                ok = mbar_wait(&sm.pv_done[t], (uint32_t)(it - 1) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
            }
#pragma unroll
            for (int c = 0; c < TN / 64; ++c) tmem_st32_nowait(lane_base + p_col + (uint32_t)(c * 32), s + c * 32);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&sm.p_full[t]);
        }
        if (ok && n_blocks > 0) ok = mbar_wait(&sm.pv_done[t], (uint32_t)(n_blocks - 1) & 1u, abort_flag);
        if (!ok && lane == 0) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); }
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* dst = out + (size_t)(t_base + tok) * nh * HD + (size_t)(kvh * G + r % G) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_base + o_col + (uint32_t)(c * 32), o);
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t w4[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            w4[k] = pack_bf16(__uint_as_float(o[8 * i + 2 * k]) * inv, __uint_as_float(o[8 * i + 2 * k + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_TN);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

bool encode(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
            const cuuint32_t* box) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Whether the kernel takes these sizes.
CELLM_API int cellm_attention_tc_supports(int hd, int nh, int nkv, int page_size) {
    if (hd != 64 || nkv <= 0 || nh % nkv) return 0;
    const int G = nh / nkv;
    if (G > 128 || 128 % G) return 0;
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

// out, q: [T, nh*64] bf16; pools: one layer's [pages][nkv][page_size][64] bf16. n_tiles = sum over the
// requests of ceil(q_len / (256 / (nh/nkv))): a CTA takes two tiles of 128 rows that share their keys.
CELLM_API int cellm_attention_tc(void* out, const void* q, const void* k_pool, const void* v_pool,
                                 const int* cu_seqlens, const int* ctx_lens, const int* block_table, int bt_stride,
                                 int B, int T, int n_tiles, int num_pages, int page_size, int nh, int nkv, int hd,
                                 float scale, int window, int* err, cudaStream_t stream) {
    if (T <= 0 || n_tiles <= 0) return CELLM_OK;
    if (!cellm_attention_tc_supports(hd, nh, nkv, page_size) || scale <= 0.f) return CELLM_ERR_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return CELLM_ERR_ALIGN;
    const int G = nh / nkv;
    CUtensorMap mq, mk, mv;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)T};
        const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)nh * HD * 2};
        const cuuint32_t box[3] = {(cuuint32_t)HD, (cuuint32_t)G, (cuuint32_t)(TM / G)};
        if (!encode(&mq, q, 3, dims, strides, box)) return CELLM_ERR_ARG;
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)num_pages * nkv * page_size};
        const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        const cuuint32_t box[2] = {(cuuint32_t)HD, (cuuint32_t)page_size};
        if (!encode(&mk, k_pool, 2, dims, strides, box) || !encode(&mv, v_pool, 2, dims, strides, box)) return CELLM_ERR_ARG;
    }
    const size_t smem = sizeof(TcSmem);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((unsigned)n_tiles, (unsigned)nkv);
    CELLM_RUN(attention_tc_kernel, grid, THREADS, smem, stream, mq, mk, mv, (__nv_bfloat16*)out, cu_seqlens,
              ctx_lens, block_table, bt_stride, B, num_pages, page_size, nh, nkv, scale * 1.4426950408889634f, window, err);
    return CELLM_OK;
}
