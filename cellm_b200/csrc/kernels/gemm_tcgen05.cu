// bfloat16 matrix product on the 5th-generation tensor cores:
//   C[M,N] = A[M,K] . W[N,K]^T, 32-bit accumulation in tensor memory.
//
// One CTA computes one 128 x BN tile of C. Three roles, one warp each or four:
//   warp 0      TMA producer: cp.async.bulk.tensor loads 128x64 of A and BNx64 of W
//               (128-byte swizzle) into a ring of shared-memory stages;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) four
//               times per stage, accumulating into BN columns of tensor memory, and
//               releases each stage with tcgen05.commit;
//   warps 2..5  epilogue: tcgen05.ld of the accumulator (one row per thread),
//               conversion, and guarded stores to C.
// Rows and columns beyond M, N and K are zero-filled by the TMA unit, so any
// M and N are taken; K must be a multiple of 8 (16-byte row pitch).
//
// Every wait on an mbarrier is bounded: after about a second without progress
// the waiting role sets CELLM_DEV_WAIT_TIMEOUT in the error word and leaves its
// loop; the CTA then frees its tensor memory and returns.
//
// Skinny products (few rows of A: decoding) run "swapped": the 128-row operand
// is a tile of W, the narrow operand (16, 32 or 64 rows) is A, so the tensor
// core tile is filled by weights and the stage ring holds almost only weights;
// the epilogue then writes its tile transposed.
//
// With split_k > 1 (skinny products, M small) blockIdx.z selects a slice of K;
// each slice writes its partial tile as float into a workspace [split_k, M, N]
// and the slice that finishes last sums them in a fixed order (see the kernel).
//
// Epilogues (template parameter EPI of gemm_tcgen05_kernel; each is described where it is defined):
//   0  C = A.W^T                      1  SwiGLU over interleaved gate and up blocks
//   2  in_proj + gated short convolution of a decode step (cellm_gemm_conv_tcgen05)
//   3  q/k/v product + head norms + rotation + cache write of a decode step (cellm_gemm_rope_tcgen05)
// 2 and 3 exist for swapped tiles whose K split is summed inside a cluster.
//
// The kernel takes part in programmatic dependent launch: barrier set-up, the
// tensor-memory allocation and the loads of W for the first stages run before
// the wait on the preceding kernel; only loads of A and all stores come after.
#include "tcgen05.cuh"

namespace {

// RED: floats in which a CTA receives, from every CTA of its cluster, the pieces of the tokens whose sums it owns.
template <int BN, int STAGES, int RED = 0>
struct alignas(1024) GemmSmem {
    uint8_t a[STAGES][BM * BK * 2];
    uint8_t b[STAGES][BN * BK * 2];
    float red[RED > 0 ? RED : 1];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full;
    uint64_t acc_full2[2];     // persistent kernel: one per accumulator buffer
    uint64_t acc_empty2[2];
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
    int conv_slots[64];         // EPI = 2: the state slots of the tile's tokens
    int rope_pos[64];           // EPI = 3: position and page of the tile's tokens
    int rope_page[64];
    float ex_ss[4];             // EPI = 3: the epilogue warps' sums of squares and normed values of one token
    float ex_y[128];
};

template <typename TO> __device__ __forceinline__ void store_row(TO* dst, const uint32_t* r, int valid, bool aligned);
template <> __device__ __forceinline__ void store_row<float>(float* dst, const uint32_t* r, int valid, bool aligned) {
    if (valid >= 32 && aligned) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = __uint_as_float(r[i]);
    }
}
template <> __device__ __forceinline__ void store_row<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t* r, int valid, bool aligned) {
    if (valid >= 32 && aligned) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * j]), __uint_as_float(r[8 * i + 2 * j + 1]));
                p[j] = *reinterpret_cast<uint32_t*>(&v);
            }
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(p[0], p[1], p[2], p[3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
    }
}

// The 128-row operand ("rows") and the BN-row operand ("cols") of a tile:
//   SWAP = false: rows = A (tokens),  cols = W;  grid (ceil(N/BN),  ceil(M/128), split_k); tile element (p, q) -> C[p][q]
//   SWAP = true:  rows = W,           cols = A;  grid (ceil(N/128), ceil(M/BN),  split_k); tile element (p, q) -> C[q][p]
//
// EPI = 0: C[M, N] = A.W^T.
// EPI = 1: W holds blocks of 64 gate rows followed by their 64 up rows; the
//          output is C[M, N/2] with C[m][64j + i] = silu(g) * u for
//          g = (A.W^T)[m][128j + i], u = (A.W^T)[m][128j + 64 + i].
//
// A tile goes through the float workspace ws[split][M][N] when K is split
// (gridDim.z > 1) or when gate and up sit in different threads (EPI = 1 with
// SWAP). With a split, every CTA of a tile adds one to the tile's counter after
// its piece is written; the CTA that finds the counter at split_k - 1 sums all
// pieces in the order of the splits, writes the output and sets the counter
// back to zero. No CTA waits for another.
//
// CLUSTER (swapped tiles only): the CTAs of a tile's K split form one thread-block
// cluster (gridDim.z of them, at most 8). Token t of the tile is summed by the CTA of
// rank t mod split: every CTA stores its piece of that token straight into the owner's
// shared memory (slot t / split of the sender's own plane, so nobody writes where
// another does), and after one cluster barrier every CTA adds the planes of its tokens
// in the order of the ranks, out of its own memory, and writes those outputs. No
// workspace, no counter, no fence to global memory, and no CTA reads a peer's memory, so
// none has to wait for the others before it leaves.
//
// EPI = 2 (swapped tiles in a cluster; every token of the step belongs to a request of its own):
// the gated short convolution in the epilogue of its in_proj. W is in_proj cut into tiles of 128
// rows that hold, for 42 channels each, the 42 rows of B, of C and of x (two rows of padding), so
// that the thread of a channel finds all three sums in its tile. It rounds them to bfloat16 as
// the plain product would have stored them, forms B*x, takes the request's last taps-1 values
// of B*x from its state slot, writes y = C * (taps . history) and moves the state on by one.
//
// EPI = 3 (swapped tiles in a cluster; every token of the step belongs to a request of its own; heads
// of 64): W is q_proj | k_proj | v_proj, so a tile of 128 rows is two whole heads. After the cluster's
// reduction the two warps of a head hold one token's 64 sums: they round them to bfloat16 as the plain
// product would have stored them, take the head's RMSNorm (q and k heads), turn the pairs (i, i + 32)
// by the token's position and write queries to C [M, nh * 64], keys and values to the request's page.
constexpr int CONV_CH = 42;          // channels per tile of 128 rows

template <int BN, int STAGES, bool SWAP, int EPI, bool CLUSTER, typename TO>
__global__ void __launch_bounds__(192, SWAP ? 2 : 1)      // swapped tiles: two CTAs an SM, so the next product's can move in early
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                    TO* __restrict__ C, float* __restrict__ ws, int* __restrict__ counters, int M, int N, int K,
                    long long ldc, int kblocks_per_split, int w_is_static, int* __restrict__ err, const ConvEpi conv, const RopeEpi rope) {
    static_assert(!CLUSTER || SWAP, "the cluster reduction serves swapped tiles");
    static_assert(EPI < 2 || CLUSTER, "the convolution and rotation epilogues are written for the cluster's reduction");
    extern __shared__ uint8_t smem_raw[];
    using Smem = GemmSmem<BN, STAGES, CLUSTER ? (BN + 8) * BM : 0>;
    auto& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = (SWAP ? blockIdx.x : blockIdx.y) * BM;    // first row of the 128-row operand
    const int q0 = (SWAP ? blockIdx.y : blockIdx.x) * BN;    // first row of the narrow operand
    const int P = SWAP ? N : M, Q = SWAP ? M : N;
    const int kblocks_total = (K + BK - 1) / BK;
    const int splits = gridDim.z;
    const int kb0 = blockIdx.z * kblocks_per_split;
    const int kb1 = min(kb0 + kblocks_per_split, kblocks_total);
    const int nkb = kb1 - kb0;           // > 0 by construction of the grid

    pdl_trigger();                       // the next kernel may set itself up beside this one
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        mbar_init(&sm.acc_full, 1);
        sm.abort_flag = 0;
        sm.is_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_rows) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_cols) : "memory");
    }
    if (warp == 1) tmem_alloc(&sm.tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if constexpr (CLUSTER) cluster_arrive();     // this CTA runs: peers may store into its shared memory
    const uint32_t tmem = sm.tmem_base;
    volatile int* abort_flag = &sm.abort_flag;
    // EPI = 2: what an epilogue thread fetches ahead of the accumulator (see there)
    float cv_wt[CONV_MAX_TAPS - 1] = {}, cv_hist[CONV_MAX_TAPS - 1] = {}, cv_wlast = 0.f, cv_bias = 0.f;
    bool cv_active = false;
    // EPI = 3: this thread's norm weight and its frequency
    float rp_w = 0.f, rp_hi = 0.f, rp_lo = 0.f;

    if (warp == 0) {
        if (lane == 0) {
            // Weights that no kernel writes (w_is_static) do not depend on the kernel
            // before this one: their loads for the first stages go out before the wait
            // on that kernel, the activations' loads after it.
            if (!w_is_static) pdl_wait();
            const CUtensorMap* map_w = SWAP ? &map_rows : &map_cols;
            const CUtensorMap* map_x = SWAP ? &map_cols : &map_rows;
            const int w0 = SWAP ? p0 : q0, x0 = SWAP ? q0 : p0;
            const int early = nkb < STAGES ? nkb : STAGES;
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(&sm.full[i], (BM + BN) * BK * 2);
                tma_load_2d(SWAP ? (void*)sm.a[i] : (void*)sm.b[i], map_w, (kb0 + i) * BK, w0, &sm.full[i]);
            }
            // Static weights beyond the ring are asked into L2 meanwhile, so that after
            // the wait they stream from there; up to 64 blocks (1 MiB of weights) a CTA.
            if (w_is_static > 1)
                for (int i = early; i < nkb && i < early + w_is_static; ++i) tma_prefetch_l2_2d(map_w, (kb0 + i) * BK, w0);
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(SWAP ? (void*)sm.b[i] : (void*)sm.a[i], map_x, (kb0 + i) * BK, x0, &sm.full[i]);
            for (int i = early; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(&sm.empty[s], phase ^ 1u, abort_flag)) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); break; }
                mbar_expect_tx(&sm.full[s], (BM + BN) * BK * 2);
                tma_load_2d(sm.a[s], &map_rows, (kb0 + i) * BK, p0, &sm.full[s]);
                tma_load_2d(sm.b[s], &map_cols, (kb0 + i) * BK, q0, &sm.full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BM, BN);
            bool ok = true;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(&sm.full[s], phase, abort_flag)) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); ok = false; break; }
                tc_fence_after();
                const uint64_t da = umma_desc(smem_u32(sm.a[s])), db = umma_desc(smem_u32(sm.b[s]));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_bf16(tmem, da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16), idesc,
                              (i | k) != 0 ? 1u : 0u);
                umma_commit(&sm.empty[s]);
            }
            if (ok) umma_commit(&sm.acc_full);
        }
    } else {
        if constexpr (EPI == 2) {
            // While the products run: the slots of the tile's tokens, this thread's taps and the history of its
            // first token. None of it is the work of a kernel of this step (the state was last written by this
            // kernel one step ago), so it does not wait for the kernel before this one.
            const int pl = (warp & 3) * 32 + lane;
            if (pl < BN) sm.conv_slots[pl] = q0 + pl < Q ? conv.slot_ids[q0 + pl] : -1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int sub = pl / CONV_CH, ch = (p0 / BM) * CONV_CH + pl % CONV_CH;
            cv_active = sub < 3 && ch < conv.H;
            if (cv_active) {
                const int rows = conv.ntaps - 1;
#pragma unroll
                for (int k = 0; k < CONV_MAX_TAPS - 1; ++k)
                    cv_wt[k] = k < rows ? __bfloat162float(conv.taps[(size_t)ch * conv.ntaps + k]) : 0.f;
                cv_wlast = __bfloat162float(conv.taps[(size_t)ch * conv.ntaps + rows]);
                cv_bias = conv.bias ? __bfloat162float(conv.bias[ch]) : 0.f;
                const int ql = (int)cluster_rank() + sub * splits;       // this thread's first token of the tile
                const int slot = ql < BN ? sm.conv_slots[ql] : -1;
#pragma unroll
                for (int k = 0; k < CONV_MAX_TAPS - 1; ++k)
                    cv_hist[k] = (k < rows && slot >= 0 && slot < conv.n_slots)
                                     ? conv.state[(long long)slot * conv.slot_stride + (size_t)k * conv.H + ch] : 0.f;
            }
        }
        if constexpr (EPI == 3) {
            // While the products run: positions and pages of the tile's tokens (the step's inputs, the work of no
            // kernel of this step), this thread's norm weight and frequency.
            const int pl = (warp & 3) * 32 + lane;
            if (pl < BN) {
                int pos = 0, page = -1;
                if (q0 + pl < Q) {
                    pos = rope.positions[q0 + pl];
                    page = rope.block_table[(size_t)(q0 + pl) * rope.bt_stride + pos / rope.page_size];
                }
                sm.rope_pos[pl] = pos;
                sm.rope_page[pl] = page;
            }
            const int hh = p0 / 64 + (pl >> 6), i = pl & 63;
            if (hh < rope.nh) rp_w = __bfloat162float(rope.q_w[i]);
            else if (hh < rope.nh + rope.nkv) rp_w = __bfloat162float(rope.k_w[i]);
            rp_hi = rope.inv_freq[2 * lane];
            rp_lo = rope.inv_freq[2 * lane + 1];
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const bool ok = mbar_wait(&sm.acc_full, 0, abort_flag);
        if (!ok && lane == 0) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); }
        tc_fence_after();
        pdl_wait();     // global writes below must not pass the kernel before this one
        const int qtr = warp & 3;                     // the quarter of the lanes this warp may read
        const int pl = qtr * 32 + lane;               // row of the tile this thread holds
        const int p = p0 + pl;
        const uint32_t lane_addr = tmem + ((uint32_t)(qtr * 32) << 16);
        const bool through_ws = !CLUSTER && (splits > 1 || (EPI == 1 && SWAP));
        if constexpr (CLUSTER) {
            // This CTA's piece goes to the owners of its tokens: plane `rank` of the owner's buffer, [slot][row of the tile].
            constexpr int W = BN < 32 ? 16 : 32;
            cluster_wait();                      // every CTA of the cluster has started
            const uint32_t rank = cluster_rank();
            const int slots = (BN + splits - 1) / splits;           // tokens of a tile that one CTA can own
            const int valid = min(Q - q0, BN);
            float* plane = sm.red + (size_t)rank * slots * BM + pl;
#pragma unroll 1
            for (int c = 0; c < BN / W; ++c) {
                if (c * W >= valid) break;
                uint32_t r[W];
                if (ok) {
                    if constexpr (W == 16) tmem_ld16(lane_addr + (uint32_t)(c * W), r);
                    else tmem_ld32(lane_addr + (uint32_t)(c * W), r);
                }
                int owner = (c * W) % splits, slot = (c * W) / splits;
#pragma unroll
                for (int j = 0; j < W; ++j) {
                    if (c * W + j < valid) st_peer_shared(plane + slot * BM, (uint32_t)owner, ok ? __uint_as_float(r[j]) : 0.f);
                    if (++owner == splits) { owner = 0; ++slot; }
                }
            }
        }
        if (ok && !through_ws && !CLUSTER) {
            if constexpr (EPI == 0 && !SWAP) {
                const bool aligned = ((reinterpret_cast<uintptr_t>(C) | (uintptr_t)(ldc * sizeof(TO))) & 15) == 0 &&
                                     ((q0 * sizeof(TO)) & 15) == 0;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(lane_addr + (uint32_t)(c * 32), r);
                    const int q = q0 + c * 32;
                    if (p < P && q < Q) store_row<TO>(C + (size_t)p * ldc + q, r, Q - q, aligned);
                }
            } else if constexpr (EPI == 0 && SWAP) {
                constexpr int W = BN < 32 ? 16 : 32;
#pragma unroll 1
                for (int c = 0; c < BN / W; ++c) {
                    uint32_t r[W];
                    if constexpr (W == 16) tmem_ld16(lane_addr + (uint32_t)(c * W), r);
                    else tmem_ld32(lane_addr + (uint32_t)(c * W), r);
                    if (p < P) {
#pragma unroll
                        for (int j = 0; j < W; ++j) {
                            const int q = q0 + c * W + j;
                            if (q < Q) C[(size_t)q * ldc + p] = from_float<TO>(__uint_as_float(r[j]));
                        }
                    }
                }
            } else if constexpr (EPI == 1 && !SWAP && BN >= 128) {
                // columns of the tile come as [64 gate | 64 up] per 128: both halves are in this thread
                const int o0 = q0 / 2;
                const bool aligned = ((reinterpret_cast<uintptr_t>(C) | (uintptr_t)(ldc * sizeof(TO))) & 15) == 0 &&
                                     ((o0 * sizeof(TO)) & 15) == 0;
#pragma unroll 1
                for (int j = 0; j < BN / 128; ++j) {
#pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        uint32_t g[32], u[32];
                        tmem_ld32(lane_addr + (uint32_t)(j * 128 + h * 32), g);
                        tmem_ld32(lane_addr + (uint32_t)(j * 128 + 64 + h * 32), u);
#pragma unroll
                        for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(silu_mul(__uint_as_float(g[i]), __uint_as_float(u[i])));
                        const int o = o0 + j * 64 + h * 32;
                        if (p < P && o < Q / 2) store_row<TO>(C + (size_t)p * ldc + o, g, Q / 2 - o, aligned);
                    }
                }
            }
        }
        if (through_ws) {
            float* mine = ws + (size_t)blockIdx.z * (size_t)M * (size_t)N;
            if (ok) {
                constexpr int W = BN < 32 ? 16 : 32;
#pragma unroll 1
                for (int c = 0; c < BN / W; ++c) {
                    uint32_t r[W];
                    if constexpr (W == 16) tmem_ld16(lane_addr + (uint32_t)(c * W), r);
                    else tmem_ld32(lane_addr + (uint32_t)(c * W), r);
                    if (p < P) {
                        if constexpr (SWAP) {
#pragma unroll
                            for (int j = 0; j < W; ++j) {
                                const int q = q0 + c * W + j;
                                if (q < Q) mine[(size_t)q * N + p] = __uint_as_float(r[j]);
                            }
                        } else {
                            const int q = q0 + c * W;
                            if (q < Q) store_row<float>(mine + (size_t)p * N + q, r, Q - q, (N & 3) == 0);
                        }
                    }
                }
            }
            bool last = true;
            if (splits > 1 && counters == nullptr) {
                last = false;          // the pieces are summed by a kernel of their own (splitk_sum_kernel)
            } else if (splits > 1) {
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
                    const int old = atomicAdd(&counters[tile], 1);
                    sm.is_last = (old == splits - 1) ? 1 : 0;
                    if (old == splits - 1) counters[tile] = 0;      // ready for the next product
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                last = sm.is_last != 0;
                __threadfence();
            } else {
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (last && !*abort_flag) {
                // Pieces are summed in the order of the splits. Eight outputs are carried at
                // a time so that eight loads are in flight for every add that has to wait.
                const size_t slice = (size_t)M * (size_t)N;
                const int q_end = min(Q, q0 + BN);
                if constexpr (SWAP) {
                    // this thread owns weight row p (an output column) for the tile's tokens
                    const bool gate = EPI == 1;
                    const int pu = p + 64;
                    const bool active = gate ? (pl < 64 && pu < P) : (p < P);
                    if (active) {
                        for (int q = q0; q < q_end; q += 8) {
                            float g[8], u[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) g[j] = u[j] = 0.f;
#pragma unroll 2
                            for (int sp = 0; sp < splits; ++sp) {
                                const float* src = ws + (size_t)sp * slice + (size_t)q * N;
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (q + j < q_end) {
                                        g[j] += src[(size_t)j * N + p];
                                        if (gate) u[j] += src[(size_t)j * N + pu];
                                    }
                                }
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                if (q + j < q_end) {
                                    if (gate) C[(size_t)(q + j) * ldc + (p0 / 2 + pl)] = from_float<TO>(silu_mul(g[j], u[j]));
                                    else C[(size_t)(q + j) * ldc + p] = from_float<TO>(g[j]);
                                }
                            }
                        }
                    }
                } else if (p < P) {
                    // this thread owns token row p for the tile's columns
                    if constexpr (EPI == 0) {
                        for (int q = q0; q < q_end; q += 8) {
                            float acc[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 2
                            for (int sp = 0; sp < splits; ++sp) {
                                const float* src = ws + (size_t)sp * slice + (size_t)p * N + q;
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    if (q + j < q_end) acc[j] += src[j];
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (q + j < q_end) C[(size_t)p * ldc + q + j] = from_float<TO>(acc[j]);
                        }
                    } else {
                        for (int q = q0; q + 64 < q_end; q += 128)
                            for (int i = 0; i < 64 && q + 64 + i < q_end; i += 8) {
                                float g[8], u[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) g[j] = u[j] = 0.f;
#pragma unroll 2
                                for (int sp = 0; sp < splits; ++sp) {
                                    const float* src = ws + (size_t)sp * slice + (size_t)p * N + q + i;
#pragma unroll
                                    for (int j = 0; j < 8; ++j)
                                        if (q + 64 + i + j < q_end) { g[j] += src[j]; u[j] += src[64 + j]; }
                                }
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    if (q + 64 + i + j < q_end) C[(size_t)p * ldc + (q / 2 + i + j)] = from_float<TO>(silu_mul(g[j], u[j]));
                            }
                    }
                }
            }
        }
    }
    if constexpr (CLUSTER) {
        if (warp < 2) cluster_wait();           // the producer's and the issuer's half of the barrier the epilogue warps passed above
        cluster_sync_all();                     // every piece is in its owner's shared memory
        if (warp >= 2 && !*abort_flag) {
            const int pl = (warp & 3) * 32 + lane, p = p0 + pl;
            const uint32_t rank = cluster_rank();
            const int q_end = min(Q, q0 + BN);
            const int slots = (BN + splits - 1) / splits;
            const size_t plane = (size_t)slots * BM;                // floats between two senders' pieces of a token
            if constexpr (EPI == 3) {
                // Tokens rank, rank + splits, ... of the tile are this CTA's, one at a time; warps 0 and 1 of the
                // epilogue hold the tile's first head (values 0..31 and 32..63), warps 2 and 3 its second.
                const int wl = warp & 3, i = pl & 63, half = wl & 1;
                const int hh = p0 / 64 + (pl >> 6);
                const int kind = hh < rope.nh ? 0 : (hh < rope.nh + rope.nkv ? 1 : (hh < rope.nh + 2 * rope.nkv ? 2 : 3));
                for (int ql = (int)rank, k = 0; q0 + ql < q_end; ql += splits, ++k) {
                    const int q = q0 + ql;
                    const float* mine = &sm.red[k * BM + pl];
                    float x = 0.f;
#pragma unroll
                    for (int r = 0; r < 8; ++r) x += r < splits ? mine[r * plane] : 0.f;
                    x = __bfloat162float(__float2bfloat16_rn(x));     // as the plain product stores it
                    // the rotation of this thread's pair, meanwhile: angle = pos * (hi + lo) in split arithmetic
                    const int pos = sm.rope_pos[ql];
                    const float fp = (float)pos, a = fp * rp_hi, e = fmaf(fp, rp_hi, -a) + fp * rp_lo;
                    float sa, ca, se, ce;
                    sincosf(a, &sa, &ca);
                    sincosf(e, &se, &ce);
                    const float cs = ca * ce - sa * se, sn = sa * ce + ca * se;
                    const float part = warp_sum(x * x);
                    if (lane == 0) sm.ex_ss[wl] = part;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const float ss = sm.ex_ss[wl & 2] + sm.ex_ss[(wl & 2) + 1];
                    const float inv = 1.0f / sqrtf(ss / 64.0f + rope.eps);
                    const float y = x * inv * rp_w;
                    sm.ex_y[pl] = y;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const float other = sm.ex_y[pl ^ 32];
                    // values i < 32 are the first of their pair, values i >= 32 the second
                    const float turned = half == 0 ? y * cs - other * sn : y * cs + other * sn;
                    if (kind == 0) {
                        C[(size_t)q * ldc + (size_t)hh * 64 + i] = from_float<TO>(turned);
                    } else if (kind < 3) {
                        const int page = sm.rope_page[ql];
                        if (page < 0 || page >= rope.num_pages) {
                            if (i == 0) atomicOr(err, CELLM_DEV_BAD_PAGE);
                        } else {
                            const int kvh = kind == 1 ? hh - rope.nh : hh - rope.nh - rope.nkv;
                            const size_t at = ((size_t)page * rope.nkv + kvh) * rope.page_size * 64 +
                                              (size_t)(pos % rope.page_size) * 64 + i;
                            if (kind == 1) rope.k_pool[at] = __float2bfloat16_rn(turned);
                            else rope.v_pool[at] = __float2bfloat16_rn(x);
                        }
                    }
                }
            }
            if constexpr (EPI == 2) {
                // Tokens rank, rank + splits, ... of the tile are this CTA's; three of them are worked on side by
                // side (threads 0..41, 42..83, 84..125: one channel each). The history of the token after this
                // one is asked for before this one's sums are, so that the two round trips overlap.
                const int sub = pl / CONV_CH, cl = pl % CONV_CH, ch = (p0 / BM) * CONV_CH + cl;
                const int rows = conv.ntaps - 1;
                if (cv_active) {
                    for (int ql = (int)rank + sub * splits, own = sub; q0 + ql < q_end; ql += 3 * splits, own += 3) {     // own: the token's slot among this CTA's
                        const int q = q0 + ql, slot = sm.conv_slots[ql];
                        float hist[CONV_MAX_TAPS - 1];
#pragma unroll
                        for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) hist[k] = cv_hist[k];
                        const int qn = ql + 3 * splits;
                        if (q0 + qn < q_end) {
                            const int sn = sm.conv_slots[qn];
#pragma unroll
                            for (int k = 0; k < CONV_MAX_TAPS - 1; ++k)
                                cv_hist[k] = (k < rows && sn >= 0 && sn < conv.n_slots)
                                                 ? conv.state[(long long)sn * conv.slot_stride + (size_t)k * conv.H + ch] : 0.f;
                        }
                        if (slot < 0 || slot >= conv.n_slots) { atomicOr(err, CELLM_DEV_BAD_SLOT); continue; }
                        const float* mine = &sm.red[own * BM + cl];
                        float b = 0.f, c = 0.f, x = 0.f;
#pragma unroll
                        for (int r = 0; r < 8; ++r)
                            if (r < splits) { b += mine[r * plane]; c += mine[r * plane + CONV_CH]; x += mine[r * plane + 2 * CONV_CH]; }
                        // the plain product stores B, C and x as bfloat16 before the convolution reads them
                        b = __bfloat162float(__float2bfloat16_rn(b));
                        c = __bfloat162float(__float2bfloat16_rn(c));
                        x = __bfloat162float(__float2bfloat16_rn(x));
                        const float bx = b * x;
                        float acc = 0.f;
#pragma unroll
                        for (int k = 0; k < CONV_MAX_TAPS - 1; ++k)
                            if (k < rows) acc += hist[k] * cv_wt[k];
                        acc += bx * cv_wlast;
                        if (conv.bias) acc += cv_bias;
                        C[(size_t)q * ldc + ch] = from_float<TO>(c * acc);
                        float* st = conv.state + (long long)slot * conv.slot_stride;
#pragma unroll
                        for (int k = 0; k < CONV_MAX_TAPS - 2; ++k)
                            if (k + 1 < rows) st[(size_t)k * conv.H + ch] = hist[k + 1];
                        if (rows > 0) st[(size_t)(rows - 1) * conv.H + ch] = bx;
                    }
                }
            }
            // Tokens rank, rank + splits, ... of the tile are summed and written by this CTA.
            if constexpr (EPI == 0) {
                for (int q = q0 + (int)rank, k = 0; q < q_end; q += splits, ++k) {
                    const float* mine = &sm.red[k * BM + pl];
                    float acc = 0.f;
#pragma unroll
                    for (int r = 0; r < 8; ++r) acc += r < splits ? mine[r * plane] : 0.f;
                    if (p < P) C[(size_t)q * ldc + p] = from_float<TO>(acc);
                }
            }
            if constexpr (EPI == 1) {
                // an output is silu(gate) * up of rows i and i + 64 of the tile: the lower 64 threads take this
                // CTA's even tokens, the upper 64 its odd ones
                const int row = pl & 63, half = pl >> 6;
                for (int q = q0 + (int)rank + half * splits, k = half; q < q_end; q += 2 * splits, k += 2) {
                    const float* mine = &sm.red[k * BM + row];
                    float g = 0.f, u = 0.f;
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        if (r < splits) { g += mine[r * plane]; u += mine[r * plane + 64]; }
                    if (p0 + row + 64 < P) C[(size_t)q * ldc + (p0 / 2 + row)] = from_float<TO>(silu_mul(g, u));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// Sum of the K-split pieces of a product with plain tiles, ws[split][M][N], in the order of the splits; one
// thread for four neighbouring outputs. EPI as in the product's kernel (1: gate and up blocks of 64 columns).
template <int EPI, typename TO>
__global__ void splitk_sum_kernel(const float* __restrict__ ws, TO* __restrict__ C, int M, int N, long long ldc, int splits) {
    pdl_trigger();
    pdl_wait();
    const int NO = EPI == 1 ? N / 2 : N;                       // output columns
    const long long groups = (long long)M * ((NO + 3) / 4);
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const int m = (int)(g / ((NO + 3) / 4)), o0 = (int)(g % ((NO + 3) / 4)) * 4;
    const size_t slice = (size_t)M * (size_t)N;
    float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
    // input column of output column o: itself, or the gate of block o / 64 (its up lies 64 further on)
    const int c0 = EPI == 1 ? (o0 / 64) * 128 + (o0 % 64) : o0;
    const bool vec = (N & 3) == 0 && o0 + 3 < NO;              // four columns never straddle a block of 64
    for (int sp = 0; sp < splits; ++sp) {
        const float* src = ws + (size_t)sp * slice + (size_t)m * N + c0;
        if (vec) {
            const float4 v = *reinterpret_cast<const float4*>(src);
            a[0] += v.x; a[1] += v.y; a[2] += v.z; a[3] += v.w;
            if (EPI == 1) {
                const float4 u = *reinterpret_cast<const float4*>(src + 64);
                b[0] += u.x; b[1] += u.y; b[2] += u.z; b[3] += u.w;
            }
        } else {
            for (int j = 0; j < 4 && o0 + j < NO; ++j) {
                a[j] += src[j];
                if (EPI == 1) b[j] += src[64 + j];
            }
        }
    }
    for (int j = 0; j < 4 && o0 + j < NO; ++j)
        C[(size_t)m * ldc + o0 + j] = from_float<TO>(EPI == 1 ? silu_mul(a[j], b[j]) : a[j]);
}

// Sixteen values of a row (the last chunk of a tile whose width is an odd multiple of 16).
template <typename TO> __device__ __forceinline__ void store_half_row(TO* dst, const uint32_t* r, int valid, bool aligned);
template <> __device__ __forceinline__ void store_half_row<float>(float* dst, const uint32_t* r, int valid, bool aligned) {
    if (valid >= 16 && aligned) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (i < valid) dst[i] = __uint_as_float(r[i]);
    }
}
template <> __device__ __forceinline__ void store_half_row<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t* r, int valid, bool aligned) {
    if (valid >= 16 && aligned) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * j]), __uint_as_float(r[8 * i + 2 * j + 1]));
                p[j] = *reinterpret_cast<uint32_t*>(&v);
            }
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(p[0], p[1], p[2], p[3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (i < valid) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
    }
}

// Persistent form for large products (plain tiles, no K split): one CTA per SM walks
// the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (row tiles of A fastest, so
// CTAs that run side by side share a tile of W in L2). The accumulator is double
// buffered in tensor memory (2 x BN columns): while the epilogue warps drain one
// buffer and store it, the MMA warp already fills the other, and the TMA warp keeps
// the stage ring full across tile borders.
template <int BN, int STAGES, int EPI, typename TO>
__global__ void __launch_bounds__(192)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                               TO* __restrict__ C, int M, int N, int K, long long ldc, int w_is_static,
                               int* __restrict__ err, int bn) {
    // bn: the width of a tile in columns, a multiple of 16 (of 128 with the SwiGLU epilogue) and at most BN, which
    // sizes the stages and the accumulators. Widths between the powers of two let the number of tiles come close
    // to a multiple of the SMs, so that the last wave is not half empty.
    extern __shared__ uint8_t smem_raw[];
    auto& sm = *reinterpret_cast<GemmSmem<BN, STAGES>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t TMEM_COLS = 2 * BN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + bn - 1) / bn, num_tiles = m_tiles * n_tiles;
    const int nkb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.acc_full2[b], 1); mbar_init(&sm.acc_empty2[b], 128); }
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    if (warp == 1) tmem_alloc(&sm.tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_trigger();
    const uint32_t tmem = sm.tmem_base;
    volatile int* abort_flag = &sm.abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool waited = false;
            if (!w_is_static) { pdl_wait(); waited = true; }
            for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
                const int p0 = (tile % m_tiles) * BM, q0 = (tile / m_tiles) * bn;
                int kb = 0;
                if (!waited) {
                    // static weights: the ring's first loads of W go out before the wait on the preceding kernel
                    const int early = nkb < STAGES ? nkb : STAGES;
                    for (int i = 0; i < early; ++i) {
                        mbar_expect_tx(&sm.full[i], (uint32_t)((BM + bn) * BK * 2));
                        tma_load_2d(sm.b[i], &map_w, i * BK, q0, &sm.full[i]);
                    }
                    pdl_wait();
                    waited = true;
                    for (int i = 0; i < early; ++i) tma_load_2d(sm.a[i], &map_a, i * BK, p0, &sm.full[i]);
                    kb = early;
                    it = early;
                }
                for (; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
                    if (!mbar_wait(&sm.empty[s], phase ^ 1u, abort_flag)) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); break; }
                    mbar_expect_tx(&sm.full[s], (uint32_t)((BM + bn) * BK * 2));
                    tma_load_2d(sm.a[s], &map_a, kb * BK, p0, &sm.full[s]);
                    tma_load_2d(sm.b[s], &map_w, kb * BK, q0, &sm.full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BM, bn);
            int it = 0, tcount = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
                const int buf = tcount & 1;
                const uint32_t acc_phase = (uint32_t)(tcount >> 1) & 1u;
                if (!mbar_wait(&sm.acc_empty2[buf], acc_phase ^ 1u, abort_flag)) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); break; }
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)(buf * BN);
                bool ok = true;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
                    if (!mbar_wait(&sm.full[s], phase, abort_flag)) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = umma_desc(smem_u32(sm.a[s])), db = umma_desc(smem_u32(sm.b[s]));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(acc, da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16), idesc,
                                  (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&sm.empty[s]);
                }
                if (!ok) break;
                umma_commit(&sm.acc_full2[buf]);
            }
        }
    } else {
        const int qtr = warp & 3;
        const int pl = qtr * 32 + lane;
        bool waited = false;
        int tcount = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
            const int buf = tcount & 1;
            const uint32_t acc_phase = (uint32_t)(tcount >> 1) & 1u;
            if (!mbar_wait(&sm.acc_full2[buf], acc_phase, abort_flag)) {
                if (lane == 0) { *abort_flag = 1; atomicOr(err, CELLM_DEV_WAIT_TIMEOUT); }
                break;
            }
            tc_fence_after();
            if (!waited) { pdl_wait(); waited = true; }    // stores must not pass the kernel before this one
            const int p0 = (tile % m_tiles) * BM, q0 = (tile / m_tiles) * bn;
            const int p = p0 + pl;
            const uint32_t lane_addr = tmem + ((uint32_t)(qtr * 32) << 16) + (uint32_t)(buf * BN);
            if constexpr (EPI == 0) {
                const bool aligned = ((reinterpret_cast<uintptr_t>(C) | (uintptr_t)(ldc * sizeof(TO))) & 15) == 0 &&
                                     ((q0 * sizeof(TO)) & 15) == 0;
                const int chunks = (bn + 31) / 32;
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    uint32_t r[32];
                    const int cols = bn - c * 32 >= 32 ? 32 : 16;          // the last chunk of a width that is an odd multiple of 16
                    if (cols == 32) tmem_ld32(lane_addr + (uint32_t)(c * 32), r);
                    else tmem_ld16(lane_addr + (uint32_t)(c * 32), r);
                    if (c == chunks - 1) { tc_fence_before(); mbar_arrive(&sm.acc_empty2[buf]); }
                    const int q = q0 + c * 32;
                    if (p < M && q < N) {
                        if (cols == 32) store_row<TO>(C + (size_t)p * ldc + q, r, N - q, aligned);
                        else store_half_row<TO>(C + (size_t)p * ldc + q, r, N - q, aligned);
                    }
                }
            } else {
                const int o0 = q0 / 2;
                const bool aligned = ((reinterpret_cast<uintptr_t>(C) | (uintptr_t)(ldc * sizeof(TO))) & 15) == 0 &&
                                     ((o0 * sizeof(TO)) & 15) == 0;
#pragma unroll 1
                for (int j = 0; j < bn / 128; ++j) {
#pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        uint32_t g[32], u[32];
                        tmem_ld32(lane_addr + (uint32_t)(j * 128 + h * 32), g);
                        tmem_ld32(lane_addr + (uint32_t)(j * 128 + 64 + h * 32), u);
                        if (j == bn / 128 - 1 && h == 1) { tc_fence_before(); mbar_arrive(&sm.acc_empty2[buf]); }
#pragma unroll
                        for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(silu_mul(__uint_as_float(g[i]), __uint_as_float(u[i])));
                        const int o = o0 + j * 64 + h * 32;
                        if (p < M && o < N / 2) store_row<TO>(C + (size_t)p * ldc + o, g, N / 2 - o, aligned);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---------------------------------------------------------------- host side
template <int BN, int STAGES, bool SWAP, int EPI, bool CLUSTER, typename TO>
int launch(const CUtensorMap& m_rows, const CUtensorMap& m_cols, TO* C, float* ws, int* counters, int M, int N, int K,
           long long ldc, int split_k, int kblocks_per_split, int w_is_static, int* err, cudaStream_t stream,
           const ConvEpi& conv, const RopeEpi& rope) {
    const size_t smem = sizeof(GemmSmem<BN, STAGES, CLUSTER ? (BN + 8) * BM : 0>) + 1024;
    static bool configured = false;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, SWAP, EPI, CLUSTER, TO>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid = SWAP ? dim3((unsigned)((N + BM - 1) / BM), (unsigned)((M + BN - 1) / BN), (unsigned)split_k)
                     : dim3((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), (unsigned)split_k);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (CLUSTER) {      // the K split of a tile is one cluster along z
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 1;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = (unsigned)split_k;
        cfg.numAttrs = 2;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, m_rows, m_cols, C, ws, counters, M, N, K, ldc, kblocks_per_split,
                                       w_is_static, err, conv, rope);
    return e == cudaSuccess ? CELLM_OK : (int)e;
}

template <int BN, int STAGES, int EPI, typename TO>
int launch_persistent(const CUtensorMap& m_a, const CUtensorMap& m_w, TO* C, int M, int N, int K, long long ldc,
                      int w_is_static, int* err, cudaStream_t stream, int bn) {
    const size_t smem = sizeof(GemmSmem<BN, STAGES>) + 1024;
    static int sms = 0;
    if (sms == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<BN, STAGES, EPI, TO>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return CELLM_ERR_ARG;
    }
    const int tiles = ((N + bn - 1) / bn) * ((M + BM - 1) / BM);
    dim3 grid((unsigned)(tiles < sms ? tiles : sms));
    cudaError_t e = cellm_launch(gemm_tcgen05_persistent_kernel<BN, STAGES, EPI, TO>, grid, dim3(192), smem, stream, m_a,
                                 m_w, C, M, N, K, ldc, w_is_static, err, bn);
    return e == cudaSuccess ? CELLM_OK : (int)e;
}

}  // namespace

// Most tiles a product may have when K is split (one counter each).
#define GEMM_MAX_COUNTERS 65536

// How a call with these sizes uses scratch memory: *ws_floats of float workspace
// (0: none) and whether the tile counters are needed. epilogue: 0 plain, 1 SwiGLU.
CELLM_API int cellm_gemm_tcgen05_plan(int M, int N, int K, int bn, int split_k, int epilogue, long long* ws_floats,
                                      int* effective_split) {
    const int kblocks = (K + BK - 1) / BK;
    if (split_k < 1) split_k = 1;
    if (split_k > kblocks) split_k = kblocks;
    const int per = (kblocks + split_k - 1) / split_k;
    split_k = (kblocks + per - 1) / per;        // no empty slice
    *effective_split = split_k;
    const bool through_ws = split_k > 1 || (epilogue == 1 && bn < 0);
    *ws_floats = through_ws ? (long long)split_k * M * N : 0;
    return CELLM_OK;
}

// A: [M, K] bf16 (row pitch lda elements), W: [N, K] bf16 (pitch ldw). epilogue 0:
// C: [M, N] of out_dtype (pitch ldc). epilogue 1 (SwiGLU): W is laid out in blocks
// of 64 gate rows followed by their 64 up rows (N a multiple of 128) and C is
// [M, N/2]. bn > 0: plain tiles of 128 rows of A by bn (64, 128, 256) rows of W;
// bn < 0: swapped tiles of 128 rows of W by -bn (16, 32, 64) rows of A.
// w_is_static: W is a weight that no kernel on the stream writes, so its loads may
// start before the preceding kernel has finished (a value n > 1 also asks up to n
// further K blocks of the CTA's weights into L2 while it waits).
// workspace: as many floats as cellm_gemm_tcgen05_plan says; counters: GEMM_MAX_COUNTERS
// zeroed ints that products on one stream may share (each product leaves them zero).
static int gemm_impl(void* C, const void* A, const void* W, int M, int N, int K, long long lda,
                     long long ldw, long long ldc, int out_dtype, int bn, int split_k, int epilogue,
                     int w_is_static, float* workspace, int* counters, int* err, cudaStream_t stream,
                     const ConvEpi& conv, const RopeEpi& rope) {
    if (M <= 0 || N <= 0) return CELLM_OK;
    if (K <= 0 || (K & 7)) return CELLM_ERR_SIZE;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((lda * 2) & 15) || ((ldw * 2) & 15)) return CELLM_ERR_ALIGN;
    if (out_dtype != CELLM_F32 && out_dtype != CELLM_BF16) return CELLM_ERR_DTYPE;
    if (epilogue < 0 || epilogue > 3) return CELLM_ERR_ARG;
    const bool swap = bn < 0;
    const int narrow = swap ? -bn : bn;
    // plain tiles: 64, 128 or 256 columns; unsplit products (the persistent kernel) also any multiple of 16 from 128 to 256
    const bool odd_width = !swap && narrow > 128 && narrow < 256 && (narrow & 15) == 0 && epilogue == 0;
    if (swap ? (narrow != 16 && narrow != 32 && narrow != 64) : (narrow != 64 && narrow != 128 && narrow != 256 && !odd_width))
        return CELLM_ERR_SIZE;
    if (epilogue == 1 && ((N & 127) || (!swap && narrow < 128))) return CELLM_ERR_SIZE;
    long long ws_floats;
    int split;
    cellm_gemm_tcgen05_plan(M, N, K, bn, split_k, epilogue, &ws_floats, &split);
    // swapped tiles whose K split fits a cluster (2..8 CTAs) sum their pieces through shared memory
    // (an unsplit SwiGLU tile takes the same road as a cluster of one: gate and up meet in shared memory)
    const bool in_cluster = swap && ((split >= 2 && split <= 8) || (split == 1 && epilogue >= 1));
    if (in_cluster) ws_floats = 0;
    if (epilogue >= 2 && !in_cluster) return CELLM_ERR_ARG;      // the convolution and rotation epilogues exist for clustered swapped tiles only
    const int kblocks = (K + BK - 1) / BK;
    const int per = (kblocks + split - 1) / split;
    if (ws_floats > 0 && workspace == nullptr) return CELLM_ERR_ARG;
    // Plain tiles without counters: the pieces go to the workspace and a second kernel sums them, all SMs at work
    // (with counters the last CTA of a tile sums its pieces alone, which is slow for tiles of 128 tokens).
    if (odd_width && split > 1) return CELLM_ERR_SIZE;
    const bool sum_later = split > 1 && !in_cluster && !swap && counters == nullptr;
    if (split > 1 && !in_cluster && !sum_later) {
        if (counters == nullptr) return CELLM_ERR_ARG;
        const long long tiles = swap ? (long long)((N + BM - 1) / BM) * ((M + narrow - 1) / narrow)
                                     : (long long)((N + narrow - 1) / narrow) * ((M + BM - 1) / BM);
        if (tiles > GEMM_MAX_COUNTERS) return CELLM_ERR_SIZE;
    }
    CUtensorMap map_a, map_w;
    if (!tensor_map(&map_a, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, swap ? (uint32_t)narrow : (uint32_t)BM)) return CELLM_ERR_ARG;
    if (!tensor_map(&map_w, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw * 2, swap ? (uint32_t)BM : (uint32_t)narrow)) return CELLM_ERR_ARG;
    const CUtensorMap& m_rows = swap ? map_w : map_a;
    const CUtensorMap& m_cols = swap ? map_a : map_w;
    int rc = CELLM_ERR_SIZE;
    // Large unsplit products with plain tiles of 128 or 256 columns run the persistent kernel.
    if (!swap && split == 1 && narrow >= 128) {
#define GOP(BN_, ST_, EP_)                                                                                          \
    do {                                                                                                            \
        if (out_dtype == CELLM_F32) rc = launch_persistent<BN_, ST_, EP_, float>(map_a, map_w, (float*)C, M, N, K, ldc, w_is_static, err, stream, narrow); \
        else rc = launch_persistent<BN_, ST_, EP_, __nv_bfloat16>(map_a, map_w, (__nv_bfloat16*)C, M, N, K, ldc, w_is_static, err, stream, narrow); \
    } while (0)
        if (narrow == 128) { if (epilogue == 0) GOP(128, 6, 0); else GOP(128, 6, 1); }
        else { if (epilogue == 0) GOP(256, 4, 0); else GOP(256, 4, 1); }       // 144 to 256 columns
#undef GOP
        return rc;
    }
#define GO3(BN_, ST_, SW_, EP_, CL_)                                                                                  \
    do {                                                                                                              \
        if (out_dtype == CELLM_F32) rc = launch<BN_, ST_, SW_, EP_, CL_, float>(m_rows, m_cols, (float*)C, workspace, counters, M, N, K, ldc, split, per, w_is_static, err, stream, conv, rope); \
        else rc = launch<BN_, ST_, SW_, EP_, CL_, __nv_bfloat16>(m_rows, m_cols, (__nv_bfloat16*)C, workspace, counters, M, N, K, ldc, split, per, w_is_static, err, stream, conv, rope); \
    } while (0)
#define GO2(BN_, ST_, SW_, EP_) GO3(BN_, ST_, SW_, EP_, false)
    // swapped: ST_ stages without, CST_ stages with the cluster's reduction buffer (two CTAs must still fit an SM); the
    // SwiGLU product, which has two CTAs an SM, takes three, so that a CTA of the product after it fits beside them
#define GOS(BN_, ST_, CST_)                                                                                           \
    do {                                                                                                              \
        if (in_cluster) { if (epilogue == 0) GO3(BN_, CST_, true, 0, true); else if (epilogue == 1) GO3(BN_, (CST_ > 3 ? 3 : CST_), true, 1, true); else if (epilogue == 2) GO3(BN_, CST_, true, 2, true); else GO3(BN_, CST_, true, 3, true); } \
        else { if (epilogue == 0) GO3(BN_, ST_, true, 0, false); else GO3(BN_, ST_, true, 1, false); }                 \
    } while (0)
#define GO(BN_, ST_, SW_)                           \
    do {                                            \
        if (epilogue == 0) GO2(BN_, ST_, SW_, 0);   \
        else GO2(BN_, ST_, SW_, 1);                 \
    } while (0)
    if (swap) {
        if (narrow == 16) GOS(16, 5, 4);
        else if (narrow == 32) GOS(32, 5, 4);
        else GOS(64, 4, 3);
    } else {
        if (narrow == 64) GO2(64, 8, false, 0);
        else if (narrow == 128) GO(128, 6, false);
        else GO(256, 4, false);
    }
#undef GO
#undef GO2
#undef GO3
#undef GOS
    if (rc == CELLM_OK && sum_later) {
        const int NO = epilogue == 1 ? N / 2 : N;
        const long long groups = (long long)M * ((NO + 3) / 4);
        const unsigned blocks = (unsigned)((groups + 255) / 256);
        if (epilogue == 0 && out_dtype == CELLM_F32) CELLM_RUN((splitk_sum_kernel<0, float>), blocks, 256, 0, stream, workspace, (float*)C, M, N, ldc, split);
        else if (epilogue == 0) CELLM_RUN((splitk_sum_kernel<0, __nv_bfloat16>), blocks, 256, 0, stream, workspace, (__nv_bfloat16*)C, M, N, ldc, split);
        else if (out_dtype == CELLM_F32) CELLM_RUN((splitk_sum_kernel<1, float>), blocks, 256, 0, stream, workspace, (float*)C, M, N, ldc, split);
        else CELLM_RUN((splitk_sum_kernel<1, __nv_bfloat16>), blocks, 256, 0, stream, workspace, (__nv_bfloat16*)C, M, N, ldc, split);
    }
    return rc;
}

// The product described above gemm_impl.
CELLM_API int cellm_gemm_tcgen05(void* C, const void* A, const void* W, int M, int N, int K, long long lda,
                                 long long ldw, long long ldc, int out_dtype, int bn, int split_k, int epilogue,
                                 int w_is_static, float* workspace, int* counters, int* err, cudaStream_t stream) {
    if (epilogue >= 2) return CELLM_ERR_ARG;     // those epilogues have entry points of their own
    const ConvEpi none{};
    const RopeEpi none3{};
    return gemm_impl(C, A, W, M, N, K, lda, ldw, ldc, out_dtype, bn, split_k, epilogue, w_is_static, workspace, counters,
                     err, stream, none, none3);
}

// in_proj and the gated short convolution of a decode step in one kernel (the kernel's EPI = 2).
// A: [M, K] bf16, one token of M different requests. Wt: in_proj in tiles of 128 rows, [Nt, K] with
// Nt = 128 * ceil(H / 42): rows 0..41 of tile j are the B rows of channels 42j..42j+41, rows 42..83
// their C rows, rows 84..125 their x rows; rows of channels beyond H and the last two rows are zero.
// Y: [M, H] bf16. taps: [H, ntaps] bf16 (1 to 4 taps), bias: [H] bf16 or null; state: [n_slots][ntaps-1][H]
// floats, slot_stride floats apart, read and moved on by one token; slot_ids: [M]. bn: -16, -32 or -64;
// the K split must leave the tile's CTAs in one cluster (at most 8), else the call is refused (-4).
CELLM_API int cellm_gemm_conv_tcgen05(void* Y, const void* A, const void* Wt, int M, int Nt, int K, long long lda,
                                      long long ldw, int H, int bn, int split_k, const void* taps, const void* bias,
                                      int ntaps, float* state, long long slot_stride, const int* slot_ids, int n_slots,
                                      int w_is_static, int* err, cudaStream_t stream) {
    if (M <= 0) return CELLM_OK;
    if (bn >= 0 || H <= 0 || (Nt & 127) || (long long)(Nt / 128) * CONV_CH < H) return CELLM_ERR_SIZE;
    if (ntaps < 1 || ntaps > CONV_MAX_TAPS) return CELLM_ERR_SIZE;
    if (!taps || !slot_ids || (ntaps > 1 && !state) || n_slots <= 0) return CELLM_ERR_ARG;
    ConvEpi conv{};
    conv.taps = (const __nv_bfloat16*)taps;
    conv.bias = (const __nv_bfloat16*)bias;
    conv.state = state;
    conv.slot_ids = slot_ids;
    conv.slot_stride = slot_stride;
    conv.H = H;
    conv.ntaps = ntaps;
    conv.n_slots = n_slots;
    const RopeEpi none3{};
    return gemm_impl(Y, A, Wt, M, Nt, K, lda, ldw, (long long)H, CELLM_BF16, bn, split_k, 2, w_is_static, nullptr, nullptr,
                     err, stream, conv, none3);
}

// The q/k/v product of a decode step with the heads' RMSNorm, the rotation and the write into the paged cache in
// its epilogue (the kernel's EPI = 3). A: [M, K] bf16, one token of M different requests. W: q_proj | k_proj | v_proj,
// [(nh + 2 nkv) * 64, K] bf16 (heads of 64, turned whole in pairs (i, i + 32)). Q: [M, nh * 64] bf16. q_w, k_w: [64]
// bf16; positions: [M]; block_table: [M][bt_stride]; pools: [pages][nkv][page_size][64] bf16; inv_freq: [32][2]
// floats (frequency and remainder). bn: -16, -32 or -64; the K split must leave the tile's CTAs in one cluster.
CELLM_API int cellm_gemm_rope_tcgen05(void* Q, const void* A, const void* W, int M, int K, long long lda, long long ldw,
                                      int bn, int split_k, const void* q_w, const void* k_w, float eps,
                                      const int* positions, const int* block_table, int bt_stride, void* k_pool,
                                      void* v_pool, int num_pages, int page_size, int nh, int nkv,
                                      const float* inv_freq, int w_is_static, int* err, cudaStream_t stream) {
    if (M <= 0) return CELLM_OK;
    if (bn >= 0 || nh <= 0 || nkv <= 0 || page_size <= 0 || num_pages <= 0 || bt_stride <= 0) return CELLM_ERR_SIZE;
    if (!q_w || !k_w || !positions || !block_table || !k_pool || !v_pool || !inv_freq) return CELLM_ERR_ARG;
    RopeEpi rope{};
    rope.q_w = (const __nv_bfloat16*)q_w;
    rope.k_w = (const __nv_bfloat16*)k_w;
    rope.positions = positions;
    rope.block_table = block_table;
    rope.k_pool = (__nv_bfloat16*)k_pool;
    rope.v_pool = (__nv_bfloat16*)v_pool;
    rope.inv_freq = inv_freq;
    rope.eps = eps;
    rope.bt_stride = bt_stride;
    rope.num_pages = num_pages;
    rope.page_size = page_size;
    rope.nh = nh;
    rope.nkv = nkv;
    const ConvEpi none{};
    return gemm_impl(Q, A, W, M, (nh + 2 * nkv) * 64, K, lda, ldw, (long long)nh * 64, CELLM_BF16, bn, split_k, 3,
                     w_is_static, nullptr, nullptr, err, stream, none, rope);
}
