// Attention for decoded tokens over the paged cache (bfloat16, tensor cores).
//
// One CTA serves one (request, key/value head, piece of the keys). The query
// heads that share the key/value head are the rows of one 16-row tile (at most
// 16 / group-size tokens per request, so a request's portion must be that
// short). The CTA walks its keys in blocks of 64 that all its threads bring in
// with cp.async (a ring of ST stages); within a block every warp takes its own run of
// 64 / NW keys and keeps an online-softmax state of its own, so the work of a
// block is spread over the warps and a CTA needs only one ring of shared memory
// (several CTAs fit an SM). The warps' partial results (maximum, sum,
// unnormalised output) are combined through shared memory at the end.
//
// When the keys of a request are split over several CTAs (gridDim.z > 1) and these are at most eight, they form
// one thread-block cluster: every CTA owns a share of the outputs, the others store their pieces (maximum, sum,
// unnormalised output) of that share into its shared memory, and after a cluster barrier it combines them in the
// order of the splits. A multiple of eight pieces forms clusters of eight that do the same, and each cluster
// leaves one piece in the workspace; other counts leave a piece per CTA there. A CTA that has left its piece adds one
// to the counter of its (request, key/value head); the one that finds the counter at gridDim.z - 1 combines the
// workspace's pieces in their order, writes the output and sets the counter back to zero. Either way no second
// kernel runs.
#include <algorithm>
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

template <int HD, int NW, bool CL>
struct DecodeSmem {
    static constexpr int KV_BYTES = FA_BN * HD * 2;
    static constexpr int ST = HD <= 64 ? 3 : 2;                           // stages of the ring
    static constexpr size_t q_off = 0;                                    // [16][HD] bfloat16, until the fragments are in registers
    static constexpr size_t kv_off = 16 * HD * 2;                         // [ST stages][K | V]
    static constexpr size_t o_off = kv_off;                               // [NW][16][HD] float, over the ring once the keys are done
    static constexpr size_t ml_off = o_off + (size_t)NW * 16 * HD * 4;    // [NW][16][2] float, over the ring as well
    static constexpr size_t flag_off = kv_off + (size_t)ST * 2 * KV_BYTES;
    // What a CTA receives from its cluster (CL). Of the outputs it owns (runs of 32 elements of the 16 x HD tile, dealt
    // out in turn) every sender's piece, [sender][owned element]; and every sender's maximum and sum of all 16 rows,
    // [8 senders][16][2] floats, where the queries lay: a CTA tells its cluster that it runs only after it has taken
    // its queries into registers, and nobody stores into a peer before all have told.
    static constexpr size_t co_off = flag_off + 16;
    static constexpr size_t cml_off = q_off;
    static constexpr size_t pages_off = co_off + (CL ? (size_t)(16 * HD + 7 * 32) * 4 : 0);   // [bt_stride] int: this CTA's slice of the block table
    static constexpr size_t fixed = pages_off;
    static_assert((size_t)NW * 16 * (HD + 2) * 4 <= (size_t)ST * 2 * KV_BYTES, "the warps' outputs must fit the ring");
    static_assert(!CL || 8 * 16 * 2 * 4 <= 16 * HD * 2, "the senders' maxima and sums must fit the queries' place");
};

// A float into the same place of the shared memory of CTA `rank` of this cluster.
__device__ __forceinline__ void st_peer(float* local, uint32_t rank, float v) {
    uint32_t addr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// CL: the CTAs of a split are clusters of cs = min(gridDim.z, 8) along z. Every CTA owns a share of the outputs; the
// others of its cluster store their pieces of that share straight into its shared memory, and after one cluster
// barrier it combines them out of its own memory. With several clusters the result is the cluster's piece in the
// workspace.
template <int HD, int NW, bool CL>
__global__ void __launch_bounds__(NW * 32)
attention_decode_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ counters, const __nv_bfloat16* __restrict__ q,
                        const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens,
                        const int* __restrict__ block_table, int bt_stride, int T, int num_pages, int page_size,
                        int nh, int nkv, float scale_log2e, int window, int* __restrict__ err) {
    constexpr int BN = FA_BN, CH = HD / 8, NT = HD / 8;
    using L = DecodeSmem<HD, NW, CL>;
    extern __shared__ __align__(128) uint8_t dec_smem[];
    uint8_t* q_s = dec_smem + L::q_off;
    float* o_s = reinterpret_cast<float*>(dec_smem + L::o_off);
    float* ml_s = reinterpret_cast<float*>(dec_smem + L::ml_off);
    int* flag_s = reinterpret_cast<int*>(dec_smem + L::flag_off);
    float* co_s = reinterpret_cast<float*>(dec_smem + L::co_off);
    float* cml_s = reinterpret_cast<float*>(dec_smem + L::cml_off);
    int* page_s = reinterpret_cast<int*>(dec_smem + L::pages_off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* kv_s = dec_smem + L::kv_off;
    constexpr int WK = FA_BN / NW;          // keys of a block that one warp takes (16 or 32)
    constexpr int THREADS = NW * 32;
    const int G = nh / nkv;
    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
    constexpr int ST = L::ST;
    pdl_trigger();
    const int t_base = cu_seqlens[b], q_len = cu_seqlens[b + 1] - t_base, rows = q_len * G;   // rows <= 16
    const int ctx = ctx_lens[b];
    // keys beyond what a row of the block table can name are reported and left out (the CTA's slice of the table in
    // shared memory is sized from the row)
    const int key_end = min(ctx + q_len, bt_stride * page_size);
    if (ctx + q_len > key_end && threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_PAGE);
    const int key_begin = window > 0 ? max(0, ctx - window + 1) : 0;
    const int kb_begin = key_begin / BN, kb_end = (key_end + BN - 1) / BN;
    const int cs = CL ? min(nsplit, 8) : 1;           // CTAs of a cluster, this CTA's rank in it, clusters
    const int crank = split % cs, n_clusters = nsplit / cs, cid = split / cs;
    const int per = (kb_end - kb_begin + nsplit - 1) / nsplit;
    const int my_begin = kb_begin + split * per, my_end = min(kb_end, my_begin + per);
    const int* bt = block_table + (size_t)b * bt_stride;
    const size_t page_elems = (size_t)nkv * page_size * HD;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;   // -1: not a power of two
    auto page_of = [&](int j) { return page_shift >= 0 ? (j >> page_shift) : (j / page_size); };
    auto slot_of = [&](int j) { return page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size); };

    // The block-table entries of this CTA's keys come into shared memory in one round trip, so that the copies of
    // a block do not each wait for a load of the table.
    const int p_lo = page_of(my_begin * BN), p_hi = my_begin < my_end ? page_of(min(key_end, my_end * BN) - 1) + 1 : p_lo;
    for (int i = threadIdx.x; i < p_hi - p_lo; i += THREADS) page_s[i] = bt[p_lo + i];
    __syncthreads();
    constexpr int KV_ITERS = (BN * CH + THREADS - 1) / THREADS;
    auto load_kv = [&](int kb, int stage) {
        uint8_t* ks = kv_s + (size_t)stage * 2 * L::KV_BYTES;
        uint8_t* vs = ks + L::KV_BYTES;
#pragma unroll
        for (int it = 0; it < KV_ITERS; ++it) {
            const int i = threadIdx.x + it * THREADS;
            if (i >= BN * CH) break;
            const int row = i / CH, chunk = i % CH, j = kb * BN + row;
            int page = (j >= key_begin && j < key_end) ? page_s[page_of(j) - p_lo] : -1;
            if (j >= key_begin && j < key_end && (page < 0 || page >= num_pages)) { atomicOr(err, CELLM_DEV_BAD_PAGE); page = -1; }
            const size_t off = page >= 0 ? (size_t)page * page_elems + ((size_t)kvh * page_size + slot_of(j)) * HD + chunk * 8 : 0;
            cp_async16(ks + tile_offset<HD>(row, chunk), k_pool + off, page >= 0 ? 16 : 0);
            cp_async16(vs + tile_offset<HD>(row, chunk), v_pool + off, page >= 0 ? 16 : 0);
        }
    };
    const int n_blk = max(0, my_end - my_begin);
    const int first = min(n_blk, ST);            // blocks that fill the ring before the walk starts
    const int old_end = ctx / BN;                // blocks below hold only keys that were in the cache before this step
    int issued = 0;
    for (; issued < first && my_begin + issued < old_end; ++issued) {
        load_kv(my_begin + issued, issued);
        cp_async_commit();
    }
    pdl_wait();                                  // the queries and this step's keys are the work of the kernels before
    for (int i = threadIdx.x; i < 16 * CH; i += NW * 32) {
        const int row = i / CH, chunk = i % CH;
        const bool ok = row < rows;
        const __nv_bfloat16* src = q + (size_t)(t_base + (ok ? row / G : 0)) * nh * HD + (size_t)(kvh * G + (ok ? row % G : 0)) * HD + chunk * 8;
        cp_async16(q_s + tile_offset<HD>(row, chunk), src, ok ? 16 : 0);
    }
    cp_async_commit();
    for (; issued < first; ++issued) {
        load_kv(my_begin + issued, issued);
        cp_async_commit();
    }
    cp_async_wait<0>();          // the Q tile and the first blocks (this thread's share)
    __syncthreads();             // everybody's share
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks], q_s + tile_offset<HD>(lane & 15, ks * 2 + (lane >> 4)));
    // this CTA runs and is done with its queries' place: its peers may store into its shared memory (the barrier's
    // other half comes before the first such store)
    if constexpr (CL) cluster_arrive();

    const int row_a = lane >> 2, row_b = row_a + 8;
    const int pos_a = row_a < rows ? ctx + row_a / G : -1, pos_b = row_b < rows ? ctx + row_b / G : -1;
    const int lo_a = window > 0 ? pos_a - window + 1 : 0, lo_b = window > 0 ? pos_b - window + 1 : 0;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    for (int kb = my_begin, it = 0; kb < my_end; ++kb, ++it) {
        const int stage = it % ST;
        // block `it` was committed ST groups ago (one group per block walked since)
        cp_async_wait<ST - 1>();
        __syncthreads();
        const uint8_t* ks_ = kv_s + (size_t)stage * 2 * L::KV_BYTES;
        const uint8_t* vs_ = ks_ + L::KV_BYTES;
        const int k0 = warp * WK;               // this warp's keys of the block: k0 .. k0 + WK - 1
        float s[WK / 8][4];
#pragma unroll
        for (int n = 0; n < WK / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < WK / 16; ++n2) {
                uint32_t kf[4];
                ldmatrix_x4(kf, ks_ + tile_offset<HD>(k0 + n2 * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * n2], qf[ks], kf[0], kf[1]);
                mma_bf16(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
            }
        }
        const int j0 = kb * BN + k0 + (lane & 3) * 2;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < WK / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j0 + n * 8 + e;
                const float va = (j <= pos_a && j >= lo_a) ? s[n][e] * scale_log2e : -INFINITY;
                const float vb = (j <= pos_b && j >= lo_b) ? s[n][2 + e] * scale_log2e : -INFINITY;
                s[n][e] = va;
                s[n][2 + e] = vb;
                mx_a = fmaxf(mx_a, va);
                mx_b = fmaxf(mx_b, vb);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float use_a = mn_a == -INFINITY ? 0.f : mn_a, use_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float corr_a = fast_exp2(m_a - use_a), corr_b = fast_exp2(m_b - use_b);
        m_a = mn_a;
        m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pf[WK / 16][4];
#pragma unroll
        for (int n = 0; n < WK / 8; ++n) {
            const float p0 = fast_exp2(s[n][0] - use_a), p1 = fast_exp2(s[n][1] - use_a);
            const float p2 = fast_exp2(s[n][2] - use_b), p3 = fast_exp2(s[n][3] - use_b);
            sum_a += p0 + p1;
            sum_b += p2 + p3;
            pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_a = l_a * corr_a + sum_a;
        l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int n = 0; n < NT; ++n) { o[n][0] *= corr_a; o[n][1] *= corr_a; o[n][2] *= corr_b; o[n][3] *= corr_b; }
#pragma unroll
        for (int kk = 0; kk < WK / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vs_ + tile_offset<HD>(k0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), n2 * 2 + (lane >> 4)));
                mma_bf16(o[2 * n2], pf[kk], vf[0], vf[1]);
                mma_bf16(o[2 * n2 + 1], pf[kk], vf[2], vf[3]);
            }
        }
        __syncthreads();
        if (kb + ST < my_end) load_kv(kb + ST, stage);       // the stage is free: the block ST further on moves in
        cp_async_commit();
    }
    cp_async_wait<0>();
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    // ---- the warps' results meet in shared memory
    {
        float* ow = o_s + (size_t)warp * 16 * HD;
        const int col = (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            *reinterpret_cast<float2*>(ow + row_a * HD + n * 8 + col) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2*>(ow + row_b * HD + n * 8 + col) = make_float2(o[n][2], o[n][3]);
        }
        if ((lane & 3) == 0) {
            ml_s[(warp * 16 + row_a) * 2] = m_a;
            ml_s[(warp * 16 + row_a) * 2 + 1] = l_a;
            ml_s[(warp * 16 + row_b) * 2] = m_b;
            ml_s[(warp * 16 + row_b) * 2 + 1] = l_b;
        }
    }
    __syncthreads();
    const size_t n_rows = (size_t)T * nh;
    // CL: runs of 32 elements are dealt out to the CTAs in turn; `chunks_mine` of them, 32 floats each, lie side by
    // side in a sender's plane of the owner's buffer
    const int chunks = (rows * HD + 31) / 32;
    const int plane = ((chunks + cs - 1) / cs) * 32;
    if constexpr (CL) { if (nsplit > 1) cluster_wait(); }          // every CTA of the cluster has started
    // element e = (row, dim) of the 16 x HD tile, owned by thread e mod (NW*32)
    for (int e = threadIdx.x; e < rows * HD; e += NW * 32) {
        const int row = e / HD, d = e % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) m = fmaxf(m, ml_s[(w * 16 + row) * 2]);
        const float use = m == -INFINITY ? 0.f : m;
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float f = exp2f(ml_s[(w * 16 + row) * 2] - use);
            l += f * ml_s[(w * 16 + row) * 2 + 1];
            acc += f * o_s[((size_t)w * 16 + row) * HD + d];
        }
        const size_t gr = (size_t)(t_base + row / G) * nh + kvh * G + row % G;
        if (nsplit == 1) {
            out[gr * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else if (CL) {
            const int chunk = e >> 5;
            st_peer(co_s + crank * plane + (chunk / cs) * 32 + (e & 31), (uint32_t)(chunk % cs), acc);
            if (d == 0)
                for (int to = 0; to < cs; ++to) {
                    st_peer(cml_s + (crank * 16 + row) * 2, (uint32_t)to, m);
                    st_peer(cml_s + (crank * 16 + row) * 2 + 1, (uint32_t)to, l);
                }
        } else {
            part_o[((size_t)split * n_rows + gr) * HD + d] = acc;
            if (d == 0) { part_ml[((size_t)split * n_rows + gr) * 2] = m; part_ml[((size_t)split * n_rows + gr) * 2 + 1] = l; }
        }
    }
    if (nsplit == 1) return;
    if constexpr (CL) {
        // ---- one barrier, then every CTA combines the outputs it owns, in the order of the splits
        cluster_arrive();
        cluster_wait();
        const int mine = (chunks - crank + cs - 1) / cs;          // runs of 32 that this CTA owns
        for (int idx = threadIdx.x; idx < mine * 32; idx += THREADS) {
            const int k = idx >> 5, i = idx & 31;
            const int e = (crank + k * cs) * 32 + i;
            if (e >= rows * HD) continue;
            const int row = e / HD, d = e % HD;
            const size_t gr = (size_t)(t_base + row / G) * nh + kvh * G + row % G;
            float m = -INFINITY;
            for (int sp = 0; sp < cs; ++sp) m = fmaxf(m, cml_s[(sp * 16 + row) * 2]);
            const float use = m == -INFINITY ? 0.f : m;
            float l = 0.f, acc = 0.f;
            for (int sp = 0; sp < cs; ++sp) {
                const float f = exp2f(cml_s[(sp * 16 + row) * 2] - use);
                l += f * cml_s[(sp * 16 + row) * 2 + 1];
                if (f != 0.f) acc += f * co_s[sp * plane + k * 32 + i];
            }
            if (n_clusters == 1) {
                out[gr * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
            } else {            // the cluster's piece
                part_o[((size_t)cid * n_rows + gr) * HD + d] = acc;
                if (d == 0) { part_ml[((size_t)cid * n_rows + gr) * 2] = m; part_ml[((size_t)cid * n_rows + gr) * 2 + 1] = l; }
            }
        }
        // nobody reads a peer's memory: a CTA may leave before the others of its cluster have finished
        if (n_clusters == 1) return;
    }

    // ---- the pieces of a split meet in the workspace; the last CTA combines them
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int idx = b * nkv + kvh;
        const int old = atomicAdd(&counters[idx], 1);
        *flag_s = (old == nsplit - 1) ? 1 : 0;
        if (old == nsplit - 1) counters[idx] = 0;
    }
    __syncthreads();
    if (*flag_s == 0) return;
    __threadfence();
    const int pieces = CL ? n_clusters : nsplit;
    for (int e = threadIdx.x; e < rows * HD; e += NW * 32) {
        const int row = e / HD, d = e % HD;
        const size_t gr = (size_t)(t_base + row / G) * nh + kvh * G + row % G;
        float m = -INFINITY;
        for (int sp = 0; sp < pieces; ++sp) m = fmaxf(m, part_ml[((size_t)sp * n_rows + gr) * 2]);
        const float use = m == -INFINITY ? 0.f : m;
        float l = 0.f, acc = 0.f;
        for (int sp = 0; sp < pieces; ++sp) {
            const float f = exp2f(part_ml[((size_t)sp * n_rows + gr) * 2] - use);
            l += f * part_ml[((size_t)sp * n_rows + gr) * 2 + 1];
            if (f != 0.f) acc += f * part_o[((size_t)sp * n_rows + gr) * HD + d];
        }
        out[gr * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
}

template <int HD, int NW>
int launch_decode(__nv_bfloat16* out, float* part_o, float* part_ml, int* counters, const __nv_bfloat16* q,
                  const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool, const int* cu, const int* ctx, const int* bt,
                  int bt_stride, int B, int T, int num_pages, int page_size, int nh, int nkv, float scale, int window,
                  int nsplit, int* err, cudaStream_t stream) {
    // the CTA's slice of a block-table row is at most the row
    const bool in_cluster = nsplit >= 2 && (nsplit <= 8 || nsplit % 8 == 0);     // clusters of nsplit, or of eight
    // A CTA keeps the block-table entries of its own keys: at most its share of the blocks a row of the table can
    // name (a page more at either end where a block's edge is not a page's), and never more than the row.
    const long long row_blocks = ((long long)(bt_stride > 0 ? bt_stride : 1) * page_size + FA_BN - 1) / FA_BN;
    const long long share = (row_blocks + nsplit - 1) / nsplit;
    const long long slice = std::min<long long>(bt_stride > 0 ? bt_stride : 1, share * FA_BN / page_size + 2);
    const size_t smem = (in_cluster ? DecodeSmem<HD, NW, true>::fixed : DecodeSmem<HD, NW, false>::fixed) + (size_t)slice * sizeof(int);
    if (smem > 200 * 1024) return CELLM_ERR_SIZE;
    static size_t configured[2] = {0, 0};
    if (smem > configured[in_cluster]) {
        cudaError_t e = in_cluster ? cudaFuncSetAttribute(attention_decode_kernel<HD, NW, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                   : cudaFuncSetAttribute(attention_decode_kernel<HD, NW, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured[in_cluster] = smem;
    }
    dim3 grid((unsigned)B, (unsigned)nkv, (unsigned)nsplit);
    if (!in_cluster) {
        CELLM_RUN((attention_decode_kernel<HD, NW, false>), grid, NW * 32, smem, stream, out, part_o, part_ml, counters, q, k_pool,
                  v_pool, cu, ctx, bt, bt_stride, T, num_pages, page_size, nh, nkv, scale * 1.4426950408889634f, window, err);
        return CELLM_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;       // the pieces of a (request, key/value head) are one cluster along z
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = (unsigned)(nsplit <= 8 ? nsplit : 8);
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    const float scale_log2e = scale * 1.4426950408889634f;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_kernel<HD, NW, true>, out, part_o, part_ml, counters, q, k_pool, v_pool, cu,
                                       ctx, bt, bt_stride, T, num_pages, page_size, nh, nkv, scale_log2e, window, err);
    return e == cudaSuccess ? CELLM_OK : (int)e;
}

}  // namespace

// out, q: [T, nh*hd] bf16; request b owns tokens cu_seqlens[b]..cu_seqlens[b+1], at most
// 16 / (nh / nkv) of them. nsplit > 8 needs part_o [nsplit, T*nh, hd], part_ml
// [nsplit, T*nh, 2] floats (a multiple of eight uses the first nsplit / 8 of them) and B*nkv zeroed counters (left
// zero by the call); 2 to 8 pieces meet in a thread-block cluster and need none of them.
CELLM_API int cellm_attention_decode(void* out, float* part_o, float* part_ml, int* counters, const void* q,
                                     const void* k_pool, const void* v_pool, const int* cu_seqlens,
                                     const int* ctx_lens, const int* block_table, int bt_stride, int B, int T,
                                     int num_pages, int page_size, int nh, int nkv, int hd, float scale, int window,
                                     int nsplit, int* err, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return CELLM_OK;
    if (nkv <= 0 || nh % nkv || nh / nkv > 16) return CELLM_ERR_SIZE;
    if (nsplit < 1 || (nsplit > 8 && (!part_o || !part_ml || !counters))) return CELLM_ERR_ARG;      // up to 8 pieces meet in a cluster
    if (nkv > 65535 || nsplit > 65535) return CELLM_ERR_SIZE;
#define GO(HD_, NW_)                                                                                                \
    return launch_decode<HD_, NW_>((__nv_bfloat16*)out, part_o, part_ml, counters, (const __nv_bfloat16*)q,         \
                                   (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, cu_seqlens, ctx_lens, \
                                   block_table, bt_stride, B, T, num_pages, page_size, nh, nkv, scale, window, nsplit, \
                                   err, stream)
    if (hd == 32) GO(32, 4);
    if (hd == 64) GO(64, 4);
    if (hd == 128) GO(128, 4);
#undef GO
    return CELLM_ERR_SIZE;
}
