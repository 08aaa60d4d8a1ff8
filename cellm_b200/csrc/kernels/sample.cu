// Token choice on the device: arg-max, and temperature sampling over the top k
// logits or the whole row, in the order of tools/infer's select_next
// (tools/infer/src/main.rs:958-1016) and of the runner's top-k list
// (crates/cellm-model/src/lfm.rs:806-815).
#include "common.cuh"

// Order-preserving 32-bit key of a logit (larger logit, larger key); non-finite logits count as -inf and -0 as +0,
// so that equal logits have equal keys.
__device__ __forceinline__ uint32_t float_key(float v) {
    if (!isfinite(v)) v = -INFINITY;
    v += 0.0f;
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
// (key of the logit, ~id): the larger of two is the larger logit, or among equal logits the lower id
__device__ __forceinline__ unsigned long long pick_key(float v, int i) {
    return ((unsigned long long)float_key(v) << 32) | (0xffffffffu - (uint32_t)i);
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, k, o);
        k = t > k ? t : k;
    }
    return k;
}

// ---------------------------------------------------------------- arg-max
// Largest logit of each row; among equal logits the lowest id wins (the
// reference's stable descending sort puts it first). Non-finite logits count
// as -inf (crates/cellm-model/src/lfm.rs:810).
__global__ void argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_trigger();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float v = row[i];
        if (!isfinite(v)) v = -INFINITY;
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? bv[lane] : -INFINITY;
        idx = lane < nw ? bi[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx;
    }
}

// The same in two steps for long rows, so that a few rows still use many SMs: ARGMAX_PARTS blocks a row each
// leave the best (logit, id) of their run of the row, and one warp a row picks among those.
#define ARGMAX_PARTS 32
__global__ void __launch_bounds__(256)
argmax_parts_kernel(unsigned long long* __restrict__ parts, const float* __restrict__ logits, int V) {
    __shared__ unsigned long long best_w[8];
    pdl_trigger();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.y * V;
    const int per = ((V + ARGMAX_PARTS - 1) / ARGMAX_PARTS + 3) & ~3;
    const int begin = blockIdx.x * per, end = min(V, begin + per);
    unsigned long long best = 0ull;
    if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        for (int i = begin + threadIdx.x * 4; i < end; i += 256 * 4) {        // per is a multiple of 4, so i + 3 < V
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            unsigned long long k = pick_key(v.x, i);
            unsigned long long t = pick_key(v.y, i + 1); k = t > k ? t : k;
            t = pick_key(v.z, i + 2); k = t > k ? t : k;
            t = pick_key(v.w, i + 3); k = t > k ? t : k;
            best = k > best ? k : best;
        }
    } else {
        for (int i = begin + threadIdx.x; i < end; i += 256) {
            const unsigned long long k = pick_key(row[i], i);
            best = k > best ? k : best;
        }
    }
    best = warp_max_u64(best);
    if ((threadIdx.x & 31) == 0) best_w[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = warp_max_u64(threadIdx.x < 8 ? best_w[threadIdx.x] : 0ull);
        if (threadIdx.x == 0) parts[(size_t)blockIdx.y * ARGMAX_PARTS + blockIdx.x] = best;
    }
}
__global__ void argmax_pick_kernel(int* __restrict__ out, const unsigned long long* __restrict__ parts) {
    pdl_trigger();
    pdl_wait();
    const unsigned long long k = warp_max_u64(threadIdx.x < ARGMAX_PARTS ? parts[(size_t)blockIdx.x * ARGMAX_PARTS + threadIdx.x] : 0ull);
    if (threadIdx.x == 0) out[blockIdx.x] = (int)(0xffffffffu - (uint32_t)(k & 0xffffffffu));
}

// parts: R * 32 64-bit words of scratch for rows of 8,192 logits or more (null: one block a row).
CELLM_API int cellm_argmax(int* out, const float* logits, int R, int V, unsigned long long* parts, cudaStream_t stream) {
    if (R <= 0) return CELLM_OK;
    if (parts != nullptr && V >= 8192) {
        CELLM_RUN(argmax_parts_kernel, dim3(ARGMAX_PARTS, (unsigned)R), 256, 0, stream, parts, logits, V);
        CELLM_RUN(argmax_pick_kernel, R, 32, 0, stream, out, (const unsigned long long*)parts);
        return CELLM_OK;
    }
    CELLM_RUN(argmax_kernel, R, 512, 0, stream, out, logits, V);
    return CELLM_OK;
}

// ------------------------------------------------------- tokens that stay on the device between two steps
// The engine may launch a step before it has read the tokens of the step before (its own work for the next step then
// runs beside the GPU's). The ids of such tokens come to this step as -1; their values are where the step before
// left them: last[state slot of the token's request].
__global__ void take_pending_tokens_kernel(int* __restrict__ ids, const int* __restrict__ seq_of_token,
                                           const int* __restrict__ slot_ids, const int* __restrict__ last, int T,
                                           int n_slots, int* __restrict__ err) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T || ids[t] >= 0) return;
    const int slot = slot_ids[seq_of_token[t]];
    if (slot < 0 || slot >= n_slots) { atomicOr(err, CELLM_DEV_BAD_SLOT); return; }
    ids[t] = last[slot];
}

__global__ void keep_last_tokens_kernel(int* __restrict__ last, const int* __restrict__ slot_ids,
                                        const int* __restrict__ tokens, int R, int n_slots) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int slot = slot_ids[r];
    if (slot >= 0 && slot < n_slots) last[slot] = tokens[r];
}

// ids: [T] token ids of the step (changed in place where -1); seq_of_token: [T] entry of each token; slot_ids: one
// per entry; last: [n_slots]. Launched as the first kernel of a step: it starts only when everything earlier on the
// stream has finished.
CELLM_API int cellm_take_pending_tokens(int* ids, const int* seq_of_token, const int* slot_ids, const int* last, int T,
                                        int n_slots, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    CELLM_RUN_SERIAL(take_pending_tokens_kernel, (unsigned)((T + 127) / 128), 128, 0, stream, ids, seq_of_token, slot_ids,
                     last, T, n_slots, err);
    return CELLM_OK;
}

// last[slot_ids[r]] = tokens[r] for the R rows of a step in which every entry is one decoded token.
CELLM_API int cellm_keep_last_tokens(int* last, const int* slot_ids, const int* tokens, int R, int n_slots,
                                     cudaStream_t stream) {
    if (R <= 0) return CELLM_OK;
    CELLM_RUN(keep_last_tokens_kernel, (unsigned)((R + 127) / 128), 128, 0, stream, last, slot_ids, tokens, R, n_slots);
    return CELLM_OK;
}

// ------------------------------------------------------- temperature sampling
// One block per row. With top_k > 0 the k largest logits are the candidates, in
// descending order of logit and ascending id among equal logits (a stable
// descending sort, crates/cellm-model/src/lfm.rs:813); with top_k = 0 the
// whole row is, in the order of the ids. Then, as tools/infer's select_next
// (tools/infer/src/main.rs:958-1016): candidates seen among the `recent` tokens
// have their score divided by repeat_penalty (if > 1); weights are
// exp((s - max) / temperature); r = u * sum; the first candidate whose running
// sum reaches r is taken. temperature <= 0 takes the arg-max. One thread walks
// the top-k candidates in order, so sums round as in the reference.
#define SAMPLE_THREADS 1024
#define SAMPLE_MAX_K 1024


// Inclusive scan of one value per thread over the block; returns this thread's
// prefix and, through `total`, the block's sum. Fixed order.
__device__ __forceinline__ float block_scan_inclusive(float v, float* warp_tot, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nw ? warp_tot[lane] : 0.f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += t;
        }
        warp_tot[lane] = w;
    }
    __syncthreads();
    const float base = warp > 0 ? warp_tot[warp - 1] : 0.f;
    *total = warp_tot[nw - 1];
    return v + base;
}

__device__ __forceinline__ int block_scan_inclusive_int(int v, int* warp_tot, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int w = lane < nw ? warp_tot[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += t;
        }
        warp_tot[lane] = w;
    }
    __syncthreads();
    const int base = warp > 0 ? warp_tot[warp - 1] : 0;
    *total = warp_tot[nw - 1];
    return v + base;
}

// Largest key of every group of 128 logits of a row, a warp a group. The k-th largest of a row's group maxima is a
// lower bound of its k-th largest logit (k different logits reach it), so sample_kernel looks only at the few logits
// that reach that bound instead of selecting among all of them.
#define SAMPLE_GROUP 128
#define SAMPLE_MAX_GROUPS 8192
__global__ void __launch_bounds__(256)
group_max_kernel(uint32_t* __restrict__ gmax, const float* __restrict__ logits, int V, int G) {
    pdl_trigger();
    pdl_wait();
    const int g = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (g >= G) return;
    const float* row = logits + (size_t)blockIdx.y * V;
    uint32_t key = 0u;
#pragma unroll
    for (int e = 0; e < SAMPLE_GROUP / 32; ++e) {
        const int i = g * SAMPLE_GROUP + e * 32 + lane;
        if (i < V) key = max(key, float_key(row[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) key = max(key, __shfl_xor_sync(0xffffffffu, key, o));
    if (lane == 0) gmax[(size_t)blockIdx.y * G + g] = key;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ u, const float* __restrict__ penalty,
              const int* __restrict__ recent, int W, int bitmap_words, const uint32_t* __restrict__ gmax, int G,
              int g_sort) {
    extern __shared__ uint32_t dyn_words[];      // the groups' maxima (top-k rows) or a bit per id (whole rows)
    __shared__ unsigned long long cand[SAMPLE_MAX_K];
    __shared__ int hist[256];
    __shared__ float fscratch[32];
    __shared__ int iscratch[32];
    __shared__ int s_recent[256];
    __shared__ uint32_t s_prefix, s_mask;
    __shared__ int s_krem, s_cnt, s_pick;
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * V;
    const float temp = temperature[r];
    const float pen = penalty ? penalty[r] : 1.0f;
    const int nrec = (pen > 1.0f && recent) ? min(W, 256) : 0;
    for (int i = tid; i < nrec; i += blockDim.x) s_recent[i] = recent[(size_t)r * W + i];
    __syncthreads();

    if (temp <= 0.0f && gmax == nullptr) {  // arg-max, lowest id among equals
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int i = tid; i < V; i += blockDim.x) {
            float v = row[i];
            if (!isfinite(v)) v = -INFINITY;
            if (v > best || (v == best && i < idx)) { best = v; idx = i; }
        }
        unsigned long long key = ((unsigned long long)float_key(best) << 32) | (0xffffffffu - (uint32_t)idx);
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long t = __shfl_xor_sync(0xffffffffu, key, o);
            key = t > key ? t : key;
        }
        if ((tid & 31) == 0) cand[tid >> 5] = key;
        __syncthreads();
        if (tid < 32) {
            key = cand[tid];
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long t = __shfl_xor_sync(0xffffffffu, key, o);
                key = t > key ? t : key;
            }
            if (tid == 0) out[r] = (int)(0xffffffffu - (uint32_t)(key & 0xffffffffu));
        }
        return;
    }

    int k = temp <= 0.0f ? 1 : top_k[r];          // with the groups' maxima the arg-max is the first of one candidate
    if (k >= V) k = 0;
    if (k > 0) {
        int n = -1;                               // candidates in cand[], or -1 while there are none
        if (gmax != nullptr && k <= G) {
            // ---- the k-th largest group maximum bounds the k-th largest logit from below
            for (int i = tid; i < g_sort; i += blockDim.x) dyn_words[i] = i < G ? gmax[(size_t)r * G + i] : 0u;
            if (tid == 0) s_cnt = 0;
            __syncthreads();
            for (int size = 2; size <= g_sort; size <<= 1) {
                for (int stride = size >> 1; stride > 0; stride >>= 1) {
                    for (int t = tid; t < g_sort / 2; t += blockDim.x) {
                        const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
                        const uint32_t a = dyn_words[lo], b = dyn_words[hi];
                        if ((a < b) == ((lo & size) == 0)) { dyn_words[lo] = b; dyn_words[hi] = a; }
                    }
                    __syncthreads();
                }
            }
            const uint32_t bound = dyn_words[k - 1];
            for (int i = tid; i < V; i += blockDim.x) {
                const uint32_t key = float_key(row[i]);
                if (key >= bound) {
                    const int p = atomicAdd(&s_cnt, 1);
                    if (p < SAMPLE_MAX_K) cand[p] = ((unsigned long long)key << 32) | (0xffffffffu - (uint32_t)i);
                }
            }
            __syncthreads();
            if (s_cnt <= SAMPLE_MAX_K) n = s_cnt;  // else (many equal logits at the bound): select among the whole row
            __syncthreads();
        }
        if (n < 0) {
        // ---- radix select of the k-th largest key
        if (tid == 0) { s_prefix = 0; s_mask = 0; s_krem = k; s_cnt = 0; }
        __syncthreads();
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hist[tid] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix, mask = s_mask;
            for (int i = tid; i < V; i += blockDim.x) {
                const uint32_t key = float_key(row[i]);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int rem = s_krem, b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= rem) break;
                    rem -= hist[b];
                }
                s_krem = rem;
                s_prefix = prefix | ((uint32_t)b << shift);
                s_mask = mask | (0xffu << shift);
            }
            __syncthreads();
        }
        const uint32_t kth = s_prefix;
        const int need_eq = s_krem;          // how many keys equal to kth are taken
        const int n_gt = k - need_eq;        // keys above kth
        for (int i = tid; i < V; i += blockDim.x) {
            const uint32_t key = float_key(row[i]);
            if (key > kth) {
                const int p = atomicAdd(&s_cnt, 1);
                cand[p] = ((unsigned long long)key << 32) | (0xffffffffu - (uint32_t)i);
            }
        }
        // equal keys: the lowest ids first
        int base = 0;
        for (int c0 = 0; c0 < V && base < need_eq; c0 += blockDim.x) {
            const int i = c0 + tid;
            const int flag = (i < V && float_key(row[i]) == kth) ? 1 : 0;
            int total;
            const int incl = block_scan_inclusive_int(flag, iscratch, &total);
            const int rank = base + incl - flag;
            if (flag && rank < need_eq) cand[n_gt + rank] = ((unsigned long long)kth << 32) | (0xffffffffu - (uint32_t)i);
            base += total;
            __syncthreads();
        }
        n = k;
        }
        int n_sort = 2;
        while (n_sort < n) n_sort <<= 1;
        for (int i = n + tid; i < n_sort; i += blockDim.x) cand[i] = 0ull;   // sorts below every real key
        __syncthreads();
        // ---- bitonic sort, descending: larger logit first, lower id first among equal logits
        for (int size = 2; size <= n_sort; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                const int j = tid ^ stride;
                if (j > tid && j < n_sort) {
                    const unsigned long long a = cand[tid], b = cand[j];
                    const bool desc = (tid & size) == 0;
                    if ((a < b) == desc) { cand[tid] = b; cand[j] = a; }
                }
                __syncthreads();
            }
        }
        if (temp <= 0.0f) {
            if (tid == 0) out[r] = (int)(0xffffffffu - (uint32_t)(cand[0] & 0xffffffffu));
            return;
        }
        // penalised scores and their weights by a thread each; one thread adds them in the candidates' order
        float sc = -INFINITY;
        int id = 0;
        if (tid < k) {
            id = (int)(0xffffffffu - (uint32_t)(cand[tid] & 0xffffffffu));
            sc = key_float((uint32_t)(cand[tid] >> 32));
            for (int j = 0; j < nrec; ++j)
                if (s_recent[j] == id) { sc = sc / pen; break; }
        }
        const float mx = block_max(sc, fscratch);
        if (tid < k) cand[tid] = ((unsigned long long)__float_as_uint(expf((sc - mx) / temp)) << 32) | (uint32_t)id;
        __syncthreads();
        if (tid == 0) {
            float sum = 0.f;
            for (int i = 0; i < k; ++i) sum += __uint_as_float((uint32_t)(cand[i] >> 32));
            int pick = (int)(cand[0] & 0xffffffffu);
            if (sum != 0.f) {
                const float rr = u[r] * sum;
                float acc = 0.f;
                pick = (int)(cand[k - 1] & 0xffffffffu);
                for (int i = 0; i < k; ++i) {
                    acc += __uint_as_float((uint32_t)(cand[i] >> 32));
                    if (rr <= acc) { pick = (int)(cand[i] & 0xffffffffu); break; }
                }
            }
            out[r] = pick;
        }
        return;
    }

    // ---- whole row, in the order of the ids
    // which ids are recent: a bit each in shared memory where the row fits, else the list is searched
    uint32_t* recent_bits = dyn_words;
    if (bitmap_words > 0 && nrec > 0) {
        for (int i = tid; i < bitmap_words; i += blockDim.x) recent_bits[i] = 0u;
        __syncthreads();
        for (int j = tid; j < nrec; j += blockDim.x) {
            const int id = s_recent[j];
            if (id >= 0 && id < V) atomicOr(&recent_bits[id >> 5], 1u << (id & 31));
        }
        __syncthreads();
    }
    auto score = [&](int i) -> float {
        float s = row[i];
        if (!isfinite(s)) s = -INFINITY;
        if (nrec > 0) {
            if (bitmap_words > 0) {
                if ((recent_bits[i >> 5] >> (i & 31)) & 1u) s = s / pen;
            } else {
                for (int j = 0; j < nrec; ++j)
                    if (s_recent[j] == i) { s = s / pen; break; }
            }
        }
        return s;
    };
    float mx = -INFINITY;
    for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, score(i));
    mx = block_max(mx, fscratch);
    __syncthreads();
    float acc = 0.f;
    for (int c0 = 0; c0 < V; c0 += blockDim.x) {
        const int i = c0 + tid;
        const float w = i < V ? expf((score(i) - mx) / temp) : 0.f;
        float total;
        block_scan_inclusive(w, fscratch, &total);
        acc += total;
        __syncthreads();
    }
    if (tid == 0) s_pick = 0x7fffffff;
    __syncthreads();
    if (acc == 0.f) {
        if (tid == 0) out[r] = 0;
        return;
    }
    const float rr = u[r] * acc;
    float run = 0.f;
    for (int c0 = 0; c0 < V; c0 += blockDim.x) {
        const int i = c0 + tid;
        const float w = i < V ? expf((score(i) - mx) / temp) : 0.f;
        float total;
        const float incl = block_scan_inclusive(w, fscratch, &total);
        if (i < V && rr <= run + incl) atomicMin(&s_pick, i);
        run += total;
        __syncthreads();
        if (s_pick != 0x7fffffff) break;
    }
    __syncthreads();
    if (tid == 0) out[r] = s_pick != 0x7fffffff ? s_pick : V - 1;
}

// logits [R, V] float32; temperature, u, penalty [R] float32; top_k [R] int32
// (0 = whole row, at most 1024); recent [R, W] int32 padded with -1 (W <= 256) or null.
// max_top_k: the largest top_k of the rows. group_max: scratch of R * ceil(V / 128) 32-bit words, or null; with it
// (and a row of 2,048 to a million logits) the rows that take the top k, or the arg-max, look only at the logits that
// reach the k-th largest of the maxima of groups of 128.
CELLM_API int cellm_sample(int* out, const float* logits, int R, int V, const float* temperature,
                           const int* top_k, const float* u, const float* penalty, const int* recent,
                           int W, int max_top_k, uint32_t* group_max, cudaStream_t stream) {
    if (R <= 0) return CELLM_OK;
    if (max_top_k > SAMPLE_MAX_K || W > 256 || W < 0) return CELLM_ERR_SIZE;
    int G = (V + SAMPLE_GROUP - 1) / SAMPLE_GROUP, g_sort = 0;
    if (group_max != nullptr && V >= 2048 && G <= SAMPLE_MAX_GROUPS) {
        g_sort = 2;
        while (g_sort < G) g_sort <<= 1;
        CELLM_RUN(group_max_kernel, dim3((unsigned)((G + 7) / 8), (unsigned)R), 256, 0, stream, group_max, logits, V, G);
    } else {
        group_max = nullptr;
        G = 0;
    }
    // a bit per id for the recent tokens of rows that draw from the whole row, where that fits beside the static arrays
    const int words = (V + 31) / 32;
    const int bitmap_words = (recent != nullptr && W > 0 && words <= 8192) ? words : 0;
    const int dyn = bitmap_words > g_sort ? bitmap_words : g_sort;
    CELLM_RUN(sample_kernel, R, SAMPLE_THREADS, (size_t)dyn * sizeof(uint32_t), stream, out, logits, V, temperature, top_k, u,
              penalty, recent, W, bitmap_words, (const uint32_t*)group_max, G, g_sort);
    return CELLM_OK;
}
