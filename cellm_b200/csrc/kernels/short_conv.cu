// Gated short convolution over portions of sequences, with the state carried
// between portions (crates/cellm-model/src/lfm.rs:363-405 is the formula for
// one token; the reference keeps one state per layer for all sessions, here a
// request has a slot of its own).
//
//   bcx[t] = [ B | C | x ]   (three runs of H values, in that order)
//   bx[t]  = B[t] * x[t]
//   conv[t][c] = sum_k w[c][k] * bx[t - (taps-1) + k][c]  (+ bias[c])   tap taps-1 meets the current token
//   y[t]   = C[t] * conv[t]
//
// History before the first token of a portion comes from the request's state
// slot: taps-1 rows of 32-bit bx values, row taps-2 the most recent; a new
// request's slot is all zeros. The forward kernel only reads the state; the
// update kernel, launched after it, writes the last taps-1 values of bx (mixing
// old rows in when the portion is shorter than taps-1).
#include "common.cuh"

#define SHORT_CONV_MAX_TAPS 16

template <typename TA, typename TW>
__global__ void short_conv_fwd_kernel(TA* __restrict__ y, const TA* __restrict__ bcx,
                                      const TW* __restrict__ w, const TW* __restrict__ bias,
                                      const float* __restrict__ state, long long slot_stride,
                                      const int* __restrict__ slot_ids, const int* __restrict__ seq_of_token,
                                      const int* __restrict__ cu_seqlens, int H, int taps, int n_slots,
                                      int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= H) return;
    const int b = seq_of_token[t];
    const int i = t - cu_seqlens[b];
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_SLOT);
        return;
    }
    const float* st = state + (long long)slot * slot_stride;
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) {
        const int j = i - (taps - 1) + k;
        float v;
        if (j >= 0) {
            const TA* row = bcx + (size_t)(t - (taps - 1) + k) * 3 * H;
            v = to_float(row[c]) * to_float(row[2 * H + c]);
        } else {
            v = st[(size_t)(taps - 1 + j) * H + c];
        }
        acc += v * to_float(w[(size_t)c * taps + k]);
    }
    if (bias) acc += to_float(bias[c]);
    y[(size_t)t * H + c] = from_float<TA>(to_float(bcx[(size_t)t * 3 * H + H + c]) * acc);
}

// The same for bfloat16 rows whose width is a multiple of 8: a thread takes eight
// neighbouring channels of one token and moves them in 16-byte pieces.
template <typename TW>
__global__ void short_conv_fwd_vec8_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bcx,
                                           const TW* __restrict__ w, const TW* __restrict__ bias,
                                           const float* __restrict__ state, long long slot_stride,
                                           const int* __restrict__ slot_ids, const int* __restrict__ seq_of_token,
                                           const int* __restrict__ cu_seqlens, int H, int taps, int n_slots,
                                           int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c0 >= H) return;
    const int b = seq_of_token[t];
    const int i = t - cu_seqlens[b];
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_SLOT);
        return;
    }
    const float* st = state + (long long)slot * slot_stride;
    auto load8 = [](const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); out[2 * j] = f.x; out[2 * j + 1] = f.y; }
    };
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < taps; ++k) {
        const int jj = i - (taps - 1) + k;
        float v[8];
        if (jj >= 0) {
            const __nv_bfloat16* row = bcx + (size_t)(t - (taps - 1) + k) * 3 * H;
            float bb[8], xx[8];
            load8(row + c0, bb);
            load8(row + 2 * H + c0, xx);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = bb[j] * xx[j];
        } else {
            const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + jj) * H + c0);
            const float4 d = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + jj) * H + c0 + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = d.x; v[5] = d.y; v[6] = d.z; v[7] = d.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[j] * to_float(w[(size_t)(c0 + j) * taps + k]);
    }
    float cc[8];
    load8(bcx + (size_t)t * 3 * H + H + c0, cc);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float r0 = cc[2 * j] * (acc[2 * j] + (bias ? to_float(bias[c0 + 2 * j]) : 0.f));
        const float r1 = cc[2 * j + 1] * (acc[2 * j + 1] + (bias ? to_float(bias[c0 + 2 * j + 1]) : 0.f));
        __nv_bfloat162 pk = __floats2bfloat162_rn(r0, r1);
        o[j] = *reinterpret_cast<uint32_t*>(&pk);
    }
    *reinterpret_cast<uint4*>(y + (size_t)t * H + c0) = make_uint4(o[0], o[1], o[2], o[3]);
}

// The same again for long portions (TAPS = 2, 3 or 4): a thread takes eight neighbouring channels
// of a run of RUN tokens and keeps the last TAPS - 1 products B.x in registers as it walks the run, so
// every row of bcx is read once. A run may cross from one request into the next: at a request's first
// token the window is taken from that request's state.
template <typename TW, int TAPS, int RUN>
__global__ void short_conv_fwd_run_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bcx,
                                          const TW* __restrict__ w, const TW* __restrict__ bias,
                                          const float* __restrict__ state, long long slot_stride,
                                          const int* __restrict__ slot_ids, const int* __restrict__ seq_of_token,
                                          const int* __restrict__ cu_seqlens, int T, int H, int n_slots,
                                          int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t0 = blockIdx.x * RUN;
    const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c0 >= H || t0 >= T) return;
    auto load8 = [](const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); out[2 * j] = f.x; out[2 * j + 1] = f.y; }
    };
    float wt[TAPS][8], bs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int k = 0; k < TAPS; ++k) wt[k][j] = to_float(w[(size_t)(c0 + j) * TAPS + k]);
        bs[j] = bias ? to_float(bias[c0 + j]) : 0.f;
    }
    float win[TAPS - 1][8];          // B.x of the TAPS - 1 tokens before the current one, oldest first
    int b = -1, b_start = 0;
    const float* st = nullptr;
    bool bad = false;
#pragma unroll 4
    for (int t = t0; t < min(T, t0 + RUN); ++t) {
        const int bt = seq_of_token[t];
        if (bt != b) {                // the run's first token, or the first token of the next request
            b = bt;
            b_start = cu_seqlens[b];
            const int slot = slot_ids[b];
            bad = slot < 0 || slot >= n_slots;
            if (bad) { if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); }
            else st = state + (long long)slot * slot_stride;
            // the window: tokens of this request before t where there are any, else rows of the state
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) {
                const int jj = (t - b_start) - (TAPS - 1) + k;     // index within the request's portion
                if (bad) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) win[k][j] = 0.f;
                } else if (jj >= 0) {
                    const __nv_bfloat16* row = bcx + (size_t)(b_start + jj) * 3 * H;
                    float bb[8], xx[8];
                    load8(row + c0, bb);
                    load8(row + 2 * H + c0, xx);
#pragma unroll
                    for (int j = 0; j < 8; ++j) win[k][j] = bb[j] * xx[j];
                } else {
                    const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(TAPS - 1 + jj) * H + c0);
                    const float4 d = *reinterpret_cast<const float4*>(st + (size_t)(TAPS - 1 + jj) * H + c0 + 4);
                    win[k][0] = a.x; win[k][1] = a.y; win[k][2] = a.z; win[k][3] = a.w;
                    win[k][4] = d.x; win[k][5] = d.y; win[k][6] = d.z; win[k][7] = d.w;
                }
            }
        }
        const __nv_bfloat16* row = bcx + (size_t)t * 3 * H;
        float bb[8], cc[8], xx[8], cur[8];
        load8(row + c0, bb);
        load8(row + H + c0, cc);
        load8(row + 2 * H + c0, xx);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            cur[j] = bb[j] * xx[j];
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) acc += win[k][j] * wt[k][j];      // oldest tap first, as the other kernels add
            acc += cur[j] * wt[TAPS - 1][j];
            cc[j] = cc[j] * (acc + bs[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 pk = __floats2bfloat162_rn(cc[2 * j], cc[2 * j + 1]);
            o[j] = *reinterpret_cast<uint32_t*>(&pk);
        }
        if (!bad) *reinterpret_cast<uint4*>(y + (size_t)t * H + c0) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
        for (int k = 0; k + 1 < TAPS - 1; ++k)
#pragma unroll
            for (int j = 0; j < 8; ++j) win[k][j] = win[k + 1][j];
#pragma unroll
        for (int j = 0; j < 8; ++j) win[TAPS - 2][j] = cur[j];
    }
}

template <typename TA>
__global__ void short_conv_state_kernel(const TA* __restrict__ bcx, float* __restrict__ state,
                                        long long slot_stride, const int* __restrict__ slot_ids,
                                        const int* __restrict__ cu_seqlens, int H, int taps, int n_slots) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= H) return;
    const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
    const int slot = slot_ids[b];
    if (n <= 0 || slot < 0 || slot >= n_slots) return;
    float* st = state + (long long)slot * slot_stride;
    const int rows = taps - 1;
    float old[SHORT_CONV_MAX_TAPS];
    for (int r = 0; r < rows; ++r) old[r] = st[(size_t)r * H + c];
    for (int r = 0; r < rows; ++r) {
        const int j = n - rows + r;
        float v;
        if (j >= 0) {
            const TA* row = bcx + (size_t)(start + j) * 3 * H;
            v = to_float(row[c]) * to_float(row[2 * H + c]);
        } else {
            v = old[r + n];
        }
        st[(size_t)r * H + c] = v;
    }
}

// Short portions (decoding: one token per request): one thread owns a channel of
// a request, walks the portion's tokens with the history in registers and writes
// the new state itself, so one launch does what the two kernels above do.
template <typename TA, typename TW>
__global__ void short_conv_walk_kernel(TA* __restrict__ y, const TA* __restrict__ bcx, const TW* __restrict__ w,
                                       const TW* __restrict__ bias, float* __restrict__ state, long long slot_stride,
                                       const int* __restrict__ slot_ids, const int* __restrict__ cu_seqlens, int H,
                                       int taps, int n_slots, int* __restrict__ err) {
    pdl_trigger();
    // The step's index arrays, the weights and the state (last written by this kernel in the step before) are the
    // work of no kernel of this step: they are fetched before the wait on the kernel before this one; only the
    // rows of bcx come after it.
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= H) return;
    const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_SLOT);
        return;
    }
    float* st = state + (long long)slot * slot_stride;
    const int rows = taps - 1;
    float hist[SHORT_CONV_MAX_TAPS], wt[SHORT_CONV_MAX_TAPS];
    for (int r = 0; r < rows; ++r) hist[r] = st[(size_t)r * H + c];
    for (int k = 0; k < taps; ++k) wt[k] = to_float(w[(size_t)c * taps + k]);
    const float bs = bias ? to_float(bias[c]) : 0.f;
    pdl_wait();
    for (int i = 0; i < n; ++i) {
        const TA* row = bcx + (size_t)(start + i) * 3 * H;
        const float bx = to_float(row[c]) * to_float(row[2 * H + c]);
        float acc = 0.f;
        for (int k = 0; k < rows; ++k) acc += hist[k] * wt[k];
        acc += bx * wt[rows];
        if (bias) acc += bs;
        y[(size_t)(start + i) * H + c] = from_float<TA>(to_float(row[H + c]) * acc);
        for (int k = 0; k + 1 < rows; ++k) hist[k] = hist[k + 1];
        if (rows > 0) hist[rows - 1] = bx;
    }
    for (int r = 0; r < rows; ++r) st[(size_t)r * H + c] = hist[r];
}

// y: [T, H]; bcx: [T, 3H]; w: [H, taps]; bias: [H] or null; state: this layer's
// [n_slots][taps-1][H] floats with slot_stride floats between slots. max_q_len: the
// longest portion of the batch (portions of up to 4 tokens take the one-launch walk).
CELLM_API int cellm_short_conv(void* y, const void* bcx, const void* w, const void* bias, int w_dtype,
                               float* state, long long slot_stride, const int* slot_ids,
                               const int* seq_of_token, const int* cu_seqlens, int T, int B, int H,
                               int taps, int n_slots, int max_q_len, int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (taps < 1 || taps > SHORT_CONV_MAX_TAPS) return CELLM_ERR_SIZE;
    const int threads = 128;
    dim3 grid_f((unsigned)T, (unsigned)((H + threads - 1) / threads));
    dim3 grid_s((unsigned)B, (unsigned)((H + threads - 1) / threads));
    dim3 grid_v((unsigned)T, (unsigned)((H / 8 + threads - 1) / threads));
    const bool vec8 = act_dtype == CELLM_BF16 && (H & 7) == 0 && (slot_stride & 3) == 0 &&
                      (((uintptr_t)y | (uintptr_t)bcx | (uintptr_t)state) & 15) == 0;
#define LAUNCH(TA, TW)                                                                              \
    do {                                                                                            \
        if (max_q_len > 0 && max_q_len <= 4) {                                                      \
            CELLM_RUN((short_conv_walk_kernel<TA, TW>), grid_s, threads, 0, stream, (TA*)y, (const TA*)bcx, \
                      (const TW*)w, (const TW*)bias, state, slot_stride, slot_ids, cu_seqlens, H, taps, n_slots, err); \
            break;                                                                                  \
        }                                                                                           \
        if (vec8 && T >= 256 && taps >= 2 && taps <= 4) {                                          \
            /* long portions: runs of eight tokens per thread, each row of bcx read once */        \
            dim3 grid_r((unsigned)((T + 7) / 8), (unsigned)((H / 8 + threads - 1) / threads));      \
            if (taps == 2) CELLM_RUN((short_conv_fwd_run_kernel<TW, 2, 8>), grid_r, threads, 0, stream, (__nv_bfloat16*)y, (const __nv_bfloat16*)bcx, (const TW*)w, (const TW*)bias, (const float*)state, slot_stride, slot_ids, seq_of_token, cu_seqlens, T, H, n_slots, err); \
            else if (taps == 3) CELLM_RUN((short_conv_fwd_run_kernel<TW, 3, 8>), grid_r, threads, 0, stream, (__nv_bfloat16*)y, (const __nv_bfloat16*)bcx, (const TW*)w, (const TW*)bias, (const float*)state, slot_stride, slot_ids, seq_of_token, cu_seqlens, T, H, n_slots, err); \
            else CELLM_RUN((short_conv_fwd_run_kernel<TW, 4, 8>), grid_r, threads, 0, stream, (__nv_bfloat16*)y, (const __nv_bfloat16*)bcx, (const TW*)w, (const TW*)bias, (const float*)state, slot_stride, slot_ids, seq_of_token, cu_seqlens, T, H, n_slots, err); \
        } else if (vec8) {                                                                          \
            CELLM_RUN(short_conv_fwd_vec8_kernel<TW>, grid_v, threads, 0, stream, (__nv_bfloat16*)y,     \
                      (const __nv_bfloat16*)bcx, (const TW*)w, (const TW*)bias, (const float*)state, slot_stride, \
                      slot_ids, seq_of_token, cu_seqlens, H, taps, n_slots, err);                   \
        } else {                                                                                    \
            CELLM_RUN((short_conv_fwd_kernel<TA, TW>), grid_f, threads, 0, stream,                  \
                      (TA*)y, (const TA*)bcx, (const TW*)w, (const TW*)bias, (const float*)state, slot_stride, slot_ids, \
                      seq_of_token, cu_seqlens, H, taps, n_slots, err);                             \
        }                                                                                           \
        if (taps > 1)                                                                               \
            CELLM_RUN(short_conv_state_kernel<TA>, grid_s, threads, 0, stream,                      \
                      (const TA*)bcx, state, slot_stride, slot_ids, cu_seqlens, H, taps, n_slots);  \
    } while (0)
    if (act_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float);
    else if (act_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}
