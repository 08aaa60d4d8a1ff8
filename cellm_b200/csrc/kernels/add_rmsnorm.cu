// Residual add fused with RMSNorm.
//
//   all rows:       x[t] += delta[t];  y[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w
//   selected rows:  v = x[rows[r]] + delta[rows[r]];  y[r] = v / sqrt(mean(v^2) + eps) * w
//
// The residual stream x is 32-bit in every mode; sum and norm are 32-bit
// (crates/cellm-kernels/src/cpu_kernels.rs:17-34 is the formula: the weight is
// used as it is, with no +1). delta may be absent (a plain norm). One block
// per row; the order of the sum depends only on the row length, so a row's
// result does not depend on what else is in the batch.
#include "common.cuh"

template <typename TA, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ delta,
                                   const TW* __restrict__ w, TA* __restrict__ y,
                                   const int* __restrict__ rows, int H, float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float* xr = x + (size_t)t * H;
    const TA* dr = delta ? delta + (size_t)t * H : nullptr;
    const bool write_back = (rows == nullptr) && (delta != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (dr) v += to_float(dr[i]);
        if (write_back) xr[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TA* yr = y + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (dr && !write_back) v += to_float(dr[i]);
        yr[i] = from_float<TA>(v * inv * to_float(w[i]));
    }
}

// The same for rows of bfloat16 activations whose length is a multiple of 8 and at
// most 8 * 1024: every thread keeps its 8 values in registers, so each element is
// read once and written once, in 16-byte pieces. The sum over a row is taken in
// the same order whatever the batch (thread partials of 8, then the block tree).
template <typename TW>
__global__ void add_rmsnorm_vec8_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                        const TW* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                        const int* __restrict__ rows, int H, float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    const int i0 = threadIdx.x * 8;
    const bool on = i0 < H;
    const bool write_back = (rows == nullptr) && (delta != nullptr);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (on) {
        const float4 a = *reinterpret_cast<const float4*>(x + (size_t)t * H + i0);
        const float4 b = *reinterpret_cast<const float4*>(x + (size_t)t * H + i0 + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        if (delta) {
            const uint4 d = *reinterpret_cast<const uint4*>(delta + (size_t)t * H + i0);
            const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(dp[j]);
                v[2 * j] += f.x;
                v[2 * j + 1] += f.y;
            }
        }
        if (write_back) {
            *reinterpret_cast<float4*>(x + (size_t)t * H + i0) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(x + (size_t)t * H + i0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
    float wv[8];                 // the weights travel while the row's sum is taken
#pragma unroll
    for (int j = 0; j < 8; ++j) wv[j] = on ? to_float(w[i0 + j]) : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    if (on) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 pk = __floats2bfloat162_rn(v[2 * j] * inv * wv[2 * j], v[2 * j + 1] * inv * wv[2 * j + 1]);
            o[j] = *reinterpret_cast<uint32_t*>(&pk);
        }
        *reinterpret_cast<uint4*>(y + (size_t)r * H + i0) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// x: [*, H] float; delta: [*, H] act dtype or null; w: [H]; y: [n_rows, H] act dtype;
// rows: null (all n_rows rows, x updated in place) or n_rows row indices (x left as is).
CELLM_API int cellm_add_rmsnorm(float* x, const void* delta, const void* w, int w_dtype, void* y,
                                const int* rows, int n_rows, int H, float eps, int act_dtype,
                                cudaStream_t stream) {
    if (n_rows <= 0) return CELLM_OK;
    if (act_dtype == CELLM_BF16 && (H & 7) == 0 && H <= 8192 && (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)y) & 15) == 0) {
        const int vthreads = ((H / 8 + 31) / 32) * 32;
        if (w_dtype == CELLM_BF16)
            CELLM_RUN(add_rmsnorm_vec8_kernel<__nv_bfloat16>, n_rows, vthreads, 0, stream, x, (const __nv_bfloat16*)delta,
                      (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rows, H, eps);
        else if (w_dtype == CELLM_F32)
            CELLM_RUN(add_rmsnorm_vec8_kernel<float>, n_rows, vthreads, 0, stream, x, (const __nv_bfloat16*)delta,
                      (const float*)w, (__nv_bfloat16*)y, rows, H, eps);
        else return CELLM_ERR_DTYPE;
        return CELLM_OK;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define LAUNCH(TA, TW) \
    CELLM_RUN((add_rmsnorm_kernel<TA, TW>), n_rows, threads, 0, stream, x, (const TA*)delta, (const TW*)w, (TA*)y, rows, H, eps)
    if (act_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float);
    else if (act_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}

// Adds a pending delta into the residual stream without a norm (used when a
// block's output is not followed by a norm that could absorb it).
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ x, const TA* __restrict__ delta, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_float(delta[i]);
}

CELLM_API int cellm_residual_add(float* x, const void* delta, long long n, int act_dtype,
                                 cudaStream_t stream) {
    if (n <= 0) return CELLM_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (act_dtype == CELLM_F32)
        CELLM_RUN(residual_add_kernel<float>, blocks, threads, 0, stream, x, (const float*)delta, (size_t)n);
    else if (act_dtype == CELLM_BF16)
        CELLM_RUN(residual_add_kernel<__nv_bfloat16>, blocks, threads, 0, stream, x, (const __nv_bfloat16*)delta, (size_t)n);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
