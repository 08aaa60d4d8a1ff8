// SwiGLU gate: h[t, j] = g * sigmoid(g) * u with g = gu[t, j], u = gu[t, ff + j]
// (crates/cellm-model/src/lfm.rs:648-654; the two products W1 m and W3 m arrive
// side by side from one matrix product over the stacked weights). 32-bit math; gate and
// up may arrive in 32-bit under bfloat16 activations, so that the only rounding is that of h.
#include "common.cuh"

template <typename T, typename TI>
__global__ void swiglu_kernel(T* __restrict__ h, const TI* __restrict__ gu, int ff, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / ff;
    const int j = (int)(i - t * ff);
    const float g = to_float(gu[t * 2 * ff + j]);
    const float u = to_float(gu[t * 2 * ff + ff + j]);
    h[i] = from_float<T>(g * (1.0f / (1.0f + expf(-g))) * u);
}

CELLM_API int cellm_swiglu(void* h, const void* gu, int T, int ff, int dtype, int gu_dtype, cudaStream_t stream) {
    const size_t n = (size_t)T * ff;
    if (n == 0) return CELLM_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == CELLM_F32 && gu_dtype == CELLM_F32)
        CELLM_RUN((swiglu_kernel<float, float>), blocks, threads, 0, stream, (float*)h, (const float*)gu, ff, n);
    else if (dtype == CELLM_BF16 && gu_dtype == CELLM_BF16)
        CELLM_RUN((swiglu_kernel<__nv_bfloat16, __nv_bfloat16>), blocks, threads, 0, stream, (__nv_bfloat16*)h, (const __nv_bfloat16*)gu, ff, n);
    else if (dtype == CELLM_BF16 && gu_dtype == CELLM_F32)
        CELLM_RUN((swiglu_kernel<__nv_bfloat16, float>), blocks, threads, 0, stream, (__nv_bfloat16*)h, (const float*)gu, ff, n);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
