// Embedding: out[t, :] = float(table[ids[t], :]) into the 32-bit residual stream.
// The reference gathers one row per token and refuses an id beyond the
// vocabulary (crates/cellm-model/src/lfm.rs:817-890). Here a bad id sets a bit
// in the device error word and its row is written as zeros.
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int H, int V, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_TOKEN);
    const T* row = table + (size_t)(ok ? id : 0) * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? to_float(row[i]) : 0.f;
}

// The step's index arrays go up in one asynchronous copy from pinned host memory (a plain call of the runtime,
// here so that the step function pays one short foreign call for it instead of a tensor operation).
CELLM_API int cellm_upload(void* dst, const void* pinned_src, long long bytes, cudaStream_t stream) {
    if (bytes <= 0) return CELLM_OK;
    const cudaError_t e = cudaMemcpyAsync(dst, pinned_src, (size_t)bytes, cudaMemcpyHostToDevice, stream);
    return e == cudaSuccess ? CELLM_OK : (int)e;
}

// The embedding is the first kernel of a forward pass: it is launched without the attribute that lets a kernel
// start under its predecessor (see common.cuh), so that no kernel of this pass overlaps the pass before it.
CELLM_API int cellm_embed(float* out, const void* table, int table_dtype, const int* ids, int T, int H,
                          int V, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == CELLM_F32)
        CELLM_RUN_SERIAL(embed_kernel<float>, T, threads, 0, stream, out, (const float*)table, ids, H, V, err);
    else if (table_dtype == CELLM_BF16)
        CELLM_RUN_SERIAL(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, out, (const __nv_bfloat16*)table, ids, H, V, err);
    else
        return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
