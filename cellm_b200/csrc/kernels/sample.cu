// Token choice on the device: arg-max, and temperature sampling over the top k
// logits or the whole row, in the order of tools/infer's select_next
// (tools/infer/src/main.rs:958-1016) and of the runner's top-k list
// (crates/cellm-model/src/lfm.rs:806-815).
#include "common.cuh"

// ---------------------------------------------------------------- arg-max
// Largest logit of each row; among equal logits the lowest id wins (the
// reference's stable descending sort puts it first). Non-finite logits count
// as -inf (crates/cellm-model/src/lfm.rs:810).
__global__ void argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V) {
    __shared__ float bv[32];
    __shared__ int bi[32];
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

CELLM_API int cellm_argmax(int* out, const float* logits, int R, int V, cudaStream_t stream) {
    if (R <= 0) return CELLM_OK;
    argmax_kernel<<<R, 512, 0, stream>>>(out, logits, V);
    CELLM_LAUNCH_CHECK();
    return CELLM_OK;
}
