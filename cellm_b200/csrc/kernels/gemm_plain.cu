// Plain matrix product on the CUDA cores: C[M,N] = A[M,K] . W[N,K]^T with
// 32-bit multiply-add and 32-bit sums, no tensor cores and no reduced-precision
// mode. Every element of C is summed over k in runs of GP_RUN consecutive
// products, each run in order, and the runs' sums are added in order: the
// rounding of a sum of K terms then grows like sqrt(GP_RUN) + sqrt(K / GP_RUN)
// units instead of sqrt(K), and the order depends on K alone, whatever the tile
// an element falls in, so a row's result does not depend on the other rows of
// the batch. It is the product of the 32-bit path and the reference for the tensor
// core kernels (the reference's own linear is a scalar loop over k,
// crates/cellm-model/src/lfm.rs:970-978).
#include "common.cuh"

#define GP_BM 64
#define GP_BN 64
#define GP_BK 16
#define GP_RUN 256    // products summed in order before their sum joins the total; a multiple of GP_BK

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(TO* __restrict__ C, const TI* __restrict__ A, const TI* __restrict__ W, int M, int N,
                  int K, long long lda, long long ldw, long long ldc) {
    __shared__ float As[GP_BK][GP_BM + 4];
    __shared__ float Ws[GP_BK][GP_BN + 4];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GP_BM, n0 = blockIdx.x * GP_BN;
    float acc[4][4], total[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = total[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GP_BK) {
        if (k0 && k0 % GP_RUN == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) { total[i][j] += acc[i][j]; acc[i][j] = 0.f; }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * 256;
            const int row = idx >> 4, kk = idx & 15;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
            As[kk][row] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[kk][row] = (gn < N && gk < K) ? to_float(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GP_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_float<TO>(total[i][j] + acc[i][j]);
        }
    }
}

// A: [M, K] (row stride lda), W: [N, K] (row stride ldw), both of in_dtype;
// C: [M, N] (row stride ldc) of out_dtype.
CELLM_API int cellm_gemm_plain(void* C, const void* A, const void* W, int M, int N, int K, long long lda,
                               long long ldw, long long ldc, int in_dtype, int out_dtype,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return CELLM_OK;
    if (K <= 0) return CELLM_ERR_SIZE;
    dim3 grid((unsigned)((N + GP_BN - 1) / GP_BN), (unsigned)((M + GP_BM - 1) / GP_BM));
    if (grid.y > 65535) return CELLM_ERR_SIZE;
#define LAUNCH(TI, TO) \
    CELLM_RUN((gemm_plain_kernel<TI, TO>), grid, 256, 0, stream, (TO*)C, (const TI*)A, (const TI*)W, M, N, K, lda, ldw, ldc)
    if (in_dtype == CELLM_F32 && out_dtype == CELLM_F32) LAUNCH(float, float);
    else if (in_dtype == CELLM_BF16 && out_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == CELLM_BF16 && out_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}
