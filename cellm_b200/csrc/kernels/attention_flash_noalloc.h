/* Paged flash attention through an entry point that allocates nothing.
 *
 * This entry point has no counterpart in jeffasante/cellm (whose attention is a
 * single-token loop on the CPU or a Metal shader); it exists for callers of this
 * library that cannot allocate device memory at the moment they need attention:
 * a host callback or latency-critical thread that must not enter the driver's
 * allocator, an embedding application that was given a fixed arena, code that
 * runs between CUDA-graph replays and has to keep every address stable.
 *
 * It computes what cellm_attention_flash computes. The caller passes inputs and
 * the output; the pieces of a split over the keys are kept in an 8 MiB array
 * that is part of the library image (2,097,152 floats; every GPU that loads the
 * library holds it until the process exits). A call needs
 * nsplit * T * nh * (hd + 2) floats of it and is refused with -5 when that is
 * more than the array holds. The first call on each device looks the array's
 * address up and should be made outside stream capture. All calls share the
 * array: calls that overlap on the GPU race and must be serialised by the caller.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* out, q: [T, nh*hd] bfloat16; k_pool, v_pool: one layer's cache
 * [pages][kv heads][page size][hd] bfloat16; cu_seqlens [B+1], ctx_lens [B],
 * block_table [B][bt_stride] int32 on the device; T must equal cu_seqlens[B] (the
 * host cannot check it: with a larger T the merge of the pieces reads rows of the
 * shared array that this call did not write); n_tiles = sum over requests of
 * ceil(q_len * (nh / nkv) / (wide ? 64 : 16)); err: device error word.
 * Returns 0, a cudaError_t (> 0), or a negative refusal code. */
int cellm_attention_flash_noalloc(void* out, const void* q, const void* k_pool, const void* v_pool,
                                  const int* cu_seqlens, const int* ctx_lens, const int* block_table,
                                  int bt_stride, int B, int T, int n_tiles, int num_pages, int page_size,
                                  int nh, int nkv, int hd, float scale, int window, int wide, int nsplit,
                                  int* err, cudaStream_t stream);

/* Floats the built-in scratch holds. */
long long cellm_attention_flash_noalloc_capacity(void);

/* A sentence for a return code of cellm_attention_flash_noalloc. */
const char* cellm_attention_flash_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
