// The forward pass of one step, launched from native code.
//
// A step that carries prompt tokens launches about ten kernels a layer; from
// Python each launch costs some ten microseconds of interpreter time, which a
// step of a few hundred tokens cannot hide. The executor walks the same layers
// and takes the same decisions (which kernel, which tile shape, which K split)
// as the Python parts do, in one foreign call per step. It knows the parts this
// package ships (pre-norm blocks of a short-convolution or attention mixer and a
// SwiGLU feed-forward, RMS norms, rotary positions); a plan with any other part
// stays with the Python path.
//
// The kernels are reached through a table of entry points that the caller fills
// (the addresses of the compiled libraries' C symbols), so this file has no
// dependency on CUDA and its decisions can be tested on a machine without a GPU
// by filling the table with recording stand-ins.
//
// All structs have 8-byte fields only, so that their layout is the same on both
// sides of the foreign call; cellm_exec_sizeof() lets the caller check.
#pragma once
#include <cstdint>

namespace cellm {

typedef long long i64;

// Element types as the kernels tag them.
enum : i64 { EXEC_F32 = 0, EXEC_BF16 = 1 };

struct ExecLinear {
    const void* w;      // [N, K], row pitch ldw elements
    i64 N, K, ldw;
    i64 dtype;          // element type of w
    i64 tc_ok;          // w meets the tensor-core kernel's alignment rules
};

struct ExecLayer {
    i64 kind;           // 0: short convolution, 1: attention
    const void* norm1_w; i64 norm1_dtype; double norm1_eps;
    const void* norm2_w; i64 norm2_dtype; double norm2_eps;
    // feed-forward
    ExecLinear gate_up, down;
    i64 ff, ff_fused;   // ff_fused: gate_up holds interleaved gate and up blocks for the product's SwiGLU epilogue
    // short convolution
    ExecLinear in_proj, conv_out;
    const void* in_proj_tiled; i64 tiled_rows;      // in_proj in tiles of 42 channels (null: none)
    const void* taps; const void* conv_bias; i64 taps_dtype, n_taps;
    // attention
    ExecLinear qkv, attn_out;
    i64 nh, nkv, hd, window; double scale;
    const void* q_norm_w; const void* k_norm_w; i64 qk_dtype; double qk_eps;
    i64 rot, interleaved; const void* inv_freq;
};

// Entry points of the kernel libraries, in the order of ExecProgram::fns.
enum ExecFn {
    FN_EMBED, FN_ADD_RMSNORM, FN_SWIGLU, FN_SHORT_CONV, FN_QK_NORM_ROPE, FN_ATTENTION_PLAIN, FN_GEMM_PLAIN,
    FN_ATTENTION_DECODE, FN_ATTENTION_TC, FN_ATTENTION_FLASH, FN_GEMM_TCGEN05, FN_GEMM_CONV, FN_GEMM_ROPE, FN_COUNT
};

struct ExecProgram {
    i64 n_layers, n_order, H, V, act_dtype;
    i64 sms, static_flag, cluster_reduce, fused_rope, max_counters;
    i64 tc_min_ctas;            // < 0: an eighth of the SMs
    double tc_min_fill;
    const void* embedding; i64 embedding_dtype;
    const void* final_w; i64 final_dtype; double final_eps;
    ExecLinear head;
    const ExecLayer* layers;    // [n_layers]
    const i64* order;           // [n_order]: the layer each item of the run order runs
    void* fns[FN_COUNT];
};

// The cache an item of the run order works on in this step.
struct ExecItem {
    void* k; void* v; const void* block_table;
    i64 bt_stride, num_pages, page_size, writes;
    void* state; i64 slot_stride, n_slots;
};

struct ExecStep {
    i64 T, B, R, max_q_len, max_total_len, n_order;   // n_order: run only the first items (<= program's)
    const void *ids, *positions, *seq_of_token, *cu_seqlens, *ctx_lens, *slot_ids, *rows;
    const i64* q_lens;          // host copy, [B]
    const ExecItem* items;      // [n_order]
    void* arena; i64 arena_bytes;
    void* logits;               // [R, V] float, or null when R = 0
    void* err; void* stream;
    void* gemm_ws; i64 gemm_ws_floats;
    void* attn_ws; i64 attn_ws_floats;
    void* counters;
    i64 launches;               // out: kernels launched
};

// What the step needs, found by walking it without a launch: need[0] bytes of arena, need[1] floats of
// the products' workspace, need[2] floats of the attention workspace. Also sets s.launches.
void exec_need(const ExecProgram& p, ExecStep& s, i64* need);
// Runs the step. 0, or the failing kernel's status (the message names it).
int exec_forward(const ExecProgram& p, ExecStep& s);

// The tile shape and K split of a product, as cellm_b200/ops/gemm_bf16.py plans it.
void plan_tiles(i64 M, i64 N, i64 K, i64 sms, i64* bn, i64* split);

}  // namespace cellm
