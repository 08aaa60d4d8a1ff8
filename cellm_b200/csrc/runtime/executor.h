// The forward pass of one step, launched from native code.
//
// A model is described to the executor as a program of op records: a prologue
// (the embedding), the records of every layer, the run order of the layers, and
// an epilogue (final norm on the wanted rows, output product). The records are
// emitted by the parts themselves (cellm_b200/parts: each part's emit()), one
// record per part, so the executor knows kinds of parts, never a model: a layer
// is whatever list of records its block arrangement emitted. A part that has no
// native record emits OP_PYTHON, and the executor calls back into the
// interpreter for that part alone; the parts around it stay native.
//
// The records work on three registers:
//   x        the 32-bit residual stream [T, H]
//   pending  an addend [T, H] that waits to be added into x (or null)
//   y        the activations the next part reads (the output of the last norm)
// A norm adds `pending` into x and leaves the normed rows in y; a mixer or a
// feed-forward reads y and leaves its output as the new `pending` (if one waits
// already, that one is added into x first).
//
// The executor also owns the decisions below the parts: which kernel serves a
// product or an attention of a given shape, which tile shape and K split. The
// interpreter's kernel wrappers ask it (cellm_exec_plan_tiles, cellm_exec_part)
// instead of deciding a second time.
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

// ---- op records ---------------------------------------------------------------------------------------------------
enum OpKind : i64 {
    OP_EMBED = 0, OP_RMS_NORM, OP_SHORT_CONV, OP_ATTENTION, OP_SWIGLU, OP_HEAD, OP_PYTHON,
    // pieces of the above by themselves, for exec_part only (the interpreter's kernel wrappers)
    OP_LINEAR, OP_ATTEND, OP_KINDS
};

struct ExecOp {
    i64 kind;
    const void* params;     // the kind's parameter struct below
};

struct EmbedParams { const void* table; i64 dtype; };                  // x = table[ids]
struct RmsNormParams { const void* w; i64 dtype; double eps; };        // x += pending; y = rms_norm(x) * w
struct ShortConvParams {
    ExecLinear in_proj, out_proj;
    const void* in_proj_tiled; i64 tiled_rows;      // in_proj in tiles of 42 channels for the fused decode kernel (null: none)
    const void* taps; const void* bias; i64 taps_dtype, n_taps;
};
struct AttentionParams {
    ExecLinear qkv, out_proj;
    i64 nh, nkv, hd, window; double scale;
    const void* q_norm_w; const void* k_norm_w; i64 qk_dtype; double qk_eps;
    i64 rot, interleaved; const void* inv_freq;     // rot = 0 with inv_freq null: no rotation
};
struct SwiGLUParams {
    ExecLinear gate_up, down;
    i64 ff, fused;      // fused: gate_up holds interleaved gate and up blocks for the product's SwiGLU epilogue
};
struct HeadParams { ExecLinear w; };                                   // logits = y . w^T in 32-bit
struct PythonParams { i64 token; };                                    // the interpreter's name for the part
struct LinearParams { ExecLinear w; i64 lda, out_dtype; };             // out [T, N] = in [T, K] (row pitch lda) . w^T
// OP_ATTEND takes AttentionParams and reads only nh, nkv, hd, window and scale: out = attention of the queries `in`
// [T, nh * hd] (normed, turned) over the item's pages.

struct ExecOps { i64 n; const ExecOp* ops; };

// The registers as a Python part sees and changes them.
struct ExecRegs {
    void* x;
    const void* pending;
    void* y;
    void* logits;       // [R, V] float, epilogue only
    i64 phase;          // 0 prologue, 1 layers, 2 epilogue (rows = the wanted rows only)
    i64 item;           // index in the run order (phase 1)
};
// Runs the part `token`; may replace pending and y. Returns 0, or non-zero after an error the caller keeps.
typedef i64 (*PythonOpFn)(i64 token, ExecRegs* regs);

// Entry points of the kernel libraries, in the order of ExecProgram::fns.
enum ExecFn {
    FN_EMBED, FN_ADD_RMSNORM, FN_RESIDUAL_ADD, FN_SWIGLU, FN_SHORT_CONV, FN_QK_NORM_ROPE, FN_ATTENTION_PLAIN, FN_GEMM_PLAIN,
    FN_ATTENTION_DECODE, FN_ATTENTION_TC, FN_ATTENTION_FLASH, FN_GEMM_TCGEN05, FN_GEMM_CONV, FN_GEMM_ROPE, FN_COUNT
};

struct ExecProgram {
    i64 n_layers, n_order, H, V, act_dtype;
    i64 sms, static_flag, max_counters;
    i64 fused_conv, fused_rope;     // decode steps: in_proj + convolution, q/k/v product + norm + rotation as one kernel each
    i64 tc_min_ctas;                // prompt attention on tcgen05 from this many CTAs (< 0: an eighth of the SMs)
    double tc_min_fill;             // and this share of its tiles' rows in use
    ExecOps prologue, epilogue;
    const ExecOps* layers;          // [n_layers]
    const i64* order;               // [n_order]: the layer each item of the run order runs
    PythonOpFn python;
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
    i64 launches;               // out: kernels launched by native records
    i64 calls[FN_COUNT];        // out: calls of each entry point
};

// What the step needs, found by walking it without a launch: need[0] bytes of arena, need[1] floats of
// the products' workspace, need[2] floats of the attention workspace. Also sets s.launches.
void exec_need(const ExecProgram& p, ExecStep& s, i64* need);
// Runs the step. 0, or throws with the failing kernel's status in the message.
int exec_forward(const ExecProgram& p, ExecStep& s);
// One record of a mixer or feed-forward (or OP_LINEAR, OP_ATTEND) by itself: reads y_in, writes out (for a mixer or
// feed-forward both [T, H] of the activations' element type); the cache is s.items[0]. With dry set nothing is launched and need[] is filled as by exec_need.
int exec_part(const ExecProgram& p, ExecStep& s, const ExecOp& op, const void* y_in, void* out, bool dry, i64* need);

// The tile shape and K split of a product of M tokens by N weight rows over K.
void plan_tiles(i64 M, i64 N, i64 K, i64 sms, i64* bn, i64* split);

}  // namespace cellm
