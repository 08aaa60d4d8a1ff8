#include "executor.h"

#include <algorithm>
#include <stdexcept>
#include <string>

namespace cellm {

namespace {

// ---- signatures of the kernel libraries' entry points (P = pointer, I = int, L = long long, F = float)
typedef void* P;
typedef const void* CP;
typedef int (*EmbedFn)(P out, CP table, int tag, CP ids, int T, int H, int V, P err, P stream);
typedef int (*AddRmsnormFn)(P x, CP delta, CP w, int w_tag, P y, CP rows, int n, int H, float eps, int act_tag, P stream);
typedef int (*ResidualAddFn)(P x, CP delta, i64 n, int act_tag, P stream);
typedef int (*SwigluFn)(P h, CP gu, int T, int ff, int tag, int gu_tag, P stream);
typedef int (*ShortConvFn)(P y, CP bcx, CP w, CP bias, int w_tag, P state, i64 slot_stride, CP slot_ids, CP seq, CP cu, int T,
                           int B, int H, int taps, int n_slots, int max_q_len, int act_tag, P err, P stream);
typedef int (*QkNormRopeFn)(P q, CP qkv, i64 row_stride, CP q_w, CP k_w, int w_tag, float eps, CP positions, CP seq, CP bt,
                            int bt_stride, P kp, P vp, int num_pages, int page_size, int T, int nh, int nkv, int hd, int rot,
                            int interleaved, CP inv_freq, int act_tag, P err, P stream);
typedef int (*AttentionPlainFn)(P out, CP q, CP kp, CP vp, CP positions, CP seq, CP bt, int bt_stride, int pages, int page_size,
                                int T, int nh, int nkv, int hd, float scale, int window, int tag, P err, P stream);
typedef int (*GemmPlainFn)(P c, CP a, CP w, int M, int N, int K, i64 lda, i64 ldw, i64 ldc, int a_tag, int out_tag, P stream);
typedef int (*AttentionDecodeFn)(P out, P part_o, P part_ml, P counters, CP q, CP kp, CP vp, CP cu, CP ctx, CP bt, int bt_stride,
                                 int B, int T, int pages, int page_size, int nh, int nkv, int hd, float scale, int window,
                                 int nsplit, P err, P stream);
typedef int (*AttentionTcFn)(P out, CP q, CP kp, CP vp, CP cu, CP ctx, CP bt, int bt_stride, int B, int T, int n_tiles, int pages,
                             int page_size, int nh, int nkv, int hd, float scale, int window, P err, P stream);
typedef int (*AttentionFlashFn)(P out, P part_o, P part_ml, CP q, CP kp, CP vp, CP cu, CP ctx, CP bt, int bt_stride, int B, int T,
                                int n_tiles, int pages, int page_size, int nh, int nkv, int hd, float scale, int window, int wide,
                                int nsplit, P err, P stream);
typedef int (*GemmTcFn)(P c, CP a, CP w, int M, int N, int K, i64 lda, i64 ldw, i64 ldc, int out_tag, int bn, int split_k,
                        int epilogue, int w_is_static, P ws, P counters, P err, P stream);
typedef int (*GemmConvFn)(P y, CP a, CP wt, int M, int Nt, int K, i64 lda, i64 ldw, int H, int bn, int split_k, CP taps, CP bias,
                          int ntaps, P state, i64 slot_stride, CP slot_ids, int n_slots, int w_is_static, P err, P stream);
typedef int (*GemmRopeFn)(P q, CP a, CP w, int M, int K, i64 lda, i64 ldw, int bn, int split_k, CP q_w, CP k_w, float eps,
                          CP positions, CP bt, int bt_stride, P kp, P vp, int pages, int page_size, int nh, int nkv, CP inv_freq,
                          int w_is_static, P err, P stream);


struct KernelError : std::runtime_error {
    int code;
    KernelError(const char* what, int c) : std::runtime_error(std::string(what) + ": status " + std::to_string(c)), code(c) {}
};

i64 ceil_div(i64 a, i64 b) { return (a + b - 1) / b; }
i64 elt(i64 dtype) { return dtype == EXEC_BF16 ? 2 : 4; }

i64 effective_split(i64 K, i64 split_k) {
    const i64 kblocks = ceil_div(K, 64);
    split_k = std::max<i64>(1, std::min(split_k, kblocks));
    const i64 per = ceil_div(kblocks, split_k);
    return ceil_div(kblocks, per);
}

// Bump allocation out of the step's arena: `x` and the two output slots live for the whole step, the rest of a
// half layer's buffers are given back when the next norm begins.
struct Arena {
    char* base;
    i64 size, top = 0, mark = 0, peak = 0;
    bool dry = false;       // sizes only: nothing is behind the addresses it hands out
    void* take(i64 bytes) {
        const i64 at = (top + 255) & ~(i64)255;
        if (!dry && at + bytes > size) throw std::runtime_error("executor: the step's arena is too small");
        top = at + bytes;
        peak = std::max(peak, top);
        return base + at;
    }
    void keep() { mark = top; }
    void release() { top = mark; }
};

struct Run {
    const ExecProgram& p;
    ExecStep& s;
    Arena arena;
    i64 act;        // element type of the activations
    bool dry = false;       // walk the step and note what it needs, launch nothing
    i64 launches = 0, need_gemm_ws = 0, need_attn_ws = 0;
    // the registers, and the two buffers that native parts leave their outputs in by turns
    ExecRegs regs{};
    void* slot[2] = {nullptr, nullptr};
    int turn = 0;

    ExecFn last_fn = FN_COUNT;
    template <typename F> F fn(ExecFn which) {
        if (!p.fns[which]) throw std::runtime_error("executor: entry point " + std::to_string((int)which) + " is not loaded");
        last_fn = which;
        return reinterpret_cast<F>(p.fns[which]);
    }
    void ok(int code, const char* what) {
        if (code != 0) throw KernelError(what, code);
        ++launches;
        if (last_fn < FN_COUNT) ++s.calls[last_fn];
    }
#define LAUNCH(call, what) ok(dry ? 0 : (call), what)

    // ---- products ------------------------------------------------------------------------------------------------
    bool tc_ok(const ExecLinear& l, i64 lda) const { return l.tc_ok && (l.K % 8) == 0 && (lda % 8) == 0; }

    void gemm_plain(void* c, const void* a, const ExecLinear& l, i64 M, i64 N, i64 lda, i64 out_dtype) {
        LAUNCH(fn<GemmPlainFn>(FN_GEMM_PLAIN)(c, a, l.w, (int)M, (int)N, (int)l.K, lda, l.ldw, N, (int)act, (int)out_dtype, s.stream),
           "gemm_plain");
    }

    // The tensor-core product with a given tile shape and split; c: [M, N] (or [M, N/2] with the SwiGLU epilogue).
    void gemm_tc(void* c, const void* a, const ExecLinear& l, i64 M, i64 N, i64 lda, i64 out_dtype, i64 bn, i64 split_k,
                 i64 epilogue) {
        const i64 split = effective_split(l.K, split_k);
        // swapped tiles whose K split is one thread-block cluster (2..8 CTAs) sum their pieces through shared
        // memory: no workspace, no counters
        const bool in_cluster = bn < 0 && ((split >= 2 && split <= 8) || (split == 1 && epilogue == 1));
        const bool through_ws = !in_cluster && (split > 1 || (epilogue == 1 && bn < 0));
        void* ws = nullptr;
        if (through_ws) {
            need_gemm_ws = std::max(need_gemm_ws, split * M * N);
            if (!dry && split * M * N > s.gemm_ws_floats) throw std::runtime_error("executor: the products' workspace is too small");
            ws = s.gemm_ws;
        }
        // plain tiles leave the sum of their K-split pieces to a second kernel; swapped tiles outside a cluster let
        // the last CTA of a tile sum them
        void* counters = (split > 1 && !in_cluster && bn < 0) ? s.counters : nullptr;
        LAUNCH(fn<GemmTcFn>(FN_GEMM_TCGEN05)(c, a, l.w, (int)M, (int)N, (int)l.K, lda, l.ldw, epilogue ? N / 2 : N, (int)out_dtype, (int)bn,
                                         (int)split_k, (int)epilogue, (int)p.static_flag, ws, counters, s.err, s.stream),
           "gemm_tcgen05");
        if (bn > 0 && split > 1) ++launches;          // the kernel that sums the K-split pieces
    }

    // a [M, K] (row pitch lda) . w^T -> c [M, N] of out_dtype
    void product(void* c, const void* a, const ExecLinear& l, i64 M, i64 lda, i64 out_dtype, i64 N = -1) {
        if (N < 0) N = l.N;
        if (l.dtype != act) throw std::runtime_error("executor: a weight whose element type differs from the activations'");
        if (act == EXEC_F32 || !tc_ok(l, lda)) {
            gemm_plain(c, a, l, M, N, lda, out_dtype);
        } else {
            i64 bn, split;
            plan_tiles(M, N, l.K, p.sms, &bn, &split);
            gemm_tc(c, a, l, M, N, lda, out_dtype, bn, split, 0);
        }
    }
    void* linear(const void* a, const ExecLinear& l, i64 M, i64 lda, i64 out_dtype, i64 N = -1) {
        void* c = arena.take(M * (N < 0 ? l.N : N) * elt(out_dtype));
        product(c, a, l, M, lda, out_dtype, N);
        return c;
    }

    // the plan of a decode product with an epilogue of its own, or false
    bool epilogue_plan(i64 M, i64 N, i64 K, i64* bn, i64* split) const {
        plan_tiles(M, N, K, p.sms, bn, split);
        return *bn < 0 && ceil_div(M, -*bn) == 1 && effective_split(K, *split) <= 8;
    }

    // ---- registers -----------------------------------------------------------------------------------------------
    // a part's output becomes the addend that waits; one that waits already goes into the stream first
    void set_pending(const void* out) {
        if (regs.pending)
            LAUNCH(fn<ResidualAddFn>(FN_RESIDUAL_ADD)(regs.x, regs.pending, s.T * p.H, (int)act, s.stream), "residual_add");
        regs.pending = out;
    }
    const void* input() const {
        if (!regs.y) throw std::runtime_error("executor: a part wants activations before any norm has left some");
        return regs.y;
    }

    void embed(const EmbedParams& e) {
        LAUNCH(fn<EmbedFn>(FN_EMBED)(regs.x, e.table, (int)e.dtype, s.ids, (int)s.T, (int)p.H, (int)p.V, s.err, s.stream), "embed");
    }
    void rms_norm(const RmsNormParams& n) {
        const bool rows = regs.phase == 2;
        arena.release();
        const i64 count = rows ? s.R : s.T;
        void* y = arena.take(count * p.H * elt(act));
        LAUNCH(fn<AddRmsnormFn>(FN_ADD_RMSNORM)(regs.x, regs.pending, n.w, (int)n.dtype, y, rows ? s.rows : nullptr, (int)count, (int)p.H,
                                            (float)n.eps, (int)act, s.stream),
           "add_rmsnorm");
        if (!rows) regs.pending = nullptr;      // with rows given the stream itself is not touched
        regs.y = y;
    }
    void head(const HeadParams& h) {
        if (regs.phase != 2) throw std::runtime_error("executor: the output product belongs to the epilogue");
        if (h.w.dtype != act) throw std::runtime_error("executor: a head whose element type differs from the activations'");
        product(regs.logits, input(), h.w, s.R, p.H, EXEC_F32);
    }
    void python(const PythonParams& py) {
        if (dry) return;
        if (!p.python) throw std::runtime_error("executor: a Python part in a program without a callback");
        if (p.python(py.token, &regs) != 0) throw std::runtime_error("executor: a Python part raised");
    }

    void feed_forward(const SwiGLUParams& L, const void* x, void* out);
    void short_conv(const ShortConvParams& L, const ExecItem& it, const void* x, void* out);
    void attention(const AttentionParams& L, const ExecItem& it, const void* x, void* out);
    void* attend(const AttentionParams& L, const ExecItem& it, const void* q, void* o = nullptr);

    // a mixer or feed-forward record: reads `in`, writes `out`
    void produce(const ExecOp& op, const ExecItem* it, const void* in, void* out) {
        switch (op.kind) {
            case OP_SHORT_CONV:
                if (!it) throw std::runtime_error("executor: a mixer outside the layers");
                short_conv(*static_cast<const ShortConvParams*>(op.params), *it, in, out);
                break;
            case OP_ATTENTION:
                if (!it) throw std::runtime_error("executor: a mixer outside the layers");
                attention(*static_cast<const AttentionParams*>(op.params), *it, in, out);
                break;
            case OP_SWIGLU: feed_forward(*static_cast<const SwiGLUParams*>(op.params), in, out); break;
            case OP_LINEAR: {
                const LinearParams& l = *static_cast<const LinearParams*>(op.params);
                product(out, in, l.w, s.T, l.lda, l.out_dtype);
                break;
            }
            case OP_ATTEND: {
                if (!it) throw std::runtime_error("executor: attention outside the layers");
                attend(*static_cast<const AttentionParams*>(op.params), *it, in, out);
                break;
            }
            default: throw std::runtime_error("executor: record kind " + std::to_string(op.kind) + " produces nothing");
        }
    }

    void run(const ExecOp& op) {
        const ExecItem* it = regs.phase == 1 ? &s.items[regs.item] : nullptr;
        switch (op.kind) {
            case OP_EMBED: embed(*static_cast<const EmbedParams*>(op.params)); break;
            case OP_RMS_NORM: rms_norm(*static_cast<const RmsNormParams*>(op.params)); break;
            case OP_HEAD: head(*static_cast<const HeadParams*>(op.params)); break;
            case OP_PYTHON: python(*static_cast<const PythonParams*>(op.params)); break;
            case OP_SHORT_CONV: case OP_ATTENTION: case OP_SWIGLU: {
                void* out = slot[turn];
                produce(op, it, input(), out);
                set_pending(out);
                turn ^= 1;
                break;
            }
            default: throw std::runtime_error("executor: unknown record kind " + std::to_string(op.kind));
        }
    }
    void run(const ExecOps& ops) {
        for (i64 i = 0; i < ops.n; ++i) run(ops.ops[i]);
    }
};

}  // namespace

void plan_tiles(i64 M, i64 N, i64 K, i64 sms, i64* bn_out, i64* split_out) {
    const i64 kblocks = ceil_div(K, 64);
    if (M <= 64) {
        // Swapped tiles: 128 weight rows by 16, 32 or 64 tokens. Enough CTAs to fill the SMs, and no CTA with much
        // more than ~300 KB of weights to stream by itself; at most 8 (the split of a tile is one thread-block
        // cluster) and at least four K blocks each. Products with tiles to spare are not split.
        const i64 narrow = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
        const i64 tiles = ceil_div(N, 128);
        i64 split;
        if (tiles >= 2 * sms) {
            split = 1;
        } else {
            const i64 fill = ceil_div(sms * 85 / 100, tiles);
            const i64 stream = ceil_div(128 * K * 2, 300 * 1024);
            split = std::max<i64>(1, std::min({std::max(fill, stream), kblocks / 4, (i64)8}));
        }
        *bn_out = -narrow;
        *split_out = split;
        return;
    }
    i64 bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
    if (bn == 256 && kblocks >= 64 && M > 256 && ceil_div(N, 256) * ceil_div(M, 128) < sms / 2) {
        // A long K (the feed-forward's way back), three row tiles or more, too few tiles of 128 x 256 for the SMs: those tiles stay, whose
        // products run nearer the tensor pipe's rate than narrower ones, and K is split until the SMs are filled; the
        // pieces go through the workspace and a second kernel sums them.
        const i64 t256 = ceil_div(N, 256) * ceil_div(M, 128);
        *bn_out = 256;
        *split_out = std::max<i64>(1, std::min({ceil_div(sms * 85 / 100, t256), kblocks / 4, (i64)16}));
        return;
    }
    if (bn == 256) {
        // The persistent kernel takes any width from 128 to 256 in steps of 16. A tile costs about 0.1 + 0.9 * width / 256
        // of a 256-wide one (a 128-wide one 0.55); the width whose waves finish soonest wins, the wider on a tie: it
        // is the one whose number of tiles comes closest to a multiple of the SMs from below.
        const i64 mt = ceil_div(M, 128);
        double best = 1e30;
        for (i64 w = 256; w >= 128; w -= 16) {
            const double cost = (double)ceil_div(mt * ceil_div(N, w), sms) * (0.1 + 0.9 * (double)w / 256.0);
            if (cost < best * 0.98) { best = cost; bn = w; }
        }
    }
    i64 tiles = ceil_div(N, bn) * ceil_div(M, 128);
    if (tiles < sms / 2) {
        // Too few plain tiles to fill the GPU (a few hundred tokens, or a narrow product).
        if (M <= 128) {
            // up to two token tiles: swapped tiles of 128 weight rows by 64 tokens, the K split summed in a cluster
            // (as for fewer tokens, no CTA with much more than ~300 KB of weights to stream by itself)
            const i64 stiles = ceil_div(N, 128) * ceil_div(M, 64);
            const i64 want = sms * 85 / 100;
            const i64 stream = ceil_div(128 * K * 2, 300 * 1024);
            *bn_out = -64;
            *split_out = stiles >= want ? 1 : std::max<i64>(1, std::min({std::max(ceil_div(want, stiles), stream), kblocks / 4, (i64)8}));
            return;
        }
        // more tokens: tiles of 128 x 128 with K split until the SMs are filled; the pieces go through the
        // workspace and a second kernel sums them
        bn = N > 64 ? 128 : 64;
        tiles = ceil_div(N, bn) * ceil_div(M, 128);
        *bn_out = bn;
        *split_out = std::max<i64>(1, std::min({ceil_div(sms * 85 / 100, tiles), kblocks / 4, (i64)16}));
        return;
    }
    *bn_out = bn;
    *split_out = 1;
}

namespace {

void Run::feed_forward(const SwiGLUParams& L, const void* x, void* out) {
    const i64 T = s.T, H = p.H;
    void* h;
    if (L.fused && act == EXEC_BF16 && tc_ok(L.gate_up, H)) {
        i64 bn, split;
        plan_tiles(T, L.gate_up.N, L.gate_up.K, p.sms, &bn, &split);
        if (bn == 64) bn = 128;
        else if (bn > 128 && bn < 256) bn = 256;       // gate and up blocks of 64: widths of 128 and 256 only
        h = arena.take(T * L.ff * elt(act));
        gemm_tc(h, x, L.gate_up, T, L.gate_up.N, H, act, bn, split, 1);
    } else if (L.fused) {
        throw std::runtime_error("executor: activations do not fit the fused SwiGLU kernel");
    } else {
        // gate and up stay in 32-bit until silu(g) * u is formed, as in the fused epilogue: one rounding, not three
        void* gu = linear(x, L.gate_up, T, H, EXEC_F32);
        h = arena.take(T * L.ff * elt(act));
        LAUNCH(fn<SwigluFn>(FN_SWIGLU)(h, gu, (int)T, (int)L.ff, (int)act, (int)EXEC_F32, s.stream), "swiglu");
    }
    product(out, h, L.down, T, L.ff, act);
}

void Run::short_conv(const ShortConvParams& L, const ExecItem& it, const void* x, void* out) {
    const i64 T = s.T, H = p.H;
    void* y = nullptr;
    if (p.fused_conv && L.in_proj_tiled && s.max_q_len == 1 && act == EXEC_BF16) {
        ExecLinear tiled = L.in_proj;
        tiled.w = L.in_proj_tiled;
        tiled.N = L.tiled_rows;
        tiled.ldw = L.in_proj.K;
        i64 bn, split;
        if (tc_ok(tiled, H) && epilogue_plan(T, L.tiled_rows, H, &bn, &split)) {
            y = arena.take(T * H * elt(act));
            LAUNCH(fn<GemmConvFn>(FN_GEMM_CONV)(y, x, L.in_proj_tiled, (int)T, (int)L.tiled_rows, (int)H, H, tiled.ldw, (int)H, (int)bn,
                                            (int)split, L.taps, L.bias, (int)L.n_taps, it.state, it.slot_stride, s.slot_ids,
                                            (int)it.n_slots, (int)p.static_flag, s.err, s.stream),
               "gemm_conv_tcgen05");
        }
    }
    if (!y) {
        void* bcx = linear(x, L.in_proj, T, H, act);
        y = arena.take(T * H * elt(act));
        LAUNCH(fn<ShortConvFn>(FN_SHORT_CONV)(y, bcx, L.taps, L.bias, (int)L.taps_dtype, it.state, it.slot_stride, s.slot_ids,
                                          s.seq_of_token, s.cu_seqlens, (int)T, (int)s.B, (int)H, (int)L.n_taps, (int)it.n_slots,
                                          (int)s.max_q_len, (int)act, s.err, s.stream),
           "short_conv");
        if (L.n_taps > 1 && !(s.max_q_len > 0 && s.max_q_len <= 4)) ++launches;     // the state update is a launch of its own
    }
    product(out, y, L.out_proj, T, H, act);
}

void* Run::attend(const AttentionParams& L, const ExecItem& it, const void* q, void* o) {
    const i64 T = s.T, nh = L.nh, nkv = L.nkv, hd = L.hd;
    if (!o) o = arena.take(T * nh * hd * elt(act));
    const float scale = (float)L.scale;
    if (act == EXEC_BF16 && (hd == 32 || hd == 64 || hd == 128) && L.scale > 0) {
        const i64 G = nh / nkv;
        if (s.max_q_len * G <= 16) {
            // decoded tokens: one CTA per (request, kv head, piece of the keys)
            const i64 blocks = ceil_div(s.max_total_len, 64);
            // Pieces of the keys: as many as fill four CTAs an SM, of four blocks of 64 keys or more. Where that asks for
            // more than one cluster of eight, pieces of two blocks and a multiple of eight of them: clusters of eight
            // combine their pieces in shared memory and only one piece a cluster goes through the workspace.
            const i64 fill = 4 * p.sms / (s.B * nkv);
            i64 nsplit = std::max<i64>(1, std::min(fill, blocks / 4));
            if (blocks / 4 > 8) nsplit = std::max<i64>(1, std::min(fill, blocks / 2));
            if (nsplit >= 16) nsplit = nsplit / 8 * 8;
            void *part_o = nullptr, *part_ml = nullptr, *counters = nullptr;
            if (nsplit > 8) {          // up to 8 pieces meet inside a thread-block cluster and need no workspace
                if (s.B * nkv > p.max_counters) throw std::runtime_error("executor: too many (request, kv head) pairs for the counters");
                const i64 rows = T * nh;
                need_attn_ws = std::max(need_attn_ws, nsplit * rows * (hd + 2));
                if (!dry && nsplit * rows * (hd + 2) > s.attn_ws_floats) throw std::runtime_error("executor: the attention workspace is too small");
                part_o = s.attn_ws;
                part_ml = (float*)s.attn_ws + nsplit * rows * hd;
                counters = s.counters;
            }
            LAUNCH(fn<AttentionDecodeFn>(FN_ATTENTION_DECODE)(o, part_o, part_ml, counters, q, it.k, it.v, s.cu_seqlens, s.ctx_lens,
                                                          it.block_table, (int)it.bt_stride, (int)s.B, (int)T, (int)it.num_pages,
                                                          (int)it.page_size, (int)nh, (int)nkv, (int)hd, scale, (int)L.window,
                                                          (int)nsplit, s.err, s.stream),
               "attention_decode");
            return o;
        }
        // prompt portions that fill the tcgen05 kernel's pairs of 128-row tiles and enough CTAs (below that the
        // mma.sync kernel with its split over the keys fills the GPU better)
        const i64 ps = it.page_size;
        if (hd == 64 && G <= 128 && 128 % G == 0 && (ps == 8 || ps == 16 || ps == 32 || ps == 64 || ps == 128)) {
            const i64 per_tile = 256 / G;
            i64 tc_tiles = 0;
            for (i64 b = 0; b < s.B; ++b) tc_tiles += ceil_div(s.q_lens[b], per_tile);
            const i64 min_ctas = p.tc_min_ctas < 0 ? p.sms / 8 : p.tc_min_ctas;
            if (tc_tiles * nkv >= min_ctas && (double)T >= p.tc_min_fill * (double)(tc_tiles * per_tile)) {
                LAUNCH(fn<AttentionTcFn>(FN_ATTENTION_TC)(o, q, it.k, it.v, s.cu_seqlens, s.ctx_lens, it.block_table, (int)it.bt_stride,
                                                      (int)s.B, (int)T, (int)tc_tiles, (int)it.num_pages, (int)ps, (int)nh, (int)nkv,
                                                      (int)hd, scale, (int)L.window, s.err, s.stream),
                   "attention_tc");
                return o;
            }
        }
        // How many CTAs share the keys of one tile: enough to fill the GPU when the batch alone does not, but at
        // least two blocks of 64 keys each.
        const bool wide = s.max_q_len * G > 16;
        const i64 bm = wide ? 64 : 16;
        i64 n_tiles = 0;
        for (i64 b = 0; b < s.B; ++b) n_tiles += ceil_div(s.q_lens[b] * G, bm);
        const i64 blocks = ceil_div(s.max_total_len, 64);
        const i64 target = ceil_div(4 * p.sms, n_tiles * nkv);
        const i64 nsplit = std::max<i64>(1, std::min(target, blocks / 2));
        void *part_o = nullptr, *part_ml = nullptr;
        if (nsplit > 1) {
            const i64 rows = T * nh;
            need_attn_ws = std::max(need_attn_ws, nsplit * rows * (hd + 2));
            if (!dry && nsplit * rows * (hd + 2) > s.attn_ws_floats) throw std::runtime_error("executor: the attention workspace is too small");
            part_o = s.attn_ws;
            part_ml = (float*)s.attn_ws + nsplit * rows * hd;
        }
        LAUNCH(fn<AttentionFlashFn>(FN_ATTENTION_FLASH)(o, part_o, part_ml, q, it.k, it.v, s.cu_seqlens, s.ctx_lens, it.block_table,
                                                    (int)it.bt_stride, (int)s.B, (int)T, (int)n_tiles, (int)it.num_pages, (int)ps,
                                                    (int)nh, (int)nkv, (int)hd, scale, (int)L.window, wide ? 1 : 0, (int)nsplit,
                                                    s.err, s.stream),
           "attention_flash");
        if (nsplit > 1) ++launches;                    // the merge of the pieces
        return o;
    }
    // 32-bit, other head sizes: one block per (token, head) over the block table
    LAUNCH(fn<AttentionPlainFn>(FN_ATTENTION_PLAIN)(o, q, it.k, it.v, s.positions, s.seq_of_token, it.block_table, (int)it.bt_stride,
                                                (int)it.num_pages, (int)it.page_size, (int)T, (int)nh, (int)nkv, (int)hd, scale,
                                                (int)L.window, (int)act, s.err, s.stream),
       "attention_plain");
    return o;
}

void Run::attention(const AttentionParams& L, const ExecItem& it, const void* x, void* out) {
    const i64 T = s.T, H = p.H, nh = L.nh, hd = L.hd;
    const i64 nkv = it.writes ? L.nkv : 0;
    void* q = nullptr;
    // decode steps, bfloat16, heads of 64 turned whole in the "half" layout, a cache of the item's own: the product,
    // the heads' norm, the rotation and the cache write as one kernel
    const bool rope_fused = p.fused_rope && s.max_q_len == 1 && it.writes && hd == 64 && act == EXEC_BF16 &&
                            L.qkv.dtype == EXEC_BF16 && L.q_norm_w && L.qk_dtype == EXEC_BF16 && L.rot == 64 && !L.interleaved &&
                            L.inv_freq && tc_ok(L.qkv, H);
    i64 bn, split;
    if (rope_fused && epilogue_plan(T, (nh + 2 * nkv) * hd, H, &bn, &split)) {
        q = arena.take(T * nh * hd * elt(act));
        LAUNCH(fn<GemmRopeFn>(FN_GEMM_ROPE)(q, x, L.qkv.w, (int)T, (int)H, H, L.qkv.ldw, (int)bn, (int)split, L.q_norm_w, L.k_norm_w,
                                        (float)L.qk_eps, s.positions, it.block_table, (int)it.bt_stride, it.k, it.v,
                                        (int)it.num_pages, (int)it.page_size, (int)nh, (int)nkv, L.inv_freq, (int)p.static_flag,
                                        s.err, s.stream),
           "gemm_rope_tcgen05");
    } else {
        const i64 width = (nh + 2 * nkv) * hd;
        void* qkv = linear(x, L.qkv, T, H, act, width);       // without a cache of its own: the query rows only
        q = arena.take(T * nh * hd * elt(act));
        LAUNCH(fn<QkNormRopeFn>(FN_QK_NORM_ROPE)(q, qkv, width, L.q_norm_w, L.k_norm_w, L.q_norm_w ? (int)L.qk_dtype : 0,
                                             (float)L.qk_eps, s.positions, s.seq_of_token, nkv ? it.block_table : nullptr,
                                             nkv ? (int)it.bt_stride : 0, nkv ? it.k : nullptr, nkv ? it.v : nullptr,
                                             nkv ? (int)it.num_pages : 0, (int)it.page_size, (int)T, (int)nh, (int)nkv, (int)hd,
                                             (int)L.rot, (int)L.interleaved, L.inv_freq, (int)act, s.err, s.stream),
           "qk_norm_rope");
    }
    void* o = attend(L, it, q);
    product(out, o, L.out_proj, T, nh * hd, act);
}

int walk(const ExecProgram& p, ExecStep& s, bool dry, i64* need) {
    Run r{p, s, Arena{static_cast<char*>(s.arena), s.arena_bytes}, p.act_dtype};
    r.dry = r.arena.dry = dry;
    const i64 T = s.T, H = p.H, e = elt(p.act_dtype);
    s.launches = 0;
    for (i64& c : s.calls) c = 0;
    if (T <= 0) return 0;
    if (s.n_order > p.n_order) throw std::runtime_error("executor: more order items than the program has");
    r.regs.x = r.arena.take(T * H * 4);
    r.slot[0] = r.arena.take(T * H * e);
    r.slot[1] = r.arena.take(T * H * e);
    r.arena.keep();
    r.regs.phase = 0;
    r.run(p.prologue);
    r.regs.phase = 1;
    for (i64 i = 0; i < s.n_order; ++i) {
        const i64 layer = p.order[i];
        if (layer < 0 || layer >= p.n_layers) throw std::runtime_error("executor: the run order names a layer the program lacks");
        r.regs.item = i;
        r.run(p.layers[layer]);
    }
    if (s.R > 0) {
        r.regs.phase = 2;
        r.regs.logits = s.logits;
        r.run(p.epilogue);
    }
    s.launches = r.launches;
    if (need) { need[0] = r.arena.peak; need[1] = r.need_gemm_ws; need[2] = r.need_attn_ws; }
    return 0;
}
}  // namespace

int exec_forward(const ExecProgram& p, ExecStep& s) { return walk(p, s, false, nullptr); }

void exec_need(const ExecProgram& p, ExecStep& s, i64* need) { walk(p, s, true, need); }

int exec_part(const ExecProgram& p, ExecStep& s, const ExecOp& op, const void* y_in, void* out, bool dry, i64* need) {
    Run r{p, s, Arena{static_cast<char*>(s.arena), s.arena_bytes}, p.act_dtype};
    r.dry = r.arena.dry = dry;
    s.launches = 0;
    for (i64& c : s.calls) c = 0;
    if (s.T > 0) {
        r.regs.phase = 1;
        r.produce(op, s.items, y_in, out);
    }
    s.launches = r.launches;
    if (need) { need[0] = r.arena.peak; need[1] = r.need_gemm_ws; need[2] = r.need_attn_ws; }
    return 0;
}

}  // namespace cellm
