"""The forward pass of a step launched by the native runtime instead of Python.

A step that carries prompt tokens is some 150 kernel launches; from Python each
costs about ten microseconds of interpreter time. `NativeForward` describes the
model once to the runtime's executor (csrc/runtime/executor.cc), which then
walks the layers and launches the kernels in one foreign call per step, with
the decisions of the Python parts (which kernel, which tile shape). It serves
plans built from the parts this package ships; `unsupported()` says why a model
is not one of them, and such a model keeps the Python path.

The executor reaches the kernels through a table of entry points: the compiled
libraries' symbols on a GPU, or stand-ins given by a test.
"""
from __future__ import annotations

import ctypes
import importlib
import os
from ctypes import POINTER, Structure, c_double, c_longlong, c_void_p
from typing import Optional

import torch

from ..cache.native import CacheError, last_error, lib
from ..ops import _lib as klib
from ..ops import gemm_bf16 as tc
from ..parts.attention import AttentionMixer
from ..parts.block import PreNormBlock
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding
from ..parts.short_conv import ShortConvMixer
from ..parts.swiglu import SwiGLU

I64, F64, PTR = c_longlong, c_double, c_void_p


class ExecLinear(Structure):
    _fields_ = [("w", PTR), ("N", I64), ("K", I64), ("ldw", I64), ("dtype", I64), ("tc_ok", I64)]


class ExecLayer(Structure):
    _fields_ = [("kind", I64),
                ("norm1_w", PTR), ("norm1_dtype", I64), ("norm1_eps", F64),
                ("norm2_w", PTR), ("norm2_dtype", I64), ("norm2_eps", F64),
                ("gate_up", ExecLinear), ("down", ExecLinear), ("ff", I64), ("ff_fused", I64),
                ("in_proj", ExecLinear), ("conv_out", ExecLinear), ("in_proj_tiled", PTR), ("tiled_rows", I64),
                ("taps", PTR), ("conv_bias", PTR), ("taps_dtype", I64), ("n_taps", I64),
                ("qkv", ExecLinear), ("attn_out", ExecLinear), ("nh", I64), ("nkv", I64), ("hd", I64), ("window", I64),
                ("scale", F64), ("q_norm_w", PTR), ("k_norm_w", PTR), ("qk_dtype", I64), ("qk_eps", F64),
                ("rot", I64), ("interleaved", I64), ("inv_freq", PTR)]


# the kernel libraries' entry points in the order of the executor's table
ENTRY_POINTS = [("kernels_common", "cellm_embed"), ("kernels_common", "cellm_add_rmsnorm"), ("kernels_common", "cellm_swiglu"),
                ("kernels_common", "cellm_short_conv"), ("kernels_common", "cellm_qk_norm_rope"),
                ("kernels_common", "cellm_attention_plain"), ("gemm_plain", "cellm_gemm_plain"),
                ("attention_decode", "cellm_attention_decode"), ("attention_tc", "cellm_attention_tc"),
                ("attention_flash", "cellm_attention_flash"), ("gemm_tcgen05", "cellm_gemm_tcgen05"),
                ("gemm_tcgen05", "cellm_gemm_conv_tcgen05"), ("gemm_tcgen05", "cellm_gemm_rope_tcgen05")]


class ExecProgram(Structure):
    _fields_ = [("n_layers", I64), ("n_order", I64), ("H", I64), ("V", I64), ("act_dtype", I64),
                ("sms", I64), ("static_flag", I64), ("cluster_reduce", I64), ("fused_rope", I64), ("max_counters", I64),
                ("tc_min_ctas", I64), ("tc_min_fill", F64),
                ("embedding", PTR), ("embedding_dtype", I64),
                ("final_w", PTR), ("final_dtype", I64), ("final_eps", F64),
                ("head", ExecLinear), ("layers", POINTER(ExecLayer)), ("order", POINTER(I64)),
                ("fns", PTR * len(ENTRY_POINTS))]


class ExecItem(Structure):
    _fields_ = [("k", PTR), ("v", PTR), ("block_table", PTR), ("bt_stride", I64), ("num_pages", I64), ("page_size", I64),
                ("writes", I64), ("state", PTR), ("slot_stride", I64), ("n_slots", I64)]


class ExecStep(Structure):
    _fields_ = [("T", I64), ("B", I64), ("R", I64), ("max_q_len", I64), ("max_total_len", I64), ("n_order", I64),
                ("ids", PTR), ("positions", PTR), ("seq_of_token", PTR), ("cu_seqlens", PTR), ("ctx_lens", PTR),
                ("slot_ids", PTR), ("rows", PTR), ("q_lens", POINTER(I64)), ("items", POINTER(ExecItem)),
                ("arena", PTR), ("arena_bytes", I64), ("logits", PTR), ("err", PTR), ("stream", PTR),
                ("gemm_ws", PTR), ("gemm_ws_floats", I64), ("attn_ws", PTR), ("attn_ws_floats", I64), ("counters", PTR),
                ("launches", I64)]


_bound = False


def _runtime():
    """The runtime library with the executor's functions typed; checks the structs' layout once."""
    global _bound
    l = lib()
    if not _bound:
        l.cellm_exec_sizeof.argtypes, l.cellm_exec_sizeof.restype = [ctypes.c_int], c_longlong
        l.cellm_exec_need.argtypes, l.cellm_exec_need.restype = [c_void_p, c_void_p, POINTER(I64)], ctypes.c_int
        l.cellm_exec_forward.argtypes, l.cellm_exec_forward.restype = [c_void_p, c_void_p], ctypes.c_int
        l.cellm_exec_plan_tiles.argtypes = [I64, I64, I64, I64, POINTER(I64)]
        l.cellm_exec_plan_tiles.restype = ctypes.c_int
        for which, cls in enumerate((ExecLinear, ExecLayer, ExecProgram, ExecItem, ExecStep)):
            if l.cellm_exec_sizeof(which) != ctypes.sizeof(cls):
                raise RuntimeError(f"native executor: {cls.__name__} is {ctypes.sizeof(cls)} bytes here and "
                                   f"{l.cellm_exec_sizeof(which)} in the runtime")
        _bound = True
    return l


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _linear(lin, rows: Optional[int] = None) -> ExecLinear:
    w = lin.weight
    ok = w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
    return ExecLinear(w.data_ptr(), rows if rows is not None else w.shape[0], w.shape[1], w.stride(0), klib.tag(w), int(ok))


def unsupported(model) -> Optional[str]:
    """Why the executor cannot run this model (None: it can). Exact types only: a part derived from a
    built-in one may do anything in its forward()."""
    if model.dtype not in (torch.bfloat16, torch.float32):
        return f"activations of {model.dtype}"
    if type(model.final_norm) is not RMSNorm:
        return f"a final norm of kind {type(model.final_norm).__name__}"
    lins = [model.head]
    for i, b in enumerate(model.blocks):
        if type(b) is not PreNormBlock:
            return f"layer {i}: a block of kind {type(b).__name__}"
        if type(b.mixer_norm) is not RMSNorm or type(b.feed_forward_norm) is not RMSNorm:
            return f"layer {i}: a norm that is no RMSNorm"
        if type(b.feed_forward) is not SwiGLU:
            return f"layer {i}: a feed-forward of kind {type(b.feed_forward).__name__}"
        lins += [b.feed_forward.gate_up, b.feed_forward.down]
        m = b.mixer
        if type(m) is ShortConvMixer:
            lins += [m.in_proj, m.out_proj]
        elif type(m) is AttentionMixer:
            lins += [m.qkv, m.out_proj]
            if m.position is not None and type(m.position) is not RotaryEmbedding:
                return f"layer {i}: a position encoding of kind {type(m.position).__name__}"
        else:
            return f"layer {i}: a mixer of kind {type(m).__name__}"
    if any(l.weight.dtype != model.dtype for l in lins):
        return "a weight matrix kept in another element type than the activations"
    return None


class NativeForward:
    def __init__(self, model, entry_points: Optional[list] = None, sms: Optional[int] = None):
        """`entry_points`: addresses for the executor's table in the order of ENTRY_POINTS (default: the compiled
        libraries' symbols, which loads, and if need be compiles, all of them). `sms`: the SM count the tile
        planning assumes (default: the device's)."""
        why = unsupported(model)
        if why:
            raise ValueError(f"the native executor does not run this model: {why}")
        self.model, self.device = model, model.device
        self._rt = _runtime()
        self._keep = []          # ctypes objects the program points to
        if entry_points is None:
            from ..csrc import build as _build
            entry_points = [ctypes.cast(getattr(_build.load(library), name), c_void_p).value for library, name in ENTRY_POINTS]
        attention = importlib.import_module("cellm_b200.ops.attention")
        self._policy = attention.TC_POLICY
        layers = (ExecLayer * len(model.blocks))()
        for L, b in zip(layers, model.blocks):
            self._describe(L, b)
        order = (I64 * len(model.plan.order))(*[e.layer for e in model.plan.order])
        p = ExecProgram()
        p.n_layers, p.n_order, p.H, p.V = len(layers), len(order), model.embedding.shape[1], model.embedding.shape[0]
        p.act_dtype = klib.tag(model.dtype)
        p.sms = sms if sms is not None else tc._sms(self.device)
        p.static_flag, p.cluster_reduce, p.max_counters = tc._STATIC_FLAG, int(tc._CLUSTER_REDUCE), tc.MAX_COUNTERS
        p.fused_rope = int(os.environ.get("CELLM_B200_FUSED_ROPE", "0") == "1")
        p.embedding, p.embedding_dtype = model.embedding.data_ptr(), klib.tag(model.embedding)
        fn = model.final_norm
        p.final_w, p.final_dtype, p.final_eps = fn.weight.data_ptr(), klib.tag(fn.weight), fn.eps
        p.head = _linear(model.head)
        p.layers, p.order = layers, order
        for i, a in enumerate(entry_points):
            p.fns[i] = a
        self._keep += [layers, order]
        self.program = p
        self._arena = self._gemm_ws = self._attn_ws = None
        self.last_launches = 0

    def _describe(self, L: ExecLayer, b) -> None:
        n1, n2, ff, m = b.mixer_norm, b.feed_forward_norm, b.feed_forward, b.mixer
        L.norm1_w, L.norm1_dtype, L.norm1_eps = n1.weight.data_ptr(), klib.tag(n1.weight), n1.eps
        L.norm2_w, L.norm2_dtype, L.norm2_eps = n2.weight.data_ptr(), klib.tag(n2.weight), n2.eps
        L.gate_up, L.down = _linear(ff.gate_up), _linear(ff.down)
        L.ff, L.ff_fused = ff.down.weight.shape[1], int(ff.fused)
        if type(m) is ShortConvMixer:
            L.kind = 0
            L.in_proj, L.conv_out = _linear(m.in_proj), _linear(m.out_proj)
            if m.in_proj_tiled is not None:
                L.in_proj_tiled, L.tiled_rows = m.in_proj_tiled.data_ptr(), m.in_proj_tiled.shape[0]
            L.taps, L.conv_bias = m.conv_w.data_ptr(), _ptr(m.conv_b)
            L.taps_dtype, L.n_taps = klib.tag(m.conv_w), m.taps
        else:
            L.kind = 1
            L.qkv, L.attn_out = _linear(m.qkv), _linear(m.out_proj)
            L.nh, L.nkv, L.hd, L.window, L.scale = m.nh, m.nkv, m.hd, m.window, m.scale
            if m.q_norm_w is not None:
                L.q_norm_w, L.k_norm_w = m.q_norm_w.data_ptr(), m.k_norm_w.data_ptr()
                L.qk_dtype, L.qk_eps = klib.tag(m.q_norm_w), m.norm_eps
            if m.position is not None:
                rot, interleaved, inv = m.position.rotation()
                L.rot, L.interleaved, L.inv_freq = rot, int(interleaved), _ptr(inv)

    def _grow(self, name: str, n: int, dtype) -> torch.Tensor:
        t = getattr(self, name)
        if t is None or t.numel() < n:
            t = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            setattr(self, name, t)
        return t

    def forward(self, ctx, bindings, logit_rows: Optional[torch.Tensor], max_layers: Optional[int] = None,
                stream: Optional[int] = None) -> Optional[torch.Tensor]:
        """As DecoderModel.forward: float32 logits [R, vocab] for the rows in `logit_rows`, or None."""
        p, model = self.program, self.model
        p.tc_min_ctas = -1 if self._policy["min_ctas"] is None else int(self._policy["min_ctas"])
        p.tc_min_fill = float(self._policy["min_fill"])
        n_order = p.n_order if max_layers is None else min(int(max_layers), p.n_order)
        R = 0 if logit_rows is None else int(logit_rows.numel())
        items = (ExecItem * max(n_order, 1))()
        for it, b in zip(items, bindings[:n_order]):
            it.writes = int(b.writes)
            if b.k is not None:
                it.k, it.v, it.block_table = b.k.data_ptr(), b.v.data_ptr(), b.block_table.data_ptr()
                it.bt_stride, it.num_pages, it.page_size = b.block_table.stride(0), b.k.shape[0], b.page_size
            if b.state is not None:
                it.state, it.slot_stride, it.n_slots = _ptr(b.state) if b.state.numel() else None, b.state.stride(0), b.state.shape[0]
        s = ExecStep()
        s.T, s.B, s.R, s.max_q_len, s.max_total_len, s.n_order = ctx.T, ctx.B, R, ctx.max_q_len, ctx.max_total_len, n_order
        s.ids, s.positions, s.seq_of_token = ctx.token_ids.data_ptr(), ctx.positions.data_ptr(), ctx.seq_of_token.data_ptr()
        s.cu_seqlens, s.ctx_lens, s.slot_ids = ctx.cu_seqlens.data_ptr(), ctx.ctx_lens.data_ptr(), ctx.slot_ids.data_ptr()
        s.rows = _ptr(logit_rows) if R else None
        q_lens = (I64 * ctx.B)(*ctx.q_lens)
        s.q_lens, s.items = q_lens, items
        s.err = ctx.err.data_ptr()
        s.stream = klib.stream_of(ctx.err) if stream is None else stream
        need = (I64 * 3)()
        if self._rt.cellm_exec_need(ctypes.byref(p), ctypes.byref(s), need) != 0:
            raise CacheError(last_error())
        arena = self._grow("_arena", need[0] + 256, torch.uint8)
        s.arena, s.arena_bytes = arena.data_ptr(), arena.numel()
        if need[1]:
            ws = self._grow("_gemm_ws", need[1], torch.float32)
            s.gemm_ws, s.gemm_ws_floats = ws.data_ptr(), ws.numel()
        if need[2]:
            ws = self._grow("_attn_ws", need[2], torch.float32)
            s.attn_ws, s.attn_ws_floats = ws.data_ptr(), ws.numel()
        s.counters = tc._counters(self.device).data_ptr()
        logits = torch.empty((R, p.V), dtype=torch.float32, device=self.device) if R else None
        s.logits = _ptr(logits)
        if self._rt.cellm_exec_forward(ctypes.byref(p), ctypes.byref(s)) != 0:
            raise RuntimeError(f"native executor: {last_error()}")
        self.last_launches = int(s.launches)
        klib.count_launch(self.last_launches)
        return logits
