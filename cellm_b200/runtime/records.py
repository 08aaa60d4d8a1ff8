"""The op records of the native executor (csrc/runtime/executor.h) as ctypes
structures, and what a part's emit() appends them to.

A part describes itself to the executor with one record: its kind and a
parameter struct that points at its weights. A part without a native record
emits a Python record instead, and the executor calls back into the
interpreter for that part alone.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_double, c_longlong, c_void_p
from typing import Optional

import torch

from ..ops import _lib as klib

I64, F64, PTR = c_longlong, c_double, c_void_p

# record kinds, in the order of the executor's OpKind
EMBED, RMS_NORM, SHORT_CONV, ATTENTION, SWIGLU, HEAD, PYTHON, LINEAR, ATTEND = range(9)


class ExecLinear(Structure):
    _fields_ = [("w", PTR), ("N", I64), ("K", I64), ("ldw", I64), ("dtype", I64), ("tc_ok", I64)]


class ExecOp(Structure):
    _fields_ = [("kind", I64), ("params", PTR)]


class EmbedParams(Structure):
    _fields_ = [("table", PTR), ("dtype", I64)]


class RmsNormParams(Structure):
    _fields_ = [("w", PTR), ("dtype", I64), ("eps", F64)]


class ShortConvParams(Structure):
    _fields_ = [("in_proj", ExecLinear), ("out_proj", ExecLinear), ("in_proj_tiled", PTR), ("tiled_rows", I64),
                ("taps", PTR), ("bias", PTR), ("taps_dtype", I64), ("n_taps", I64)]


class AttentionParams(Structure):
    _fields_ = [("qkv", ExecLinear), ("out_proj", ExecLinear), ("nh", I64), ("nkv", I64), ("hd", I64), ("window", I64),
                ("scale", F64), ("q_norm_w", PTR), ("k_norm_w", PTR), ("qk_dtype", I64), ("qk_eps", F64),
                ("rot", I64), ("interleaved", I64), ("inv_freq", PTR)]


class SwiGLUParams(Structure):
    _fields_ = [("gate_up", ExecLinear), ("down", ExecLinear), ("ff", I64), ("fused", I64)]


class HeadParams(Structure):
    _fields_ = [("w", ExecLinear)]


class PythonParams(Structure):
    _fields_ = [("token", I64)]


class LinearParams(Structure):
    _fields_ = [("w", ExecLinear), ("lda", I64), ("out_dtype", I64)]


class ExecOps(Structure):
    _fields_ = [("n", I64), ("ops", POINTER(ExecOp))]


class ExecRegs(Structure):
    _fields_ = [("x", PTR), ("pending", PTR), ("y", PTR), ("logits", PTR), ("phase", I64), ("item", I64)]


PythonOpFn = ctypes.CFUNCTYPE(c_longlong, c_longlong, POINTER(ExecRegs))

# the kernel libraries' entry points in the order of the executor's table (ExecFn)
ENTRY_POINTS = [("kernels_common", "cellm_embed"), ("kernels_common", "cellm_add_rmsnorm"), ("kernels_common", "cellm_residual_add"),
                ("kernels_common", "cellm_swiglu"), ("kernels_common", "cellm_short_conv"), ("kernels_common", "cellm_qk_norm_rope"),
                ("kernels_common", "cellm_attention_plain"), ("gemm_plain", "cellm_gemm_plain"),
                ("attention_decode", "cellm_attention_decode"), ("attention_tc", "cellm_attention_tc"),
                ("attention_flash", "cellm_attention_flash"), ("gemm_tcgen05", "cellm_gemm_tcgen05"),
                ("gemm_tcgen05", "cellm_gemm_conv_tcgen05"), ("gemm_tcgen05", "cellm_gemm_rope_tcgen05")]
# libraries a model whose activations are 32-bit never calls into (they need not be compiled for it)
BF16_ONLY_LIBRARIES = ("attention_decode", "attention_tc", "attention_flash", "gemm_tcgen05")


class ExecProgram(Structure):
    _fields_ = [("n_layers", I64), ("n_order", I64), ("H", I64), ("V", I64), ("act_dtype", I64),
                ("sms", I64), ("static_flag", I64), ("max_counters", I64), ("fused_conv", I64), ("fused_rope", I64),
                ("tc_min_ctas", I64), ("tc_min_fill", F64),
                ("prologue", ExecOps), ("epilogue", ExecOps), ("layers", POINTER(ExecOps)), ("order", POINTER(I64)),
                ("python", PythonOpFn), ("fns", PTR * len(ENTRY_POINTS))]


class ExecItem(Structure):
    _fields_ = [("k", PTR), ("v", PTR), ("block_table", PTR), ("bt_stride", I64), ("num_pages", I64), ("page_size", I64),
                ("writes", I64), ("state", PTR), ("slot_stride", I64), ("n_slots", I64)]


class ExecStep(Structure):
    _fields_ = [("T", I64), ("B", I64), ("R", I64), ("max_q_len", I64), ("max_total_len", I64), ("n_order", I64),
                ("ids", PTR), ("positions", PTR), ("seq_of_token", PTR), ("cu_seqlens", PTR), ("ctx_lens", PTR),
                ("slot_ids", PTR), ("rows", PTR), ("q_lens", POINTER(I64)), ("items", POINTER(ExecItem)),
                ("arena", PTR), ("arena_bytes", I64), ("logits", PTR), ("err", PTR), ("stream", PTR),
                ("gemm_ws", PTR), ("gemm_ws_floats", I64), ("attn_ws", PTR), ("attn_ws_floats", I64), ("counters", PTR),
                ("launches", I64), ("calls", I64 * len(ENTRY_POINTS))]


# in the order cellm_exec_sizeof() numbers them
LAYOUT_CHECKED = (ExecLinear, ExecOp, ExecProgram, ExecItem, ExecStep, ExecRegs, EmbedParams, RmsNormParams, ShortConvParams,
                  AttentionParams, SwiGLUParams, HeadParams, PythonParams, ExecOps, LinearParams)


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def linear(weight: torch.Tensor, rows: Optional[int] = None) -> ExecLinear:
    """A weight matrix [N, K] as the executor's products read it (`rows`: only its first rows)."""
    w = weight
    ok = w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
    return ExecLinear(w.data_ptr(), rows if rows is not None else w.shape[0], w.shape[1], w.stride(0), klib.tag(w), int(ok))


class Record:
    """One op record with what it points to kept alive."""

    def __init__(self, kind: int, params: Structure, keep=(), part=None, role: str = ""):
        self.kind, self.params, self.keep, self.part, self.role = kind, params, list(keep), part, role
        self.op = ExecOp(kind, ctypes.cast(ctypes.pointer(params), c_void_p).value)


class Emitter:
    """What a part's emit() appends its records to. `act_dtype` is the element type of the activations the records
    will work on: a part whose weights do not fit it emits a Python record (`python(role, part)`) instead."""

    def __init__(self, act_dtype: torch.dtype, tokens: list):
        self.act_dtype = act_dtype
        self.records: list[Record] = []
        self._tokens = tokens          # the program's list of (role, part) that Python records name by index

    def native(self, kind: int, params: Structure, keep=(), part=None) -> None:
        self.records.append(Record(kind, params, keep, part))

    def python(self, role: str, part) -> None:
        """`role`: "embedding", "norm", "mixer", "feed_forward", "block" or "head": which forward() the executor's
        call-back runs on the registers (see Program._python_op)."""
        self._tokens.append((role, part))
        self.records.append(Record(PYTHON, PythonParams(len(self._tokens) - 1), part=part, role=role))

    def fits(self, *weights: torch.Tensor) -> bool:
        """Whether matrices kept in these element types can be multiplied with the activations natively."""
        return all(w.dtype == self.act_dtype for w in weights)
