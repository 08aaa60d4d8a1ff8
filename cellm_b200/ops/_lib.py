"""ctypes bindings to the compiled kernels. A missing or unbuildable library
raises at first use; there is no fallback to another implementation."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc import build as _build

P, I, L, F = c_void_p, c_int, c_longlong, c_float

DTYPE_TAG = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {-1: "unsupported element type", -2: "a size this kernel does not take",
           -3: "a pointer or stride breaks an alignment rule", -4: "missing or contradictory argument"}

_SIGNATURES = {
    "kernels_common": {
        "cellm_embed": [P, P, I, P, I, I, I, P, P],
        "cellm_upload": [P, P, L, P],
        "cellm_add_rmsnorm": [P, P, P, I, P, P, I, I, F, I, P],
        "cellm_residual_add": [P, P, L, I, P],
        "cellm_swiglu": [P, P, I, I, I, I, P],
        "cellm_short_conv": [P, P, P, P, I, P, L, P, P, P, I, I, I, I, I, I, I, P, P],
        "cellm_qk_norm_rope": [P, P, L, P, P, I, F, P, P, P, I, P, P, I, I, I, I, I, I, I, I, P, I, P, P],
        "cellm_attention_plain": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P],
        "cellm_argmax": [P, P, I, I, P, P],
        "cellm_take_pending_tokens": [P, P, P, P, I, I, P, P],
        "cellm_keep_last_tokens": [P, P, P, I, I, P],
        "cellm_sample": [P, P, I, I, P, P, P, P, P, I, I, P, P],
    },
    "gemm_plain": {
        "cellm_gemm_plain": [P, P, P, I, I, I, L, L, L, I, I, P],
    },
    "attention_decode": {
        "cellm_attention_decode": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, P],
    },
    "attention_tc": {
        "cellm_attention_tc": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P],
        "cellm_attention_tc_supports": [I, I, I, I],
    },
    "attention_flash": {
        "cellm_attention_flash": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, I, P, P],
        "cellm_attention_flash_supports": [I],
    },
    "gemm_tcgen05": {
        "cellm_gemm_tcgen05": [P, P, P, I, I, I, L, L, L, I, I, I, I, I, P, P, P, P],
        "cellm_gemm_conv_tcgen05": [P, P, P, I, I, I, L, L, I, I, I, P, P, I, P, L, P, I, I, P, P],
        "cellm_gemm_rope_tcgen05": [P, P, P, I, I, L, L, I, I, P, P, F, P, P, I, P, P, I, I, I, I, P, I, P, P],
    },
}

_funcs: dict[str, ctypes._CFuncPtr] = {}

# Kernels launched through these bindings since the process began: every entry
# point launches one kernel unless listed here.
LAUNCHES = [0]
_KERNELS_PER_CALL = {}


def count_launch(n: int = 1) -> None:
    LAUNCHES[0] += n


def register_signatures(library: str, signatures: dict) -> None:
    _SIGNATURES.setdefault(library, {}).update(signatures)


def fn(library: str, name: str):
    f = _funcs.get(name)
    if f is None:
        lib = _build.load(library)
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[library][name]
        f.restype = c_int
        _funcs[name] = f
    return f


def check(code: int, name: str) -> None:
    if code == 0:
        LAUNCHES[0] += _KERNELS_PER_CALL.get("cellm_" + name, 1)
        return
    if code < 0:
        raise ValueError(f"{name}: refused: {_ERRORS.get(code, code)}")
    raise RuntimeError(f"{name}: CUDA error {code} at launch")


def ptr(t):
    return None if t is None else t.data_ptr()


def tag(t_or_dtype) -> int:
    dt = t_or_dtype if isinstance(t_or_dtype, torch.dtype) else t_or_dtype.dtype
    try:
        return DTYPE_TAG[dt]
    except KeyError:
        raise ValueError(f"element type {dt} is not supported by the kernels") from None


# The raw handle of the current stream, asked from torch's C layer where that entry point exists: the Python
# wrapper (torch.cuda.current_stream) costs about 8 us a call, which every launch would pay.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_of(t: torch.Tensor) -> int:
    if _raw_stream is not None:
        return _raw_stream(t.device.index or 0)
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("kernel arguments must be contiguous CUDA tensors "
                             f"(got device={t.device}, contiguous={t.is_contiguous()})")
