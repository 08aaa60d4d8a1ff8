"""Python entry points of the hand-written kernels. Each function checks its
arguments, allocates its output with torch and launches on the current stream."""
from .basic import (embed, add_rmsnorm, residual_add, swiglu, short_conv, qk_norm_rope,
                    attention_plain, argmax, sample, upload, take_pending_tokens, keep_last_tokens)
from .gemm import gemm, gemm_plain
from .attention import attention
from .gemm_bf16 import gemm_swiglu_bf16, tensor_core_ok

__all__ = ["embed", "add_rmsnorm", "residual_add", "swiglu", "short_conv", "qk_norm_rope",
           "attention_plain", "argmax", "sample", "upload", "take_pending_tokens", "keep_last_tokens", "gemm", "gemm_plain", "attention", "gemm_swiglu_bf16", "tensor_core_ok"]
