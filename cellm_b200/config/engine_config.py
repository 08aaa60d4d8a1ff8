"""Sizes of the engine around a model (the reference's `EngineConfig`,
crates/cellm-sdk/src/lib.rs:18-54, keeps tokens_per_block, total_blocks and
the sampling defaults in one struct; sampling has a struct of its own here)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported; use bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not supported; use bfloat16 or float32") from None


@dataclass
class EngineConfig:
    tokens_per_block: int = 16        # page size in tokens (tools/infer --tokens-per-block)
    total_blocks: int = 256           # pages in every paged group (tools/infer --total-blocks)
    max_num_seqs: int = 64            # live requests = slots for fixed-size state
    max_batch_tokens: int = 2048      # token budget of one step
    prefill_chunk: int = 2048         # longest portion of one prompt in one step
    dtype: torch.dtype = torch.bfloat16
    device: str = "cuda:0"
    seed: int = 1
    use_cuda_graphs: bool = True
    # A decode step's shape (requests, block-table width bucket) is captured as a graph when it is met for this many
    # times; before that its steps are launched kernel by kernel (a capture costs several steps' time, and a batch
    # that shrinks as requests end meets many shapes once or twice).
    capture_after: int = 3
    # A captured decode step whose tokens are all arg-maxes leaves them on the device for the step after it, and the
    # engine plans and launches that step before it reads them (its own work runs beside the GPU's); step() then
    # returns a step's tokens one call later. False: every step's tokens are read before the next is planned.
    run_ahead: bool = True

    def __post_init__(self):
        self.dtype = parse_dtype(self.dtype)
        for n in ("tokens_per_block", "total_blocks", "max_num_seqs", "max_batch_tokens", "prefill_chunk", "capture_after"):
            if getattr(self, n) <= 0:
                raise ValueError(f"EngineConfig.{n} must be positive")
