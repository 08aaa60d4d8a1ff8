"""Sampling options, with the names and meanings of tools/infer's flags
(tools/infer/src/main.rs:83-101) and of the reference engine's SamplingParams
(crates/cellm-sdk/src/lib.rs:100-116)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 0.8        # 0 = greedy
    top_k: int = 40                 # candidates kept when temperature > 0; 0 = the whole vocabulary
    seed: int = 1
    repeat_penalty: float = 1.05    # scores of recently seen tokens are divided by it; 1.0 disables
    repeat_window: int = 64
    max_new_tokens: int = 8         # tools/infer --gen
    stop_eos: bool = True

    def __post_init__(self):
        if self.top_k < 0 or self.top_k > 1024:
            raise ValueError("top_k must lie in 0..1024")
        if not 0 <= self.repeat_window <= 256:
            raise ValueError("repeat_window must lie in 0..256")
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")

    @classmethod
    def greedy(cls, max_new_tokens: int = 8, stop_eos: bool = True) -> "SamplingParams":
        return cls(temperature=0.0, top_k=0, repeat_penalty=1.0, max_new_tokens=max_new_tokens, stop_eos=stop_eos)
