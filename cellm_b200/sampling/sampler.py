"""Chooses next tokens on the device for the rows of a step's logits."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams
from .rng import XorShift64


class RequestSampler:
    """Per-request sampling state: options, random stream, and all tokens so far
    (the repetition window looks at prompt and generated tokens alike, as
    tools/infer's `all_ids` does, tools/infer/src/main.rs:458-465)."""

    def __init__(self, params: SamplingParams, seed: int, history: Sequence[int]):
        self.params = params
        self.rng = XorShift64(seed)
        self.history = list(history)


def sample_rows(logits: torch.Tensor, samplers: Sequence[RequestSampler],
                argmax: torch.Tensor | None = None) -> list[int]:
    """One token for each row of float32 logits [R, V]; advances the random
    stream of every request that samples with temperature. `argmax`: the rows'
    arg-max if the step has computed it already (int32 [R])."""
    R = logits.shape[0]
    assert R == len(samplers)
    if all(s.params.temperature <= 0.0 for s in samplers):
        return (argmax if argmax is not None and argmax.shape[0] == R else ops.argmax(logits)).tolist()
    W = max((s.params.repeat_window for s in samplers if s.params.repeat_penalty > 1.0), default=0)
    # one upload: temperature, uniform number, penalty (float32 bits), top_k, then the recent tokens
    buf = np.empty((4 * R + R * W,), dtype=np.int32)
    f = buf[:3 * R].view(np.float32).reshape(3, R)
    k = buf[3 * R:4 * R]
    recent = buf[4 * R:].reshape(R, W)
    recent.fill(-1)
    for r, s in enumerate(samplers):
        p = s.params
        f[0, r] = p.temperature
        f[1, r] = s.rng.next_f32() if p.temperature > 0.0 else 0.0
        f[2, r] = p.repeat_penalty
        k[r] = p.top_k
        if p.repeat_penalty > 1.0 and p.repeat_window > 0 and s.history:
            tail = s.history[-p.repeat_window:]
            recent[r, :len(tail)] = tail
    d = torch.from_numpy(buf).to(logits.device)
    fd = d[:3 * R].view(torch.float32).view(3, R)
    out = ops.sample(logits, fd[0], d[3 * R:4 * R], fd[1], fd[2], d[4 * R:].view(R, W) if W > 0 else None,
                     int(k.max()))
    return out.tolist()
