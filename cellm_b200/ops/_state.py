"""Per-device state the kernels share: the SM count, the tile counters of split kernels and the error word."""
from __future__ import annotations

import torch

MAX_COUNTERS = 65536
STATIC_WEIGHTS_FLAG = 1          # weights are static: their first loads may leave before the preceding kernel ends

_SM_COUNT: dict[int, int] = {}
_COUNTERS: dict[torch.device, torch.Tensor] = {}
_ERR: dict[torch.device, torch.Tensor] = {}


def sm_count(device) -> int:
    i = torch.device(device).index or 0
    if i not in _SM_COUNT:
        _SM_COUNT[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _SM_COUNT[i]


def counters(device) -> torch.Tensor:
    """Tile counters of split products and split attention: zero between kernels, shared by all kernels of one
    stream (each leaves them zero), never reallocated."""
    device = torch.device(device)
    c = _COUNTERS.get(device)
    if c is None:
        c = torch.zeros(MAX_COUNTERS, dtype=torch.int32, device=device)
        _COUNTERS[device] = c
    return c


def error_word(device) -> torch.Tensor:
    """The device error word the kernels report a bad index or a timed-out wait in."""
    device = torch.device(device)
    e = _ERR.get(device)
    if e is None:
        e = torch.zeros(1, dtype=torch.int32, device=device)
        _ERR[device] = e
    return e
