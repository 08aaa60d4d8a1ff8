"""Loads a model's tensors from safetensors by name and checks them against
what the plan's parts declare, before anything is put on the GPU.

The reference reads tensors by their HF names from one mapped file and fails on
the first unknown name or wrong shape (crates/cellm-model/src/cellm_file.rs:
138-146, crates/cellm-model/src/lfm.rs:952-959, :894-900). Here all faults of a
file are collected into one error.

Element types: bfloat16 stays bfloat16; a tensor stored in 32-bit stays 32-bit;
float16 is converted to bfloat16; integer tables become int32. With
dtype=float32 every floating tensor is widened to float32 (exactly) so that the
whole model runs in 32-bit.
"""
from __future__ import annotations

import glob
import json
import os

import torch

from ..config.plan import ModelPlan, PartSpec
from ..parts.base import TensorSpec
from ..parts.registry import part_class
from .errors import WeightError
from .safetensors_io import SafetensorsFile


def _part_tensors(family: str, spec: PartSpec, out: dict[str, TensorSpec]) -> None:
    cls = part_class(family, spec.kind)
    for local, ts in cls.weight_specs(spec.params).items():
        name = spec.weights.get(local)
        if name is None:
            if ts.optional:
                continue
            raise WeightError(f"plan error: part {spec.kind!r} has no file tensor for its weight {local!r}")
        if name in out:
            if out[name].shape != ts.shape:
                raise WeightError(f"plan error: tensor {name!r} is used with shapes {out[name].shape} and {ts.shape}")
            continue        # a tensor two parts share (a tied head) keeps the first part's description
        out[name] = ts


def expected_tensors(plan: ModelPlan) -> dict[str, TensorSpec]:
    """File tensor name -> shape and value class, for every tensor the model reads."""
    out: dict[str, TensorSpec] = {}
    _part_tensors("embedding", plan.embedding, out)
    _part_tensors("head", plan.head, out)
    _part_tensors("norm", plan.final_norm, out)
    for layer in plan.layers:
        _part_tensors("norm", layer.mixer_norm, out)
        _part_tensors("mixer", layer.mixer, out)
        _part_tensors("norm", layer.feed_forward_norm, out)
        _part_tensors("feed_forward", layer.feed_forward, out)
    return out


def _open_files(folder: str) -> list[SafetensorsFile]:
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(single):
        paths = [single]
    elif os.path.isfile(index):
        with open(index) as f:
            paths = sorted({os.path.join(folder, p) for p in json.load(f)["weight_map"].values()})
    else:
        paths = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not paths:
        raise WeightError(f"no model.safetensors in {folder!r}")
    return [SafetensorsFile(p) for p in paths]


def _convert(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if t.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return t.to(torch.int32)
    if dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype == torch.float16:
        return t.to(torch.float32).to(torch.bfloat16)
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    raise WeightError(f"element type {t.dtype} cannot be used")


def load_weights(folder: str, plan: ModelPlan, dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    files = _open_files(folder)
    where: dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.names():
            where[name] = f
    want = expected_tensors(plan)
    missing = sorted(n for n in want if n not in where)
    unexpected = sorted(n for n in where if n not in want)
    wrong_shape, wrong_dtype = [], []
    for name, ts in want.items():
        f = where.get(name)
        if f is None:
            continue
        e = f.entries[name]
        if tuple(e.shape) != tuple(ts.shape):
            wrong_shape.append((name, tuple(e.shape), tuple(ts.shape)))
        if not e.dtype.is_floating_point or e.dtype == torch.float64:
            wrong_dtype.append((name, str(e.dtype)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        lines = [f"{folder}: the file's tensors do not match the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, got, exp in wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(exp)}")
        for name, dt in wrong_dtype:
            lines.append(f"  wrong element type: {name} is {dt}, expected bfloat16, float16 or float32")
        raise WeightError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype)
    out = {}
    for name in want:
        out[name] = _convert(where[name].tensor(name), dtype).to(device).contiguous()
    for f in files:
        f.close()
    return out
