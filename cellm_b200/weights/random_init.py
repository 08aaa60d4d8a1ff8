"""Random-weights mode: writes a model folder (config.json, model.safetensors)
from a configuration and a seed. The reference has no such mode; the value
classes follow its tensors: linears and embeddings N(0, std), convolution taps
N(0, tap_std), biases N(0, bias_std), norm weights 1 + U(-jitter, jitter).

Every tensor has a generator of its own, seeded from the seed and the tensor's
name, so a tensor's values do not depend on which other tensors exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass

import torch

from ..config.engine_config import parse_dtype
from ..config.registry import config_from_dict
from .loader import expected_tensors
from .safetensors_io import save_file


@dataclass(frozen=True)
class InitSpec:
    linear_std: float = 0.02
    embedding_std: float = 0.02
    conv_tap_std: float = 0.1
    bias_std: float = 0.02
    norm_jitter: float = 0.1


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensor(name: str, shape, init: str, seed: int, spec: InitSpec) -> torch.Tensor:
    g = _generator(seed, name)
    if init == "norm":
        return 1.0 + (torch.rand(shape, generator=g, dtype=torch.float32) * 2.0 - 1.0) * spec.norm_jitter
    std = {"linear": spec.linear_std, "embedding": spec.embedding_std, "conv_tap": spec.conv_tap_std,
           "bias": spec.bias_std}[init]
    return torch.randn(shape, generator=g, dtype=torch.float32) * std


def write_random_model(folder: str, config: dict, seed: int = 0, dtype="bfloat16",
                       init: InitSpec = InitSpec()) -> str:
    """Creates `folder` with config.json and model.safetensors; returns the folder.
    `dtype` is the element type the tensors are stored in."""
    store = parse_dtype(dtype)
    cfg, plan = config_from_dict(config)
    tensors = {}
    for name, ts in expected_tensors(plan).items():
        tensors[name] = random_tensor(name, ts.shape, ts.init, seed, init).to(store)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict() if hasattr(cfg, "to_dict") else config, f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"),
              {"format": "pt", "seed": seed, "generator": "cellm_b200.weights.random_init"})
    return folder
