"""Replays given tokens through the engine's own model, step function and
cache manager (used by bin/trace_run and by tests). Tokens are given, so no
sampling takes part (the nearest thing in the reference is `infer --tokens`,
tools/infer/src/main.rs:103-105)."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from .cache.manager import CacheManager
from .engine.step import StepEntry, StepRunner
from .models import load_model


class Replayer:
    def __init__(self, model_dir, dtype: str, max_tokens: int, tokens_per_block: int = 16,
                 max_requests: int = 4, device: str = "cuda:0", use_graphs: bool = True):
        """`model_dir`: a model folder, or the (config, plan, model) triple that
        `load_model` returned (several replays may share one loaded model).
        `max_tokens`: the most tokens live requests hold at any time, each
        request's count rounded up to a multiple of 64; the pools are made for
        exactly this many, so pages are used again.
        `use_graphs`: steps made of single tokens whose logits are wanted are replayed as CUDA
        graphs, as the engine's decode steps are; False launches every step kernel by kernel."""
        import torch
        if isinstance(model_dir, (str, bytes)) or hasattr(model_dir, "__fspath__"):
            model_dir = load_model(model_dir, dtype, device)
        self.cfg, self.plan, self.model = model_dir
        from .config import parse_dtype
        if self.model.dtype != parse_dtype(dtype):
            raise ValueError(f"the loaded model computes in {self.model.dtype}, the replay was asked for {dtype}")
        pages = max(1, (int(max_tokens) + tokens_per_block - 1) // tokens_per_block)
        needs = self.model.cache_needs()
        self.cache = CacheManager(needs, [e.cache_of for e in self.plan.order], tokens_per_block, pages,
                                  max_requests, self.model.dtype, device)
        self.runner = StepRunner(self.model, self.cache, use_graphs=use_graphs)
        self._ids: dict = {}
        self._next = 0
        self._torch = torch

    def _rid(self, name) -> int:
        if name not in self._ids:
            self._ids[name] = self._next
            self._next += 1
            self.cache.add(self._ids[name])
        return self._ids[name]

    def step(self, entries: Sequence[dict], end: Sequence = ()) -> Optional[np.ndarray]:
        """Runs one step; returns the wanted logits [wanted, vocab] float32 or None."""
        out = None
        if entries:
            batch = [StepEntry(self._rid(e["id"]), list(e["tokens"]), list(e.get("want", []))) for e in entries]
            logits = self.runner.run(batch)
            if logits is not None:
                out = logits.to("cpu").numpy()
            self.runner.check()
        for name in end:
            if name in self._ids:
                self.cache.release(self._ids.pop(name))
        return out
