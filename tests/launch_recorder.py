"""Runs the package's Python side of a step without a GPU: the kernels' entry points are replaced by
recorders, so that a test can see which kernels a step of a given shape would launch and with which
sizes. Weights are zeros on the CPU; nothing is computed."""
import importlib

import numpy as np
import torch


class Recorder:
    def __init__(self, monkeypatch, sms: int = 148):
        """Patches (through `monkeypatch`, so that everything is put back) the look-up of the compiled
        entry points, the checks that operands lie on a GPU, the stream and SM queries."""
        from cellm_b200.ops import _lib, basic, gemm_bf16
        gemm = importlib.import_module("cellm_b200.ops.gemm")
        attention = importlib.import_module("cellm_b200.ops.attention")
        self.calls: list[tuple[str, dict]] = []
        sigs = _lib._SIGNATURES

        def fn(library, name):
            sig = sigs[library][name]

            def call(*args):
                assert len(args) == len(sig), f"{name}: {len(args)} arguments for a signature of {len(sig)}"
                self.calls.append((name, args))
                return 0
            return call
        for m in (_lib, basic, gemm, gemm_bf16, attention):
            for attr, value in (("fn", fn), ("require_cuda", lambda *a: None), ("stream_of", lambda t: 0)):
                if hasattr(m, attr):
                    monkeypatch.setattr(m, attr, value)
        monkeypatch.setattr(gemm_bf16, "_sms", lambda device: sms)
        monkeypatch.setitem(gemm_bf16._ERR, torch.device("cpu"), torch.zeros(1, dtype=torch.int32))
        monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
        monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True), raising=False)
        gemm_bf16.plan_tiles.cache_clear()

    def names(self) -> list[str]:
        return [n for n, _ in self.calls]

    def of(self, name: str) -> list[tuple]:
        return [a for n, a in self.calls if n == name]


def zero_model(config: dict, dtype=torch.bfloat16):
    """(typed config, plan, DecoderModel) with all-zero weights on the CPU."""
    from cellm_b200 import parts  # noqa: F401  (registers the built-in parts)
    from cellm_b200.config import config_from_dict
    from cellm_b200.models.decoder import DecoderModel
    from cellm_b200.weights.loader import expected_tensors
    cfg, plan = config_from_dict(config)
    tensors = {n: torch.zeros(ts.shape, dtype=dtype) for n, ts in expected_tensors(plan).items()}
    return cfg, plan, DecoderModel(plan, tensors, dtype, "cpu")


def run_step(model, plan, q_lens, ctx_lens, page: int = 16):
    """One step of entries with `q_lens` new tokens after `ctx_lens` cached ones; logits wanted at each entry's last token."""
    from cellm_b200.cache.manager import CacheManager
    from cellm_b200.parts.base import StepContext
    B, T = len(q_lens), sum(q_lens)
    width = max((c + q + page - 1) // page for c, q in zip(ctx_lens, q_lens)) + 1
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in plan.order], page, B * width + 4, B + 1, model.dtype, "cpu")
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    tables = []
    for g in range(len(cache.paged_keys)):
        tables.append(torch.full((B, width), -1, dtype=torch.int32))
    for b in range(B):
        cache.add(b)
        cache.reserve(b, ctx_lens[b] + q_lens[b])
        for g, t in enumerate(tables):
            cache.block_table(b, g, t[b].numpy())
    cu = [0] + [int(v) for v in np.cumsum(q_lens)]
    ctx = StepContext(T=T, B=B, dtype=model.dtype, device=torch.device("cpu"), token_ids=i32(list(range(T))),
                      positions=i32([c + j for c, q in zip(ctx_lens, q_lens) for j in range(q)]),
                      seq_of_token=i32([b for b, q in enumerate(q_lens) for _ in range(q)]), cu_seqlens=i32(cu),
                      ctx_lens=i32(list(ctx_lens)), slot_ids=i32([cache.slot(b) for b in range(B)]),
                      err=torch.zeros(1, dtype=torch.int32), q_lens=list(q_lens), ctx_lens_host=list(ctx_lens),
                      max_q_len=max(q_lens), max_total_len=max(c + q for c, q in zip(ctx_lens, q_lens)))
    return model.forward(ctx, cache.bindings(tables), i32([c - 1 for c in cu[1:]]))
