"""A decoder built from a plan: embedding, the layers in their run order, a
final norm on the rows whose logits are wanted, and the output product
(crates/cellm-model/src/lfm.rs:263-763 is the reference's forward for one
token; here one call serves every token of a step).

The model holds the parts; the walk over them is the native executor's
(cellm_b200/runtime/program.py): each part has described itself to it with an
op record, and a step's forward pass is one foreign call."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.errors import ConfigError
from ..config.plan import ModelPlan, PartSpec
from ..parts.base import CacheBinding, StepContext
from ..parts.registry import part_class


def _weights_of(spec: PartSpec, tensors: dict) -> dict:
    return {local: tensors[name] for local, name in spec.weights.items() if name in tensors}


def _build(family: str, spec: PartSpec, tensors: dict, dtype):
    return part_class(family, spec.kind)(spec.params, _weights_of(spec, tensors), dtype)


class DecoderModel:
    def __init__(self, plan: ModelPlan, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device):
        self.plan, self.dtype, self.device = plan, dtype, torch.device(device)
        self.embedding = _build("embedding", plan.embedding, tensors, dtype)
        self.head = _build("head", plan.head, tensors, dtype)
        self.final_norm = _build("norm", plan.final_norm, tensors, dtype)
        self.blocks = []
        self.mixer_classes = []
        for spec in plan.layers:
            mixer = _build("mixer", spec.mixer, tensors, dtype)
            ffn = _build("feed_forward", spec.feed_forward, tensors, dtype)
            n1 = _build("norm", spec.mixer_norm, tensors, dtype)
            n2 = _build("norm", spec.feed_forward_norm, tensors, dtype)
            self.blocks.append(part_class("block", spec.block)(n1, mixer, n2, ffn))
            self.mixer_classes.append(type(mixer))
        # a decode step may be captured in a CUDA graph only if every part says that its forward() just launches
        every = [self.embedding, self.head, self.final_norm]
        for b in self.blocks:
            every += [b] + [getattr(b, n) for n in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm") if hasattr(b, n)]
            position = getattr(getattr(b, "mixer", None), "position", None)
            if position is not None:
                every.append(position)
        self.graph_safe = all(getattr(part, "graph_safe", False) for part in every)
        for i, e in enumerate(plan.order):
            if e.cache_of is not None:
                if not self.mixer_classes[e.layer].can_read_foreign_cache:
                    raise ConfigError(f"layer order item {i}: a {plan.layers[e.layer].mixer.kind!r} mixer "
                                      f"cannot read another item's cache")
                a, b = self.cache_need(i), self.cache_need(e.cache_of)
                if a != b:
                    raise ConfigError(f"layer order item {i} needs {a} but item {e.cache_of} keeps {b}")
        self.program = None         # the model as records of the native executor, made at the first forward pass

    def cache_need(self, item: int):
        """What the cache of order item `item` must hold (also for items that borrow one)."""
        spec = self.plan.layers[self.plan.order[item].layer].mixer
        return self.mixer_classes[self.plan.order[item].layer].cache_need(spec.params)

    def cache_needs(self) -> list:
        """Per order item: its need, or None when it has no cache of its own."""
        return [None if e.cache_of is not None else self.cache_need(i) for i, e in enumerate(self.plan.order)]

    def forward(self, ctx: StepContext, bindings: list[CacheBinding], logit_rows: Optional[torch.Tensor],
                max_layers: Optional[int] = None) -> Optional[torch.Tensor]:
        """Runs the step's T tokens through all layers; returns float32 logits
        [R, vocab] for the rows in `logit_rows` (None: no logits are formed).
        `max_layers` runs only the first items of the order (tools/infer's
        --max-layers, crates/cellm-model/src/lfm.rs:179-181)."""
        if self.program is None:
            from ..runtime.program import Program
            self.program = Program(self)
        if logit_rows is not None and logit_rows.numel() == 0:
            logit_rows = None
        return self.program.forward(ctx, bindings, logit_rows, max_layers)
