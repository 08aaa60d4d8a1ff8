"""A decoder built from a plan: embedding, the layers in their run order, a
final norm on the rows whose logits are wanted, and the output product
(crates/cellm-model/src/lfm.rs:263-763 is the reference's forward for one
token; here one call serves every token of a step)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.errors import ConfigError
from ..config.plan import ModelPlan, PartSpec
from ..parts.base import CacheBinding, Residual, StepContext
from ..parts.linear import Linear
from ..parts.registry import part_class


def _weights_of(spec: PartSpec, tensors: dict) -> dict:
    return {local: tensors[name] for local, name in spec.weights.items() if name in tensors}


class DecoderModel:
    def __init__(self, plan: ModelPlan, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device):
        self.plan, self.dtype, self.device = plan, dtype, torch.device(device)
        self.embedding = tensors[plan.embedding]
        self.head = Linear(tensors[plan.head] if plan.head is not None else self.embedding, dtype)
        self.final_norm = part_class("norm", plan.final_norm.kind)(
            plan.final_norm.params, _weights_of(plan.final_norm, tensors), dtype)
        self.blocks = []
        self.mixer_classes = []
        for spec in plan.layers:
            mixer_cls = part_class("mixer", spec.mixer.kind)
            mixer = mixer_cls(spec.mixer.params, _weights_of(spec.mixer, tensors), dtype)
            ffn = part_class("feed_forward", spec.feed_forward.kind)(
                spec.feed_forward.params, _weights_of(spec.feed_forward, tensors), dtype)
            n1 = part_class("norm", spec.mixer_norm.kind)(spec.mixer_norm.params,
                                                         _weights_of(spec.mixer_norm, tensors), dtype)
            n2 = part_class("norm", spec.feed_forward_norm.kind)(spec.feed_forward_norm.params,
                                                                _weights_of(spec.feed_forward_norm, tensors), dtype)
            self.blocks.append(part_class("block", spec.block)(n1, mixer, n2, ffn))
            self.mixer_classes.append(mixer_cls)
        self.graph_safe = self.final_norm.graph_safe and all(
            b.graph_safe and b.mixer.graph_safe and b.feed_forward.graph_safe and b.mixer_norm.graph_safe
            and b.feed_forward_norm.graph_safe and getattr(getattr(b.mixer, "position", None), "graph_safe", True)
            for b in self.blocks)
        for i, e in enumerate(plan.order):
            if e.cache_of is not None:
                if not self.mixer_classes[e.layer].can_read_foreign_cache:
                    raise ConfigError(f"layer order item {i}: a {plan.layers[e.layer].mixer.kind!r} mixer "
                                      f"cannot read another item's cache")
                a, b = self.cache_need(i), self.cache_need(e.cache_of)
                if a != b:
                    raise ConfigError(f"layer order item {i} needs {a} but item {e.cache_of} keeps {b}")

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
        residual = Residual(ops.embed(self.embedding, ctx.token_ids, ctx.err))
        order = self.plan.order if max_layers is None else self.plan.order[:max_layers]
        for i, e in enumerate(order):
            self.blocks[e.layer].forward(residual, ctx, bindings[i])
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        xf = self.final_norm.forward(residual, rows=logit_rows)
        return self.head(xf, out_dtype=torch.float32)
