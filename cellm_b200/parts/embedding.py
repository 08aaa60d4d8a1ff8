"""The two ends of the model: the token embedding that starts the residual
stream (crates/cellm-model/src/lfm.rs:817-890: a row of the table, no scaling)
and the output product that turns the last normed rows into logits
(:689-757; the reference always reads the embedding table for it)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, TensorSpec
from .linear import Linear
from .registry import register_embedding, register_head


class TokenEmbedding(Embedding):
    graph_safe = True

    """params: vocab_size, dim. weights: weight [vocab, dim]."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": TensorSpec((params["vocab_size"], params["dim"]), "embedding")}

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.weight = weights["weight"].contiguous()

    def emit(self, emitter) -> None:
        from ..ops._lib import tag
        from ..runtime import records as R
        emitter.native(R.EMBED, R.EmbedParams(self.weight.data_ptr(), tag(self.weight)), part=self)

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        return ops.embed(self.weight, token_ids, ctx.err)


class LinearHead(Head):
    graph_safe = True

    """params: vocab_size, dim. weights: weight [vocab, dim] (the embedding's tensor when the two are tied)."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": TensorSpec((params["vocab_size"], params["dim"]), "linear")}

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.linear = Linear(weights["weight"], dtype)
        self.weight = self.linear.weight

    def emit(self, emitter) -> None:
        from ..runtime import records as R
        if not emitter.fits(self.weight):
            return super().emit(emitter)
        emitter.native(R.HEAD, R.HeadParams(R.linear(self.weight)), part=self)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear(x, out_dtype=torch.float32)


register_embedding("lookup", TokenEmbedding)
register_head("linear", LinearHead)
