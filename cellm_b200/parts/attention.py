"""Grouped-query attention mixer over the paged cache
(crates/cellm-model/src/lfm.rs:418-601): q, k, v projections, RMSNorm of every
q and k head, position encoding, keys and values written to the request's
pages, softmax(q.k * scale) over all earlier keys (or a window), out_proj."""
from __future__ import annotations

import os

import torch

from .. import ops
from ..config.errors import ConfigError
from ..config.plan import PartSpec
from .base import CacheBinding, Mixer, PagedKV, StepContext, TensorSpec
from .linear import Linear, stack_rows
from .registry import part_class, register_mixer


class AttentionMixer(Mixer):
    graph_safe = True

    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window,
    qk_norm (PartSpec of a norm over head_dim, or None), position (PartSpec or None).
    weights: q_proj [nh*hd, H], k_proj, v_proj [nkv*hd, H], out_proj [H, nh*hd],
    q_norm, k_norm [hd] if qk_norm."""

    can_read_foreign_cache = True

    @classmethod
    def weight_specs(cls, params):
        H, nh, nkv, hd = params["hidden_size"], params["num_heads"], params["num_kv_heads"], params["head_dim"]
        specs = {"q_proj": TensorSpec((nh * hd, H), "linear"), "k_proj": TensorSpec((nkv * hd, H), "linear"),
                 "v_proj": TensorSpec((nkv * hd, H), "linear"), "out_proj": TensorSpec((H, nh * hd), "linear")}
        if params.get("qk_norm") is not None:
            specs["q_norm"] = TensorSpec((hd,), "norm")
            specs["k_norm"] = TensorSpec((hd,), "norm")
        return specs

    @classmethod
    def cache_need(cls, params):
        return PagedKV(int(params["num_kv_heads"]), int(params["head_dim"]), int(params.get("window", 0)))

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.nh, self.nkv, self.hd = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if self.nh % self.nkv:
            raise ConfigError(f"attention: {self.nh} heads are not a multiple of {self.nkv} key/value heads")
        self.scale = float(params["scale"])
        self.window = int(params.get("window", 0))
        self.dtype = dtype
        dev = weights["q_proj"].device
        self.qkv = Linear(stack_rows(weights["q_proj"], weights["k_proj"], weights["v_proj"]), dtype)
        self.q_only = Linear(self.qkv.weight[:self.nh * self.hd], dtype)   # rows of the stacked matrix, no copy
        self.out_proj = Linear(weights["out_proj"], dtype)
        qk: PartSpec | None = params.get("qk_norm")
        self.q_norm_w = self.k_norm_w = None
        self.norm_eps = 0.0
        if qk is not None:
            if qk.kind != "rms_norm":
                raise ConfigError(f"attention: head norm of kind {qk.kind!r}; the fused kernel takes 'rms_norm'")
            self.norm_eps = float(qk.params["eps"])
            self.q_norm_w = weights["q_norm"].contiguous()
            self.k_norm_w = weights["k_norm"].to(self.q_norm_w.dtype).contiguous()
        pos: PartSpec | None = params.get("position")
        self.position = part_class("position", pos.kind)(pos.params, dev) if pos is not None else None

    def _fused_rope_ok(self, x, ctx, cache, rot) -> bool:
        """One token per request, bfloat16 throughout, heads of 64 turned whole in the "half" layout, own cache.
        Asked for with CELLM_B200_FUSED_ROPE=1: the kernel is tested, its effect on a step's time is not measured yet."""
        bf = torch.bfloat16
        return (ctx.max_q_len == 1 and cache.writes and self.hd == 64 and x.dtype == bf and self.qkv.weight.dtype == bf
                and self.q_norm_w is not None and self.q_norm_w.dtype == bf and rot is not None
                and rot[0] == 64 and not rot[1] and cache.k.dtype == bf
                and os.environ.get("CELLM_B200_FUSED_ROPE", "0") == "1" and ops.tensor_core_ok(x, self.qkv.weight))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        nh, nkv, hd = self.nh, (self.nkv if cache.writes else 0), self.hd
        rot = self.position.rotation() if self.position is not None else (0, False, None)
        bt, kp, vp = (cache.block_table, cache.k, cache.v) if nkv else (None, None, None)
        if self._fused_rope_ok(x, ctx, cache, rot):
            # decode steps: the product, the heads' norm, the rotation and the cache write as one kernel
            from ..ops import gemm_bf16 as tc
            plan = tc.gemm_rope_plan(ctx.T, nh, nkv, hd, x.shape[1], x.device)
            if plan is not None:
                q = tc.gemm_rope_bf16(x, self.qkv.weight, self.q_norm_w, self.k_norm_w, self.norm_eps, ctx.positions,
                                      bt, kp, vp, nh, nkv, rot[2], plan, ctx.err)
                o = ops.attention(q, cache.k, cache.v, ctx, cache.block_table, nh, self.scale, self.window)
                return self.out_proj(o)
        qkv = self.qkv(x) if cache.writes else self.q_only(x)
        if rot is not None:
            rotary_dim, interleaved, inv_freq = rot
            q = ops.qk_norm_rope(qkv, self.q_norm_w, self.k_norm_w, self.norm_eps, ctx.positions,
                                 ctx.seq_of_token, bt, kp, vp, cache.page_size, nh, nkv, hd, rotary_dim,
                                 interleaved, inv_freq, ctx.err)
        else:
            # A position encoding that is no rotation the fused kernel knows: head norms,
            # the part's own apply(), then the write into the pages, as three steps.
            q = ops.qk_norm_rope(qkv[:, :nh * hd], self.q_norm_w, self.q_norm_w, self.norm_eps, ctx.positions,
                                 ctx.seq_of_token, None, None, None, cache.page_size, nh, 0, hd, 0, False,
                                 None, ctx.err)
            k = None
            if nkv:
                k = ops.qk_norm_rope(qkv[:, nh * hd:(nh + nkv) * hd], self.k_norm_w, self.k_norm_w, self.norm_eps,
                                     ctx.positions, ctx.seq_of_token, None, None, None, cache.page_size, nkv, 0,
                                     hd, 0, False, None, ctx.err)
            q, k = self.position.apply(q.view(-1, nh, hd), k.view(-1, nkv, hd) if nkv else None, ctx.positions)
            q = q.reshape(-1, nh * hd).contiguous()
            if nkv:
                kv = torch.cat([k.reshape(-1, nkv * hd), qkv[:, (nh + nkv) * hd:]], dim=1).contiguous()
                ops.qk_norm_rope(kv, None, None, 0.0, ctx.positions, ctx.seq_of_token, bt, kp, vp,
                                 cache.page_size, 0, nkv, hd, 0, False, None, ctx.err)
        o = ops.attention(q, cache.k, cache.v, ctx, cache.block_table, nh, self.scale, self.window)
        return self.out_proj(o)


register_mixer("attention", AttentionMixer)
