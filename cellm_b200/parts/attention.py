"""Grouped-query attention mixer over the paged cache
(crates/cellm-model/src/lfm.rs:418-601): q, k, v projections, RMSNorm of every
q and k head, position encoding, keys and values written to the request's
pages, softmax(q.k * scale) over all earlier keys (or a window), out_proj."""
from __future__ import annotations

import torch

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
        self.H = int(params["hidden_size"])
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
                raise ConfigError(f"attention: head norm of kind {qk.kind!r}; the kernels take 'rms_norm'")
            self.norm_eps = float(qk.params["eps"])
            self.q_norm_w = weights["q_norm"].contiguous()
            self.k_norm_w = weights["k_norm"].to(self.q_norm_w.dtype).contiguous()
        pos: PartSpec | None = params.get("position")
        self.position = part_class("position", pos.kind)(pos.params, dev) if pos is not None else None
        self._record = self._attend = None

    def record(self):
        """The part as an op record of the native executor. None if its matrices are kept in another element type
        than the activations, or if its position encoding is no rotation the kernels apply (forward() then runs
        the head norms, the encoding's own apply() and the cache write as separate steps)."""
        from ..ops._lib import tag
        from ..runtime import records as R
        rot = self.position.rotation() if self.position is not None else (0, False, None)
        if self._record is None and rot is not None and self.qkv.weight.dtype == self.dtype == self.out_proj.weight.dtype:
            p = self._attend_params()
            p.qkv, p.out_proj = R.linear(self.qkv.weight), R.linear(self.out_proj.weight)
            if self.q_norm_w is not None:
                p.q_norm_w, p.k_norm_w = self.q_norm_w.data_ptr(), self.k_norm_w.data_ptr()
                p.qk_dtype, p.qk_eps = tag(self.q_norm_w), self.norm_eps
            p.rot, p.interleaved, p.inv_freq = int(rot[0]), int(rot[1]), R.ptr(rot[2])
            self._record = R.Record(R.ATTENTION, p, keep=[rot[2]], part=self)
        return self._record

    def _attend_params(self):
        from ..runtime import records as R
        p = R.AttentionParams()
        p.nh, p.nkv, p.hd, p.window, p.scale = self.nh, self.nkv, self.hd, self.window, self.scale
        return p

    def emit(self, emitter) -> None:
        rec = self.record()
        if rec is None:
            return super().emit(emitter)
        emitter.records.append(rec)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        from ..runtime import records as R
        from ..runtime.program import part_program
        rec = self.record()
        if rec is not None:
            return part_program(self.dtype, x.device, self.H).run_part(rec, x, ctx, cache)
        nh, nkv, hd = self.nh, (self.nkv if cache.writes else 0), self.hd
        bt, kp, vp = (cache.block_table, cache.k, cache.v) if nkv else (None, None, None)
        qkv = self.qkv(x) if cache.writes else self.q_only(x)
        rot = self.position.rotation() if self.position is not None else (0, False, None)
        if rot is not None:
            rotary_dim, interleaved, inv_freq = rot
            q = ops.qk_norm_rope(qkv, self.q_norm_w, self.k_norm_w, self.norm_eps, ctx.positions,
                                 ctx.seq_of_token, bt, kp, vp, cache.page_size, nh, nkv, hd, rotary_dim,
                                 interleaved, inv_freq, ctx.err)
        else:
            # A position encoding that is no rotation the kernels know: head norms,
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
        # the attention itself by the executor's choice of kernel
        if self._attend is None:
            self._attend = R.Record(R.ATTEND, self._attend_params(), part=self)
        o = torch.empty_like(q)
        part_program(q.dtype, q.device, self.H).run_part(self._attend, q, ctx, cache, out=o)
        return self.out_proj(o)


register_mixer("attention", AttentionMixer)
