"""Typed configuration of the LFM2 architecture, read from config.json keys.

The reference keeps nine numbers in `ModelConfig`
(crates/cellm-model/src/lib.rs:15-26) and looks up `layer_types` and
`conv_L_cache` loosely (crates/cellm-model/src/lfm.rs:95-122). Here every key
the model needs is a typed field. Keys the reference's readers give a default
keep that default; a size has none and must be present.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from .errors import ConfigError

_MISSING = object()


def _get(d: dict, key: str, typ, default=_MISSING, alt: Optional[str] = None):
    if key in d and d[key] is not None:
        v = d[key]
    elif alt is not None and alt in d and d[alt] is not None:
        v, key = d[alt], alt
    elif default is not _MISSING:
        return default
    else:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    if typ is float and isinstance(v, (int, float)) and not isinstance(v, bool):
        return float(v)
    if typ is int and isinstance(v, float) and v == int(v):
        v = int(v)
    if not isinstance(v, typ) or (typ is int and isinstance(v, bool)):
        raise ConfigError(f"config.json: key {key!r} should be {typ.__name__}, got {v!r}")
    return v


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    block_auto_adjust_ff_dim: bool
    block_multiple_of: int
    block_ffn_dim_multiplier: float
    norm_eps: float
    rope_theta: float
    conv_L_cache: int
    conv_bias: bool
    tie_embedding: bool
    layer_types: tuple[str, ...]
    max_position_embeddings: int
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    # Engine extension, absent from LFM2's own config.json: the order in which
    # layers run. Items are a layer index or {"layer": i, "cache_of": j}.
    layer_order: Optional[tuple] = None

    ATTENTION_NAMES = ("full_attention", "attention")   # crates/cellm-model/src/lfm.rs:418
    CONV_NAME = "conv"

    @classmethod
    def from_dict(cls, d: dict) -> "Lfm2Config":
        n_layers = _get(d, "num_hidden_layers", int)
        hidden = _get(d, "hidden_size", int)
        heads = _get(d, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive")
        if "layer_types" in d and d["layer_types"] is not None:
            lt = d["layer_types"]
            if not isinstance(lt, list) or not all(isinstance(s, str) for s in lt):
                raise ConfigError("config.json: layer_types should be a list of strings")
            layer_types = tuple(lt)
        elif "full_attn_idxs" in d and d["full_attn_idxs"] is not None:
            idx = d["full_attn_idxs"]
            if not isinstance(idx, list) or not all(isinstance(i, int) for i in idx):
                raise ConfigError("config.json: full_attn_idxs should be a list of integers")
            if any(not 0 <= i < n_layers for i in idx):
                raise ConfigError(f"config.json: full_attn_idxs {idx} outside 0..{n_layers - 1}")
            layer_types = tuple("full_attention" if i in set(idx) else "conv" for i in range(n_layers))
        else:
            raise ConfigError("config.json: neither layer_types nor full_attn_idxs is given")
        order = d.get("layer_order")
        if order is not None:
            if not isinstance(order, list):
                raise ConfigError("config.json: layer_order should be a list")
            norm = []
            for it in order:
                if isinstance(it, int) and not isinstance(it, bool):
                    norm.append((it, None))
                elif isinstance(it, dict) and isinstance(it.get("layer"), int):
                    norm.append((it["layer"], it.get("cache_of")))
                else:
                    raise ConfigError(f"config.json: layer_order item {it!r} is neither an index "
                                      f"nor {{'layer': i, 'cache_of': j}}")
            order = tuple(norm)
        cfg = cls(
            vocab_size=_get(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=_get(d, "num_key_value_heads", int, default=heads),
            # crates/cellm-model/src/lfm.rs:130-142: the header's value, else H / heads
            # (the reference's guess from k_proj's rows is not taken over).
            head_dim=_get(d, "head_dim", int, default=hidden // heads),
            intermediate_size=_get(d, "intermediate_size", int, alt="block_ff_dim"),
            block_auto_adjust_ff_dim=_get(d, "block_auto_adjust_ff_dim", bool, default=False),
            block_multiple_of=_get(d, "block_multiple_of", int, default=256),
            block_ffn_dim_multiplier=_get(d, "block_ffn_dim_multiplier", float, default=1.0),
            # tools/convert_lfm.py:173 reads rms_norm_eps or 1e-5.
            norm_eps=_get(d, "norm_eps", float, default=1e-5, alt="rms_norm_eps"),
            # tools/convert_lfm.py:174 defaults rope_theta to 1e6.
            rope_theta=_get(d, "rope_theta", float, default=1e6),
            # crates/cellm-model/src/lfm.rs:117-122 defaults conv_L_cache to 3.
            conv_L_cache=_get(d, "conv_L_cache", int, default=3),
            conv_bias=_get(d, "conv_bias", bool, default=False),
            tie_embedding=_get(d, "tie_embedding", bool, default=True, alt="tie_word_embeddings"),
            layer_types=layer_types,
            max_position_embeddings=_get(d, "max_position_embeddings", int),
            eos_token_id=_get(d, "eos_token_id", int, default=None),
            bos_token_id=_get(d, "bos_token_id", int, default=None),
            pad_token_id=_get(d, "pad_token_id", int, default=None),
            layer_order=order,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        def positive(name):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive, got {getattr(self, name)}")
        for n in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "intermediate_size", "block_multiple_of",
                  "conv_L_cache", "max_position_embeddings"):
            positive(n)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotate-half RoPE")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError(f"config.json: layer_types has {len(self.layer_types)} items for "
                              f"{self.num_hidden_layers} layers")
        for i, t in enumerate(self.layer_types):
            if t != self.CONV_NAME and t not in self.ATTENTION_NAMES:
                # crates/cellm-model/src/lfm.rs:602-606 rejects an unknown kind.
                raise ConfigError(f"config.json: layer_types[{i}] = {t!r}; known kinds are "
                                  f"'conv', 'full_attention', 'attention'")
        if self.norm_eps <= 0 or self.rope_theta <= 0 or self.block_ffn_dim_multiplier <= 0:
            raise ConfigError("config.json: norm_eps, rope_theta and block_ffn_dim_multiplier must be positive")

    @property
    def ff_dim(self) -> int:
        """Width of the SwiGLU hidden layer. The reference takes it from the
        weights (tools/convert_lfm.py:150-159); here it follows the config:
        two thirds of intermediate_size, times the multiplier, rounded up to
        block_multiple_of, when block_auto_adjust_ff_dim is set."""
        ff = self.intermediate_size
        if self.block_auto_adjust_ff_dim:
            ff = int(2 * ff / 3)
            ff = int(self.block_ffn_dim_multiplier * ff)
            m = self.block_multiple_of
            ff = m * ((ff + m - 1) // m)
        return ff

    def is_attention(self, layer: int) -> bool:
        return self.layer_types[layer] in self.ATTENTION_NAMES

    @property
    def attention_layers(self) -> tuple[int, ...]:
        return tuple(i for i in range(self.num_hidden_layers) if self.is_attention(i))

    @property
    def conv_layers(self) -> tuple[int, ...]:
        return tuple(i for i in range(self.num_hidden_layers) if not self.is_attention(i))

    def to_dict(self) -> dict:
        d = asdict(self)
        d["layer_types"] = list(self.layer_types)
        if self.layer_order is None:
            del d["layer_order"]
        else:
            d["layer_order"] = [l if c is None else {"layer": l, "cache_of": c}
                                for l, c in self.layer_order]
        for k in ("eos_token_id", "bos_token_id", "pad_token_id"):
            if d[k] is None:
                del d[k]
        d["architectures"] = ["Lfm2ForCausalLM"]
        d["model_type"] = "lfm2"
        return d
