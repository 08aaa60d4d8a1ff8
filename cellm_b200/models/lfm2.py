"""LFM2 as a plan: which parts make each layer and which file tensors they read.

Tensor names are the ones the reference reads
(crates/cellm-model/src/lfm.rs:333, :356, :374, :410, :422-424, :488, :516,
:596, :615, :634, :641, :658, :671, :744). Everything numeric comes from the
configuration; the parts themselves do not know they are in an LFM2.
"""
from __future__ import annotations

from ..config.lfm2 import Lfm2Config
from ..config.plan import LayerSpec, ModelPlan, OrderEntry, PartSpec
from ..config.registry import register_architecture


def _norm(cfg: Lfm2Config, dim: int, tensor: str) -> PartSpec:
    # One eps for every norm, the per-head ones included (crates/cellm-model/src/lfm.rs:144).
    return PartSpec("rms_norm", {"dim": dim, "eps": cfg.norm_eps}, {"weight": tensor})


def build_plan(cfg: Lfm2Config) -> ModelPlan:
    H, hd = cfg.hidden_size, cfg.head_dim
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        if cfg.is_attention(l):
            mixer = PartSpec(
                "attention",
                {"hidden_size": H, "num_heads": cfg.num_attention_heads,
                 "num_kv_heads": cfg.num_key_value_heads, "head_dim": hd,
                 # crates/cellm-cache/src/kvcache.rs:753: scores are scaled by 1/sqrt(head_dim);
                 # crates/cellm-model/src/lfm.rs:582-591 passes no window and no soft cap.
                 "scale": hd ** -0.5, "window": 0,
                 "qk_norm": _norm(cfg, hd, ""),
                 # crates/cellm-model/src/lfm.rs:553: rotary_dim = head_dim, rotate-half layout.
                 "position": PartSpec("rope", {"head_dim": hd, "rotary_dim": hd,
                                               "theta": cfg.rope_theta, "layout": "half"})},
                {"q_proj": p + "self_attn.q_proj.weight", "k_proj": p + "self_attn.k_proj.weight",
                 "v_proj": p + "self_attn.v_proj.weight", "out_proj": p + "self_attn.out_proj.weight",
                 "q_norm": p + "self_attn.q_layernorm.weight", "k_norm": p + "self_attn.k_layernorm.weight"})
        else:
            w = {"in_proj": p + "conv.in_proj.weight", "conv": p + "conv.conv.weight",
                 "out_proj": p + "conv.out_proj.weight"}
            if cfg.conv_bias:
                w["conv_bias"] = p + "conv.conv.bias"
            mixer = PartSpec("short_conv", {"hidden_size": H, "taps": cfg.conv_L_cache,
                                            "bias": cfg.conv_bias}, w)
        ffn = PartSpec("swiglu", {"hidden_size": H, "ff_dim": cfg.ff_dim},
                       {"w1": p + "feed_forward.w1.weight", "w3": p + "feed_forward.w3.weight",
                        "w2": p + "feed_forward.w2.weight"})
        layers.append(LayerSpec("pre_norm", mixer, ffn,
                                _norm(cfg, H, p + "operator_norm.weight"),
                                _norm(cfg, H, p + "ffn_norm.weight")))
    if cfg.layer_order is None:
        order = tuple(OrderEntry(l) for l in range(cfg.num_hidden_layers))
    else:
        order = tuple(OrderEntry(l, c) for l, c in cfg.layer_order)
    return ModelPlan(
        hidden_size=H, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding="model.embed_tokens.weight",
        final_norm=_norm(cfg, H, "model.embedding_norm.weight"),
        # The reference always reads the embedding for the output
        # (crates/cellm-model/src/lfm.rs:744); an untied head is read from lm_head.weight.
        head=None if cfg.tie_embedding else "lm_head.weight",
        layers=tuple(layers), order=order,
        eos_token_id=cfg.eos_token_id, bos_token_id=cfg.bos_token_id)


# tools/infer/src/main.rs:191 and tools/bench/src/main.rs:86 accept "lfm2" and "lfm".
register_architecture("Lfm2ForCausalLM", Lfm2Config, build_plan, model_types=("lfm2", "lfm"))
