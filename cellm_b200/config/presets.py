"""Shapes of the LFM2 family as config.json dictionaries, for runs with random
weights (benchmarks and workloads; no checkpoint is read). The keys are the
architecture's own; the reference hard-codes the same attention layout for
LFM2-1.2B when a header lacks `layer_types`
(crates/cellm-model/src/lfm.rs:104-114)."""
from __future__ import annotations

_COMMON = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 65536, "num_key_value_heads": 8, "head_dim": 64,
    "block_auto_adjust_ff_dim": True, "block_multiple_of": 256, "block_ffn_dim_multiplier": 1.0,
    "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 128000,
}

LFM2_SHAPES = {
    # 16 layers, feed-forward 12288 -> 8192
    "lfm2-1.2b": dict(_COMMON, hidden_size=2048, num_hidden_layers=16, full_attn_idxs=[2, 5, 8, 10, 12, 14],
                      num_attention_heads=32, intermediate_size=12288),
    # 30 layers, feed-forward 10752 -> 7168
    "lfm2-2.6b": dict(_COMMON, hidden_size=2048, num_hidden_layers=30, full_attn_idxs=[2, 6, 10, 14, 18, 21, 24, 27],
                      num_attention_heads=32, intermediate_size=10752),
    # 16 layers, width 1536, feed-forward 10240 -> 6912
    "lfm2-700m": dict(_COMMON, hidden_size=1536, num_hidden_layers=16, full_attn_idxs=[2, 5, 8, 10, 12, 14],
                      num_attention_heads=24, intermediate_size=10240),
}


def shape(name: str) -> dict:
    try:
        return dict(LFM2_SHAPES[name.lower()])
    except KeyError:
        raise ValueError(f"unknown shape {name!r}; known: {sorted(LFM2_SHAPES)}") from None
