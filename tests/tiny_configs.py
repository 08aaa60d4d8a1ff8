"""Two tiny LFM2 configurations that differ in every size and option, and
helpers that write them as model folders with random weights."""
import os

from cellm_b200.weights import InitSpec, write_random_model

TINY_A = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 512, "hidden_size": 64, "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 192, "block_auto_adjust_ff_dim": False,
    "rope_theta": 10000.0, "conv_L_cache": 3, "conv_bias": False, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 256, "eos_token_id": 7,
}

TINY_B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 1000, "hidden_size": 96, "num_hidden_layers": 6,
    "layer_types": ["conv", "conv", "full_attention", "conv", "full_attention", "full_attention"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 320, "block_auto_adjust_ff_dim": True, "block_multiple_of": 32,
    "block_ffn_dim_multiplier": 1.0,
    "rope_theta": 1000000.0, "conv_L_cache": 4, "conv_bias": True, "norm_eps": 1e-6,
    "tie_embedding": False, "max_position_embeddings": 512, "eos_token_id": 2,
}

# Layers of LFM2-1.2B's own sizes (width 2048, 32 query heads on 8 key/value heads of 64, feed-forward 12288
# adjusted to 8192, vocabulary 65536, three taps) in a model of four layers: the sizes at which the serving
# kernels take their large-tile, split and clustered forms, which the tiny configurations never reach.
FULL_WIDTH = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "block_ffn_dim_multiplier": 1.0, "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False,
    "norm_eps": 1e-5, "tie_embedding": True, "max_position_embeddings": 128000,
}
FULL_WIDTH_INIT = InitSpec(linear_std=0.03, embedding_std=0.03, conv_tap_std=0.3, norm_jitter=0.1)

CONFIGS = {"tiny_a": TINY_A, "tiny_b": TINY_B}
SEEDS = {"tiny_a": 11, "tiny_b": 23}

# Random weights of std 0.02 give logits so flat that a wrong key or a stale
# page barely moves them; tests use larger linears so that faults show, and a
# small embedding so that the tied output does not just repeat the last token.
TEST_INIT = InitSpec(linear_std=0.15, embedding_std=0.1, conv_tap_std=0.3, bias_std=0.05, norm_jitter=0.1)


def make_model(tmpdir, name, dtype="bfloat16", init=TEST_INIT, overrides=None, seed=None):
    cfg = dict(CONFIGS[name])
    if overrides:
        cfg.update(overrides)
    folder = os.path.join(str(tmpdir), f"{name}_{dtype}")
    return write_random_model(folder, cfg, SEEDS[name] if seed is None else seed, dtype, init)
