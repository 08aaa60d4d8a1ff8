"""Configuration: typed fields from config.json keys, derived sizes, errors, registry."""
import json

import pytest

import plain_lfm2 as plain
from cellm_b200.config import ConfigError, Lfm2Config, config_from_dict, load_config, registered_architectures
from tiny_configs import TINY_A, TINY_B


def test_tiny_configs_parse_and_differ_in_every_size():
    a, b = Lfm2Config.from_dict(TINY_A), Lfm2Config.from_dict(TINY_B)
    for f in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
              "head_dim", "ff_dim", "rope_theta", "conv_L_cache", "conv_bias", "norm_eps", "tie_embedding",
              "max_position_embeddings", "layer_types"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.ff_dim == 192 and b.ff_dim == 224
    assert a.attention_layers == (1, 3) and b.conv_layers == (0, 1, 3)


@pytest.mark.parametrize("inter,mult,expect", [(12288, 256, 8192), (10752, 256, 7168), (10240, 256, 6912), (320, 32, 224)])
def test_feed_forward_size_examples(inter, mult, expect):
    d = dict(TINY_B, intermediate_size=inter, block_multiple_of=mult, block_auto_adjust_ff_dim=True)
    assert Lfm2Config.from_dict(d).ff_dim == expect
    assert plain.feed_forward_size(d) == expect       # the plain implementation's own copy of the rule
    assert Lfm2Config.from_dict(dict(d, block_auto_adjust_ff_dim=False)).ff_dim == inter


def test_multiplier_and_defaults():
    d = dict(TINY_B, block_ffn_dim_multiplier=1.5)
    assert Lfm2Config.from_dict(d).ff_dim == 32 * -(-int(1.5 * int(2 * 320 / 3)) // 32)
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "norm_eps", "rope_theta", "conv_L_cache", "conv_bias", "tie_embedding")}
    c = Lfm2Config.from_dict(d)
    assert (c.head_dim, c.norm_eps, c.rope_theta, c.conv_L_cache, c.conv_bias, c.tie_embedding) == (16, 1e-5, 1e6, 3, False, True)
    assert Lfm2Config.from_dict(dict(d, rms_norm_eps=1e-6)).norm_eps == 1e-6
    assert Lfm2Config.from_dict(dict(d, tie_word_embeddings=False)).tie_embedding is False


def test_full_attn_idxs_gives_layer_types():
    d = {k: v for k, v in TINY_B.items() if k != "layer_types"}
    d["full_attn_idxs"] = [2, 4, 5]
    assert Lfm2Config.from_dict(d).layer_types == tuple(TINY_B["layer_types"])


@pytest.mark.parametrize("change,needle", [
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"layer_types": ["conv"]}, "layer_types has 1 items"),
    ({"layer_types": ["conv", "mamba", "conv", "conv"]}, "mamba"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"conv_L_cache": 0}, "conv_L_cache"),
    ({"layer_order": [0, {"layr": 1}]}, "layer_order"),
])
def test_bad_configs_are_refused_with_the_key_named(change, needle):
    d = dict(TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert needle in str(e.value)


def test_registry_resolves_by_architecture_then_model_type():
    assert "Lfm2ForCausalLM" in registered_architectures()
    cfg, plan = config_from_dict(TINY_A)
    assert isinstance(cfg, Lfm2Config) and len(plan.layers) == 4 and plan.tied
    d = dict(TINY_B)
    d.pop("architectures")
    cfg, plan = config_from_dict(dict(d, model_type="lfm"))
    assert plan.head.weights == {"weight": "lm_head.weight"} and not plan.tied
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"], model_type="llama"))
    assert "LlamaForCausalLM" in str(e.value) and "Lfm2ForCausalLM" in str(e.value)


def test_plan_carries_every_constant_and_the_order():
    cfg, plan = config_from_dict(dict(TINY_B, layer_order=[0, 1, 2, 2, {"layer": 4, "cache_of": 2}, 5]))
    att = plan.layers[2].mixer
    assert att.kind == "attention" and att.params["num_kv_heads"] == 1 and att.params["scale"] == 32 ** -0.5
    assert att.params["position"].params["theta"] == 1e6 and att.params["qk_norm"].params["eps"] == 1e-6
    conv = plan.layers[0].mixer
    assert conv.kind == "short_conv" and conv.params["taps"] == 4 and conv.params["bias"] is True
    assert [(e.layer, e.cache_of) for e in plan.order] == [(0, None), (1, None), (2, None), (2, None), (4, 2), (5, None)]
    with pytest.raises(ConfigError):
        config_from_dict(dict(TINY_B, layer_order=[0, {"layer": 2, "cache_of": 3}]))
    with pytest.raises(ConfigError):
        config_from_dict(dict(TINY_B, layer_order=[0, 9]))


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    cfg, _ = load_config(str(tmp_path))
    assert cfg.to_dict()["hidden_size"] == 64 and Lfm2Config.from_dict(cfg.to_dict()) == cfg
