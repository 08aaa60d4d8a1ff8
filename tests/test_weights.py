"""Weights: the safetensors reader and writer, the loader's single error that
lists every fault, element types kept, and the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from cellm_b200.config import load_config
from cellm_b200.weights import SafetensorsFile, WeightError, expected_tensors, load_weights, save_file
from tiny_configs import make_model


def test_random_model_folder_is_readable_by_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file
    folder = make_model(tmp_path, "tiny_b")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    cfg, plan = load_config(folder)
    theirs = load_file(os.path.join(folder, "model.safetensors"))
    want = expected_tensors(plan)
    assert set(theirs) == set(want)
    assert "lm_head.weight" in want and "model.layers.0.conv.conv.bias" in want
    for name, ts in want.items():
        assert tuple(theirs[name].shape) == ts.shape and theirs[name].dtype == torch.bfloat16
    ours = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    for name in want:
        assert torch.equal(ours.tensor(name), theirs[name])


def test_reader_reads_what_the_library_writes(tmp_path):
    from safetensors.torch import save_file as their_save
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    their_save(t, str(tmp_path / "x.safetensors"))
    f = SafetensorsFile(str(tmp_path / "x.safetensors"))
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v)


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a = SafetensorsFile(os.path.join(make_model(tmp_path / "1", "tiny_a", seed=5), "model.safetensors"))
    b = SafetensorsFile(os.path.join(make_model(tmp_path / "2", "tiny_a", seed=5), "model.safetensors"))
    c = SafetensorsFile(os.path.join(make_model(tmp_path / "3", "tiny_a", seed=6), "model.safetensors"))
    n = "model.layers.1.self_attn.q_proj.weight"
    assert torch.equal(a.tensor(n), b.tensor(n)) and not torch.equal(a.tensor(n), c.tensor(n))
    w = a.tensor("model.layers.0.operator_norm.weight").float()
    assert (w - 1).abs().max() <= 0.1 + 1e-2 and (w - 1).abs().max() > 0


def test_element_types_are_kept(tmp_path):
    folder = make_model(tmp_path, "tiny_a")
    _, plan = load_config(folder)
    w = load_weights(folder, plan, torch.bfloat16, "cpu")
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    w32 = load_weights(folder, plan, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert all(torch.equal(w32[k], w[k].float()) for k in w)          # widening is exact
    # a tensor stored in 32-bit stays so in the bfloat16 mode; float16 becomes bfloat16
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    t["model.embedding_norm.weight"] = t["model.embedding_norm.weight"].float() + 1e-4
    t["model.layers.0.ffn_norm.weight"] = t["model.layers.0.ffn_norm.weight"].half()
    save_file(t, os.path.join(folder, "model.safetensors"))
    w = load_weights(folder, plan, torch.bfloat16, "cpu")
    assert w["model.embedding_norm.weight"].dtype == torch.float32
    assert w["model.layers.0.ffn_norm.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model(tmp_path, "tiny_b")
    _, plan = load_config(folder)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.2.self_attn.k_layernorm.weight"]
    del t["lm_head.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(3)
    t["model.layers.0.feed_forward.w1.weight"] = torch.zeros(320, 96).bfloat16()     # unadjusted width
    t["model.layers.1.conv.conv.weight"] = torch.zeros(96, 4).bfloat16()             # squeezed
    t["model.embed_tokens.weight"] = torch.zeros(1000, 96, dtype=torch.int32)
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        load_weights(folder, plan, torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.2.self_attn.k_layernorm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.0.feed_forward.w1.weight", "model.layers.1.conv.conv.weight"}
    assert [n for n, _ in err.wrong_dtype] == ["model.embed_tokens.weight"]
    msg = str(err)
    for needle in ("lm_head.weight", "extra.weight", "[320, 96]", "[224, 96]", "[96, 1, 4]"):
        assert needle in msg


def test_broken_files_are_refused(tmp_path):
    folder = make_model(tmp_path, "tiny_a")
    _, plan = load_config(folder)
    path = os.path.join(folder, "model.safetensors")
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[:len(blob) // 2])                                   # truncated
    with pytest.raises(WeightError, match="truncated|outside"):
        load_weights(folder, plan, torch.bfloat16, "cpu")
    open(path, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")                       # header longer than the file
    with pytest.raises(WeightError, match="header length"):
        load_weights(folder, plan, torch.bfloat16, "cpu")
    open(path, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(WeightError, match="JSON"):
        load_weights(folder, plan, torch.bfloat16, "cpu")
    os.unlink(path)
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_weights(folder, plan, torch.bfloat16, "cpu")


def test_sharded_folder_with_index(tmp_path):
    folder = make_model(tmp_path, "tiny_a")
    _, plan = load_config(folder)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    names = sorted(f.names())
    half = len(names) // 2
    save_file({n: f.tensor(n).clone() for n in names[:half]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file({n: f.tensor(n).clone() for n in names[half:]}, os.path.join(folder, "model-00002-of-00002.safetensors"))
    ref = load_weights(folder, plan, torch.bfloat16, "cpu")
    os.unlink(path)
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors") for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    got = load_weights(folder, plan, torch.bfloat16, "cpu")
    assert all(torch.equal(ref[k], got[k]) for k in ref)
