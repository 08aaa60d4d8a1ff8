"""Configurations off the beaten path: head sizes in steps of 16 (16, 48, 80,
128), widths and vocabularies that are no multiple of 8 or 64, one and many
key/value heads, one to five convolution taps, a model without attention,
several page sizes. Each is
replayed whole, in portions and mixed, in both modes, against the plain
implementation."""
import numpy as np
import pytest

import plain_lfm2 as plain
import traces
from tiny_configs import TEST_INIT
from token_checks import check_greedy
from tolerances import check_close

pytestmark = pytest.mark.gpu


def cfg(**kw):
    base = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "rope_theta": 50000.0, "norm_eps": 1e-5,
            "conv_bias": False, "tie_embedding": True, "block_auto_adjust_ff_dim": False, "max_position_embeddings": 512}
    base.update(kw)
    return base


ODD = {
    # width 100 (no multiple of 8: every product takes the plain kernel), 5 heads of 16, feed-forward 130, vocabulary 777
    "w100": (cfg(vocab_size=777, hidden_size=100, num_hidden_layers=3, layer_types=["full_attention", "conv", "full_attention"],
                 num_attention_heads=5, num_key_value_heads=5, head_dim=16, intermediate_size=130, conv_L_cache=2), 8),
    # heads of 48 with one key/value head (group of 3), feed-forward 200 (no multiple of 64), untied head, bias, five taps
    "hd48": (cfg(vocab_size=1031, hidden_size=72, num_hidden_layers=3, layer_types=["conv", "full_attention", "conv"],
                 num_attention_heads=3, num_key_value_heads=1, head_dim=48, intermediate_size=200, conv_L_cache=5,
                 conv_bias=True, tie_embedding=False, norm_eps=1e-6), 16),
    # heads of 80, six query heads on two key/value heads, width 96, page of 32
    "hd80": (cfg(vocab_size=600, hidden_size=96, num_hidden_layers=2, layer_types=["full_attention", "full_attention"],
                 num_attention_heads=6, num_key_value_heads=2, head_dim=80, intermediate_size=256, rope_theta=1e6), 32),
    # heads of 128 (tensor-core attention), width 256, feed-forward adjusted 1000 -> 704, page of 4
    "hd128": (cfg(vocab_size=2000, hidden_size=256, num_hidden_layers=3, layer_types=["conv", "full_attention", "full_attention"],
                  num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=1000,
                  block_auto_adjust_ff_dim=True, block_multiple_of=64, conv_L_cache=4), 4),
    # sixteen query heads on one key/value head (the decode tile is full), heads of 64, width 128
    "g16": (cfg(vocab_size=512, hidden_size=128, num_hidden_layers=2, layer_types=["full_attention", "conv"],
                num_attention_heads=16, num_key_value_heads=1, head_dim=64, intermediate_size=192), 16),
    # no attention at all: requests hold a state slot and no page; a single tap (no state to carry) is the other edge
    "convonly": (cfg(vocab_size=300, hidden_size=72, num_hidden_layers=2, layer_types=["conv", "conv"],
                     num_attention_heads=3, num_key_value_heads=3, head_dim=16, intermediate_size=128, conv_L_cache=4,
                     conv_bias=True), 16),
    "onetap": (cfg(vocab_size=400, hidden_size=64, num_hidden_layers=3, layer_types=["conv", "full_attention", "conv"],
                   num_attention_heads=2, num_key_value_heads=1, head_dim=32, intermediate_size=128, conv_L_cache=1), 8),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ODD))
def test_odd_configuration_in_every_cutting(tmp_path, name, dtype):
    from cellm_b200.replay import Replayer
    from cellm_b200.weights import write_random_model
    config, page = ODD[name]
    folder = write_random_model(str(tmp_path / name), config, seed=31, dtype="bfloat16", init=TEST_INIT)
    c, w = plain.load_folder(folder)
    rng = np.random.default_rng(7)
    reqs = {f"r{i}": rng.integers(0, config["vocab_size"], n).tolist() for i, n in enumerate((70, 9, 130, 33, 2))}
    ref = {r: plain.forward(c, w, t).numpy() for r, t in reqs.items()}
    for make in (traces.whole, traces.tail_one_by_one, traces.portions, traces.mixed):
        steps = make(reqs)
        rp = Replayer(folder, dtype, traces.max_live_tokens(steps), page, 4)
        got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
        for r, t in reqs.items():
            check_close(traces.as_matrix(got[r], len(t)), ref[r], dtype, f"{name} {dtype} {make.__name__} {r}")


@pytest.mark.parametrize("name,page", [("g16", 16), ("g16", 8), ("hd64g2", 32)])
def test_prompt_attention_on_tcgen05_in_every_cutting(tmp_path, monkeypatch, name, page):
    """Small portions are sent to the tcgen05 prompt kernel (which otherwise takes
    only batches that fill the GPU): same traces, same plain implementation."""
    from cellm_b200.replay import Replayer
    from cellm_b200.runtime import program
    from cellm_b200.weights import write_random_model
    monkeypatch.setitem(program.OPTIONS, "attention_tc_min_ctas", 0)
    monkeypatch.setitem(program.OPTIONS, "attention_tc_min_fill", 0.0)
    before = program.CALLS["cellm_attention_tc"]
    config = ODD["g16"][0] if name == "g16" else cfg(
        vocab_size=900, hidden_size=192, num_hidden_layers=3, layer_types=["full_attention", "conv", "full_attention"],
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=320)
    folder = write_random_model(str(tmp_path / name), config, seed=32, dtype="bfloat16", init=TEST_INIT)
    c, w = plain.load_folder(folder)
    rng = np.random.default_rng(8)
    reqs = {f"r{i}": rng.integers(0, config["vocab_size"], n).tolist() for i, n in enumerate((150, 9, 300, 67))}
    ref = {r: plain.forward(c, w, t).numpy() for r, t in reqs.items()}
    for make in (traces.whole, traces.tail_one_by_one, traces.portions, traces.mixed):
        steps = make(reqs)
        rp = Replayer(folder, "bfloat16", traces.max_live_tokens(steps), page, 4)
        got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
        for r, t in reqs.items():
            check_close(traces.as_matrix(got[r], len(t)), ref[r], "bfloat16", f"{name} tc {make.__name__} {r}")
    assert program.CALLS["cellm_attention_tc"] > before


def test_decode_with_and_without_the_fused_decode_kernels(tmp_path, monkeypatch):
    """Decode steps of 64-wide heads run the q/k/v product that norms, turns and stores in its epilogue, and in_proj
    with the short convolution in its epilogue. With both switched off the same traces go through the separate
    kernels: the same plain implementation, and the two ways agree within the bound between cuttings."""
    from cellm_b200.replay import Replayer
    from cellm_b200.runtime import program
    from cellm_b200.weights import write_random_model
    from tolerances import K_SELF
    config = cfg(vocab_size=900, hidden_size=192, num_hidden_layers=3, layer_types=["full_attention", "conv", "full_attention"],
                 num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=320)
    folder = write_random_model(str(tmp_path / "m"), config, seed=32, dtype="bfloat16", init=TEST_INIT)
    c, w = plain.load_folder(folder)
    rng = np.random.default_rng(8)
    reqs = {f"r{i}": rng.integers(0, config["vocab_size"], n).tolist() for i, n in enumerate((150, 9, 300, 67))}
    ref = {r: plain.forward(c, w, t).numpy() for r, t in reqs.items()}
    results = {}
    for fused in (True, False):
        monkeypatch.setitem(program.OPTIONS, "fused_rope", fused)
        monkeypatch.setitem(program.OPTIONS, "fused_conv", fused)
        before = dict(program.CALLS)
        for make in (traces.tail_one_by_one, traces.mixed):
            steps = make(reqs)
            rp = Replayer(folder, "bfloat16", traces.max_live_tokens(steps), 32, 4, use_graphs=False)
            got = results[fused, make.__name__] = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
            for r, t in reqs.items():
                check_close(traces.as_matrix(got[r], len(t)), ref[r], "bfloat16", f"fused {fused} {make.__name__} {r}")
        ran = {k: program.CALLS[k] - before[k] for k in before}
        assert (ran["cellm_gemm_rope_tcgen05"] > 0) == fused and (ran["cellm_gemm_conv_tcgen05"] > 0) == fused
    for make in ("tail_one_by_one", "mixed"):
        for r, t in reqs.items():
            check_close(traces.as_matrix(results[True, make][r], len(t)), traces.as_matrix(results[False, make][r], len(t)),
                        "bfloat16", f"fused vs separate kernels {make} {r}", k=K_SELF["bfloat16"])


def test_odd_configuration_generates(tmp_path):
    from cellm_b200 import Engine, SamplingParams
    from cellm_b200.weights import write_random_model
    config, page = ODD["hd128"]
    folder = write_random_model(str(tmp_path / "m"), config, seed=31, dtype="bfloat16", init=TEST_INIT)
    c, w = plain.load_folder(folder)
    prompts = [np.random.default_rng(i).integers(0, 2000, n).tolist() for i, n in enumerate((3, 40, 17))]
    for dtype in ("float32", "bfloat16"):
        eng = Engine(folder, dtype=dtype, tokens_per_block=page, total_blocks=64, max_num_seqs=3, max_batch_tokens=24, prefill_chunk=16)
        outs = eng.generate(prompts, SamplingParams.greedy(8, stop_eos=False))
        for p, o in zip(prompts, outs):
            assert len(o) == 8
            check_greedy(c, w, p, o, dtype, f"{dtype} prompt of {len(p)}")
