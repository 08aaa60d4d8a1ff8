"""Layers of LFM2-1.2B's own sizes (width 2048, 32 query heads on 8 key/value
heads of 64, feed-forward 12288 adjusted to 8192, vocabulary 65536, three taps)
in a model of four layers, against the plain implementation in every cutting:
the sizes at which the serving kernels take their large-tile, split and
clustered forms, which the tiny configurations never reach."""
import numpy as np
import pytest

import plain_lfm2 as plain
import traces
from tolerances import K, K_SELF, check_close

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "block_ffn_dim_multiplier": 1.0, "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False,
    "norm_eps": 1e-5, "tie_embedding": True, "max_position_embeddings": 128000,
}
LENGTHS = (37, 300, 129, 8)
# The bounds of tolerances.py are stated for sums of a few thousand products (the tiny
# configurations). Here the longest sum has 8192 (the feed-forward's second product), four times
# as many, and the rounding of a 32-bit sum grows with the square root of its length: twice the
# bound against the plain implementation in 32-bit. bfloat16's bound is set by the rounding of the
# activations, not by the sums, and stays. Cuttings are compared with each other at the usual bounds.
K_PLAIN = {"float32": 2 * K["float32"], "bfloat16": K["bfloat16"]}


@pytest.fixture(scope="module")
def full(tmp_path_factory):
    from cellm_b200.weights import InitSpec, write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("full") / "m"), CONFIG, seed=5, dtype="bfloat16",
                                init=InitSpec(linear_std=0.03, embedding_std=0.03, conv_tap_std=0.3, norm_jitter=0.1))
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(9)
    reqs = {f"r{i}": rng.integers(0, CONFIG["vocab_size"], n).tolist() for i, n in enumerate(LENGTHS)}
    ref = {r: plain.forward(cfg, w, t).numpy() for r, t in reqs.items()}
    return folder, reqs, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_size_layers_in_every_cutting(full, dtype):
    from cellm_b200.models import load_model
    from cellm_b200.replay import Replayer
    folder, reqs, ref = full
    loaded = load_model(folder, dtype, "cuda:0")
    results = {}
    for make in (traces.whole, traces.tail_one_by_one, traces.portions, traces.mixed):
        steps = make(reqs)
        rp = Replayer(loaded, dtype, traces.max_live_tokens(steps), 16, 4)
        got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
        results[make.__name__] = got
        for r, t in reqs.items():
            check_close(traces.as_matrix(got[r], len(t)), ref[r], dtype, f"{dtype} {make.__name__} {r}",
                        k=K_PLAIN[dtype])
    for fam in ("tail_one_by_one", "portions", "mixed"):
        for r, t in reqs.items():
            check_close(traces.as_matrix(results[fam][r], len(t)), traces.as_matrix(results["whole"][r], len(t)),
                        dtype, f"{dtype} {fam} vs whole {r}", k=K_SELF[dtype])
