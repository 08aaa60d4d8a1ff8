"""The whole LFM2-1.2B shape, all sixteen layers with attention at its own places [2, 5, 8, 10, 12, 14]
(ten short-convolution layers, six attention layers, width 2048, vocabulary 65536), random weights, against
the plain implementation: each request whole, and mixed with the others in portions beside decoded
tokens, in 32-bit and in bfloat16. The depth is what the four-layer models of the other tests lack."""
import numpy as np
import pytest

import plain_lfm2 as plain
import traces
from tiny_configs import FULL_WIDTH_INIT
from tolerances import K_SELF, check_close, k_for_depth

pytestmark = pytest.mark.gpu
LENGTHS = (8, 64, 23, 41)


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from cellm_b200.config.presets import shape
    from cellm_b200.weights import write_random_model
    config = shape("lfm2-1.2b")
    assert config["num_hidden_layers"] == 16 and config["full_attn_idxs"] == [2, 5, 8, 10, 12, 14]
    folder = write_random_model(str(tmp_path_factory.mktemp("depth") / "m"), config, seed=16, dtype="bfloat16",
                                init=FULL_WIDTH_INIT)
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(16)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate(LENGTHS)}
    ref = {r: plain.forward(cfg, w, t).numpy() for r, t in reqs.items()}
    del w
    return folder, reqs, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sixteen_layers_whole_and_mixed(model, dtype):
    from cellm_b200.models import load_model
    from cellm_b200.replay import Replayer
    folder, reqs, ref = model
    loaded = load_model(folder, dtype, "cuda:0")
    k = k_for_depth(dtype, 16)
    results = {}
    for make in (traces.whole, traces.mixed):
        steps = make(reqs)
        rp = Replayer(loaded, dtype, traces.max_live_tokens(steps), 16, 4)
        got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
        results[make.__name__] = got
        for r, t in reqs.items():
            check_close(traces.as_matrix(got[r], len(t)), ref[r], dtype, f"{dtype} {make.__name__} {r}", k=k)
    for r, t in reqs.items():
        check_close(traces.as_matrix(results["mixed"][r], len(t)), traces.as_matrix(results["whole"][r], len(t)),
                    dtype, f"{dtype} mixed vs whole {r}", k=K_SELF[dtype])
