"""Layers of LFM2-1.2B's own sizes (width 2048, 32 query heads on 8 key/value
heads of 64, feed-forward 12288 adjusted to 8192, vocabulary 65536, three taps)
in a model of four layers, against the plain implementation in every cutting:
the sizes at which the serving kernels take their large-tile, split and
clustered forms, which the tiny configurations never reach."""
import numpy as np
import pytest

import plain_lfm2 as plain
import traces
from tiny_configs import FULL_WIDTH, FULL_WIDTH_INIT
from tolerances import K, K_SELF, check_close

pytestmark = pytest.mark.gpu

CONFIG = FULL_WIDTH
LENGTHS = (37, 300, 129, 8)
K_PLAIN = K      # the bounds of tolerances.py, as for the tiny configurations


@pytest.fixture(scope="module")
def full(tmp_path_factory):
    from cellm_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("full") / "m"), CONFIG, seed=5, dtype="bfloat16",
                                init=FULL_WIDTH_INIT)
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
    # the decode steps above ran as CUDA graphs, as in serving; kernel by kernel they give the same
    for make in (traces.tail_one_by_one, traces.mixed):
        steps = make(reqs)
        rp = Replayer(loaded, dtype, traces.max_live_tokens(steps), 16, 4, use_graphs=False)
        got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
        assert not rp.runner._graphs
        for r, t in reqs.items():
            check_close(traces.as_matrix(got[r], len(t)), ref[r], dtype, f"{dtype} {make.__name__} no graphs {r}",
                        k=K_PLAIN[dtype])
            check_close(traces.as_matrix(got[r], len(t)), traces.as_matrix(results[make.__name__][r], len(t)),
                        dtype, f"{dtype} {make.__name__}: kernel by kernel vs graphs {r}", k=K_SELF[dtype])
