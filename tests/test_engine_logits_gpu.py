"""The logits of the steps that serving runs: Engine.step() with the index arrays written by the runtime,
decode steps replayed as CUDA graphs (block tables padded to the graph's width bucket, arg-max inside the
graph), at the numbers of live requests the benchmark reports. Every step's logits are copied out through
Engine.on_logits and compared with the plain implementation."""
import numpy as np
import pytest

import plain_lfm2 as plain
from tiny_configs import CONFIGS, FULL_WIDTH, FULL_WIDTH_INIT, make_model
from tolerances import K, K_SELF, check_close

pytestmark = pytest.mark.gpu


def run_engine(eng, prompts, params):
    """Adds the prompts, steps to the end; returns per request the generated tokens and the logits row
    behind each of them, and the kinds of step that ran."""
    import torch
    got = {}

    def keep(rows, logits):
        host = logits.to("cpu").numpy()
        for r, row in zip(rows, host):
            got.setdefault(r, []).append(row.copy())
    eng.on_logits = keep
    ids = [eng.add_request(p, params) for p in prompts]
    graph_steps = eager_steps = 0
    while eng.has_unfinished():
        eng.step()
        if eng.runner.last_argmax is not None:
            graph_steps += 1
        else:
            eager_steps += 1
    torch.cuda.synchronize()
    return [(eng.output(i).tokens, np.stack(got[i])) for i in ids], graph_steps, eager_steps


@pytest.fixture(scope="module")
def full_width(tmp_path_factory):
    from cellm_b200.models import load_model
    from cellm_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("fw") / "m"), FULL_WIDTH, seed=6, dtype="bfloat16",
                                init=FULL_WIDTH_INIT)
    return plain.load_folder(folder), load_model(folder, "bfloat16", "cuda:0")


@pytest.mark.parametrize("live", [8, 64])
def test_logits_of_served_steps_with_many_live_requests(full_width, live):
    """Layers of LFM2-1.2B's own sizes, bfloat16, 8 and 64 live requests: the decode products take their
    16-, 32- and 64-token tiles, the short convolution's epilogue works on several tokens side by side, decode
    attention runs hundreds of (request, key/value head) groups. Prompts of 8 to 40 tokens, 40 decoded tokens."""
    from cellm_b200 import Engine, SamplingParams
    (cfg, w), loaded = full_width
    rng = np.random.default_rng(live)
    prompts = [rng.integers(0, cfg["vocab_size"], int(n)).tolist() for n in rng.integers(8, 41, live)]
    n_new = 40
    eng = Engine(loaded, dtype="bfloat16", tokens_per_block=16, total_blocks=6 * live, max_num_seqs=live,
                 max_batch_tokens=2048, prefill_chunk=512)
    outs, graph_steps, eager_steps = run_engine(eng, prompts, SamplingParams.greedy(n_new, stop_eos=False))
    assert graph_steps >= n_new - 4 and eager_steps >= 1          # a shape is captured when it is met the third time
    assert max(key[0] for key in eng.runner._graphs) == live, "no decode step held all the requests"
    # the plain model on every request (8 live) or every fourth (64 live): 64-bit on the CPU takes its time
    for i in range(0, live, 1 if live <= 8 else 4):
        tokens, logits = outs[i]
        seq = prompts[i] + tokens[:-1]
        ref = plain.forward(cfg, w, seq, rows=list(range(len(prompts[i]) - 1, len(seq)))).numpy()
        check_close(logits, ref, "bfloat16", f"{live} live, request {i}")
        # greedy: each token is the arg-max of the row behind it (computed inside the step's graph)
        assert tokens == logits.argmax(axis=-1).tolist()
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_decoding_past_a_graph_width_bucket(tmp_path, dtype):
    """Captured decode steps are keyed by the block-table width rounded up to 32 pages. With pages of 8 tokens a
    request of 200 tokens that decodes 100 more crosses from the first bucket (256 tokens) into the second, beside
    a short request that stays in the first. Logits with graphs, without them, and of the plain model agree, and
    every greedy token that differs from the plain model's sits at a near-tie."""
    from cellm_b200 import Engine, SamplingParams
    folder = make_model(tmp_path, "tiny_b")
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (200, 11)]
    kw = dict(dtype=dtype, tokens_per_block=8, total_blocks=64, max_num_seqs=2, max_batch_tokens=256, prefill_chunk=128)
    runs = {}
    for graphs in (True, False):
        eng = Engine(folder, use_cuda_graphs=graphs, **kw)
        runs[graphs], graph_steps, _ = run_engine(eng, prompts, SamplingParams.greedy(100, stop_eos=False))
        assert (graph_steps > 0) == graphs
        if graphs:
            assert {key[1] for key in eng.runner._graphs} == {32, 64}, "both width buckets were to be met"
    for i, p in enumerate(prompts):
        tokens, logits = runs[True][i]
        seq = p + tokens[:-1]
        ref = plain.forward(cfg, w, seq, rows=list(range(len(p) - 1, len(seq)))).numpy()
        check_close(logits, ref, dtype, f"{dtype} graphs, request {i}")
        tol = K[dtype] * (1 + np.abs(ref).max())
        for j, t in enumerate(tokens):      # a token other than the plain model's only where its top two are within the bound
            best = int(ref[j].argmax())
            assert t == best or ref[j][best] - ref[j][t] <= 2 * tol, f"request {i} token {j}: {t} vs {best}"
        # without graphs: the same tokens fed, so the same rows as long as the tokens agree
        tokens2, logits2 = runs[False][i]
        same = next((j for j in range(len(tokens)) if tokens[j] != tokens2[j]), len(tokens))
        assert same >= 1
        check_close(logits2[:same + 1] if same < len(tokens) else logits2, logits[:same + 1] if same < len(tokens) else logits,
                    dtype, f"{dtype} kernel by kernel vs graphs, request {i}", k=K_SELF[dtype])
        if dtype == "float32":
            assert tokens == tokens2


def test_decoding_at_a_long_context_beside_a_short_one(tmp_path):
    """One request with 2,300 tokens behind it decodes beside one with 20: the decode attention cuts the keys into 16
    pieces (two clusters of eight CTAs that leave a piece each in the workspace), most of which are empty for the
    short request. The logits of every decoded token against the plain model. (With random weights 2,300 keys weigh
    about the same, so this run shows the step's wiring at that size: workspace, counters, graph replay; that no
    piece is lost is shown where one key towers, test_kernels_gpu.py.)"""
    from cellm_b200 import Engine, SamplingParams
    from cellm_b200.runtime import program
    folder = make_model(tmp_path, "tiny_b", overrides={"max_position_embeddings": 4096})
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (2300, 20)]
    eng = Engine(folder, dtype="bfloat16", tokens_per_block=16, total_blocks=160, max_num_seqs=2, max_batch_tokens=4096,
                 prefill_chunk=4096)
    before = program.CALLS.get("cellm_attention_decode", 0)
    outs, graph_steps, _ = run_engine(eng, prompts, SamplingParams.greedy(12, stop_eos=False))
    assert graph_steps >= 8 and program.CALLS.get("cellm_attention_decode", 0) > before
    for i, p in enumerate(prompts):
        tokens, logits = outs[i]
        seq = p + tokens[:-1]
        ref = plain.forward(cfg, w, seq, rows=list(range(len(p) - 1, len(seq)))).numpy()
        check_close(logits, ref, "bfloat16", f"request {i}")
