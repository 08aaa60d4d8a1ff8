"""Generation through the Python entry point against the plain implementation:
greedy, temperature with a seed, long decoding, and a pool so small that
requests are preempted and recomputed."""
import numpy as np
import pytest

import plain_lfm2 as plain
from tiny_configs import CONFIGS, make_model
from token_checks import check_greedy, check_sampled

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    d = tmp_path_factory.mktemp("models")
    return {name: make_model(d, name) for name in CONFIGS}


def _prompts(vocab, lengths, seed=1):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, n).tolist() for n in lengths]


def _margin_ok(cfg, w, prompt, out, k=2e-3):
    """True if every greedy choice along `out` has a clear margin in the plain
    model, so that 32-bit rounding cannot flip it."""
    toks = list(prompt)
    for t in out:
        lg = plain.forward(cfg, w, toks)[-1]
        top = lg.topk(2).values
        if float(top[0] - top[1]) < k * (1 + float(lg.abs().max())):
            return False
        toks.append(t)
    return True


def test_greedy_generation_tiny_a(folders):
    """The workload of the first tiny configuration: prompts of 1, 7, 33 and 64 tokens, 16 greedy tokens each, page 8."""
    from cellm_b200 import Engine, SamplingParams
    cfg, w = plain.load_folder(folders["tiny_a"])
    prompts = _prompts(cfg["vocab_size"], [1, 7, 33, 64])
    eng = Engine(folders["tiny_a"], dtype="float32", tokens_per_block=8, total_blocks=64, max_num_seqs=4,
                 max_batch_tokens=48, prefill_chunk=24)
    outs = eng.generate(prompts, SamplingParams.greedy(16, stop_eos=False))
    for p, o in zip(prompts, outs):
        ref = plain.generate(cfg, w, p, 16)
        if o != ref:
            i = next(j for j in range(16) if o[j] != ref[j])
            assert not _margin_ok(cfg, w, p, ref[:i + 1]), f"token {i} differs: {o} vs {ref}"
        assert len(o) == 16
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"] and s["free_slots"] == 4


def test_temperature_generation_tiny_b(folders):
    """The workload of the second tiny configuration: prompts 5/50/200 in portions of 13 mixed with
    decode steps, 24 tokens at temperature 0.8 with a fixed seed, page 16."""
    from cellm_b200 import Engine, SamplingParams
    from cellm_b200.sampling import session_seed
    cfg, w = plain.load_folder(folders["tiny_b"])
    prompts = _prompts(cfg["vocab_size"], [5, 50, 200], seed=2)
    eng = Engine(folders["tiny_b"], dtype="float32", tokens_per_block=16, total_blocks=40, max_num_seqs=3,
                 max_batch_tokens=32, prefill_chunk=13)
    params = SamplingParams(temperature=0.8, top_k=40, seed=1234, repeat_penalty=1.05, repeat_window=64,
                            max_new_tokens=24, stop_eos=False)
    outs = eng.generate(prompts, params)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o) == 24
        # every token is the plain model's draw from the same random number, given the tokens before it; a
        # draw that lands within rounding of a boundary of the distribution may take the neighbour
        check_sampled(cfg, w, p, o, "float32", temperature=0.8, top_k=40, seed=session_seed(i, 1234),
                      repeat_penalty=1.05, repeat_window=64, what=f"request {i}")


def test_bfloat16_greedy_runs_and_frees(folders):
    from cellm_b200 import Engine, SamplingParams
    cfg, w = plain.load_folder(folders["tiny_b"])
    prompts = _prompts(cfg["vocab_size"], [9, 40, 3, 77, 120, 16], seed=3)
    eng = Engine(folders["tiny_b"], dtype="bfloat16", tokens_per_block=16, total_blocks=64, max_num_seqs=4,
                 max_batch_tokens=64, prefill_chunk=32)
    outs = eng.generate(prompts, SamplingParams.greedy(12, stop_eos=False))
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o) == 12
        check_greedy(cfg, w, p, o, "bfloat16", f"request {i}")       # all 12 tokens: the plain arg-max or a near-tie
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"]


def test_preemption_gives_the_same_tokens(folders):
    """With too few pages for all requests at once, running requests are
    preempted and recomputed; the tokens are the same as with a large pool."""
    from cellm_b200 import Engine, SamplingParams
    cfg, _ = plain.load_folder(folders["tiny_a"])
    prompts = _prompts(cfg["vocab_size"], [30, 30, 30, 30], seed=4)
    params = SamplingParams.greedy(40, stop_eos=False)
    big = Engine(folders["tiny_a"], dtype="float32", tokens_per_block=8, total_blocks=64, max_num_seqs=4)
    ref = big.generate(prompts, params)
    small = Engine(folders["tiny_a"], dtype="float32", tokens_per_block=8, total_blocks=20, max_num_seqs=4)
    out = small.generate(prompts, params)
    assert small.stats()["preemptions"] > 0
    assert out == ref
    assert small.stats()["free_pages"] == small.stats()["total_pages"]


def test_long_decoding_matches_plain(folders):
    """One short prompt decoded far beyond several pages, 32-bit, logits of the
    sampled path compared through greedy agreement with the plain model."""
    from cellm_b200 import Engine, SamplingParams
    cfg, w = plain.load_folder(folders["tiny_a"])
    prompt = _prompts(cfg["vocab_size"], [3], seed=6)[0]
    eng = Engine(folders["tiny_a"], dtype="float32", tokens_per_block=8, total_blocks=32, max_num_seqs=1)
    out = eng.generate([prompt], SamplingParams.greedy(200, stop_eos=False))[0]
    assert len(out) == 200
    toks = prompt + out
    lg = plain.forward(cfg, w, toks[:-1])
    ref_next = lg.argmax(dim=-1).tolist()[len(prompt) - 1:]
    mism = [i for i in range(200) if out[i] != ref_next[i]]
    for i in mism:   # only allowed where the plain model's top two are within rounding
        top = lg[len(prompt) - 1 + i].topk(2).values
        assert float(top[0] - top[1]) < 2e-3 * (1 + float(lg.abs().max()))


def test_stop_at_eos_and_request_too_large(folders):
    from cellm_b200 import Engine, SamplingParams
    from cellm_b200.engine import SchedulerError
    cfg, w = plain.load_folder(folders["tiny_a"])
    eng = Engine(folders["tiny_a"], dtype="float32", tokens_per_block=8, total_blocks=8, max_num_seqs=2)
    with pytest.raises(SchedulerError):
        eng.add_request(list(range(60)), SamplingParams.greedy(40))      # 100 tokens > 8 pages of 8
    with pytest.raises(SchedulerError):
        eng.add_request(list(range(200)), SamplingParams.greedy(100))    # beyond max_position_embeddings
    with pytest.raises(ValueError):
        eng.add_request([5, 100000], SamplingParams.greedy(4))


def test_generation_stops_at_the_end_of_sequence_token(tmp_path):
    """The same weights in a folder whose eos_token_id is the plain model's third greedy token: generation ends
    with that token, after three; with stop_eos off it goes on."""
    from cellm_b200 import Engine, SamplingParams
    cfg, w = plain.load_folder(make_model(tmp_path / "a", "tiny_a"))
    for seed in range(100, 140):        # a prompt whose third token is new and whose choices are clear
        p = _prompts(cfg["vocab_size"], [4], seed=seed)[0]
        ref = plain.generate(cfg, w, p, 6)
        if ref[2] not in ref[:2] and _margin_ok(cfg, w, p, ref):
            break
    else:
        raise AssertionError("no prompt with a clear greedy continuation among 40")
    folder = make_model(tmp_path / "b", "tiny_a", overrides={"eos_token_id": ref[2]})
    kw = dict(dtype="float32", tokens_per_block=8, total_blocks=8, max_num_seqs=2)
    assert Engine(folder, **kw).generate([p], SamplingParams.greedy(6, stop_eos=True)) == [ref[:3]]
    assert Engine(folder, **kw).generate([p], SamplingParams.greedy(6, stop_eos=False)) == [ref]


def test_captured_steps_are_dropped_least_recently_used_first(folders):
    """Decode steps are captured per (requests in the step, block-table width). With room for two
    captures only, requests that finish one after the other (4, 3, 2, 1 in a step) force captures
    out and, for the widths that come back, in again: the tokens are those of the uncaptured run."""
    from cellm_b200 import Engine, SamplingParams
    cfg, _ = plain.load_folder(folders["tiny_a"])
    prompts = _prompts(cfg["vocab_size"], [5, 9, 3, 12], seed=8)
    kw = dict(dtype="float32", tokens_per_block=8, total_blocks=64, max_num_seqs=4)
    ref_eng = Engine(folders["tiny_a"], use_cuda_graphs=False, **kw)
    eng = Engine(folders["tiny_a"], use_cuda_graphs=True, **kw)
    eng.runner.max_graphs = 2
    ids_ref, ids = [], []
    for i, p in enumerate(prompts):
        params = SamplingParams.greedy(6 + 7 * i, stop_eos=False)
        ids_ref.append(ref_eng.add_request(p, params))
        ids.append(eng.add_request(p, params))
    while ref_eng.has_unfinished():
        ref_eng.step()
    seen = 0
    while eng.has_unfinished():
        eng.step()
        seen = max(seen, len(eng.runner._graphs))
    assert seen == 2
    assert [eng.output(i).tokens for i in ids] == [ref_eng.output(i).tokens for i in ids_ref]
