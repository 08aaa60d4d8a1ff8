"""Decode steps that run ahead of their tokens (EngineConfig.run_ahead): a captured decode step of greedy requests
leaves its tokens on the device, the engine launches the next step before it reads them, and a token that ends a
request (end of sequence) is read one step late, when the request already has a row in the step after it. The
outcome must be what the engine gives when it reads every step's tokens at once: same tokens, same reasons, every
page back."""
import numpy as np
import pytest

from tiny_configs import make_model

pytestmark = pytest.mark.gpu

ENGINE = dict(tokens_per_block=8, total_blocks=64, max_num_seqs=8, max_batch_tokens=64, prefill_chunk=32)


def run(folder, prompts, params, run_ahead, dtype="float32", late=(), **kw):
    """Generates through Engine.step(); `late`: (after this many steps, prompt) pairs added while the others decode.
    Returns (tokens, finish reason) per request, the pairs step() returned in order, the number of steps."""
    from cellm_b200 import Engine
    eng = Engine(folder, dtype=dtype, run_ahead=run_ahead, **{**ENGINE, **kw})
    ids = [eng.add_request(p, params) for p in prompts]
    late = list(late)
    stream, steps = [], 0
    while eng.has_unfinished() or late:
        while late and late[0][0] <= steps:
            ids.append(eng.add_request(late.pop(0)[1], params))
        stream.append(eng.step())
        steps += 1
        assert steps < 2000
    eng.runner.check()
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"] and s["free_slots"] == eng.cache.num_slots
    return [(eng.output(i).tokens, eng.output(i).finish_reason) for i in ids], stream, steps, s


def prompts_of(cfg_vocab, lens, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg_vocab, n).tolist() for n in lens]


@pytest.mark.parametrize("name,dtype", [("tiny_a", "float32"), ("tiny_b", "float32"), ("tiny_b", "bfloat16")])
def test_the_same_tokens_with_and_without_running_ahead(tmp_path, name, dtype):
    """Different lengths to generate (requests leave one by one, by their length), greedy."""
    from cellm_b200 import SamplingParams
    folder = make_model(tmp_path, name, dtype="float32" if dtype == "float32" else "bfloat16")
    prompts = prompts_of(500, (5, 17, 9, 30, 3, 12), seed=1)
    outs = {}
    for ahead in (False, True):
        from cellm_b200 import Engine
        eng = Engine(folder, dtype=dtype, run_ahead=ahead, **ENGINE)
        ids = [eng.add_request(p, SamplingParams.greedy(6 + 5 * i, stop_eos=False)) for i, p in enumerate(prompts)]
        lag = 0
        while eng.has_unfinished():
            lag += eng._ahead is not None
            eng.step()
        outs[ahead] = [(eng.output(i).tokens, eng.output(i).finish_reason) for i in ids]
        assert (lag > 0) == ahead, "decode steps were to run ahead exactly when asked to"
        s = eng.stats()
        assert s["idle"] and s["free_pages"] == s["total_pages"]
    assert outs[True] == outs[False]
    assert [len(t) for t, _ in outs[True]] == [6 + 5 * i for i in range(6)] and all(r == "length" for _, r in outs[True])


def test_a_token_that_ends_a_request_is_read_a_step_late(tmp_path):
    """The end-of-sequence id is one that the requests are known to produce at different places (found by a run without
    stops). Each request must end with that token and no later one, although a step with a row of it was already
    running when the token was read."""
    from cellm_b200 import SamplingParams
    folder = make_model(tmp_path, "tiny_a", dtype="float32")
    prompts = prompts_of(500, (5, 17, 9, 30, 3, 12, 21, 8), seed=2)
    free, _, _, _ = run(folder, prompts, SamplingParams.greedy(40, stop_eos=False), run_ahead=False)
    counts = {}
    for toks, _ in free:
        for t in set(toks[2:]):
            counts[t] = counts.get(t, 0) + 1
    eos = max(counts, key=lambda t: (counts[t], -t))           # the token most requests come to
    assert counts[eos] >= 2
    stopping = make_model(tmp_path / "eos", "tiny_a", dtype="float32", overrides={"eos_token_id": int(eos)})
    params = SamplingParams.greedy(40, stop_eos=True)
    a, stream_a, steps_a, _ = run(stopping, prompts, params, run_ahead=False)
    b, stream_b, steps_b, _ = run(stopping, prompts, params, run_ahead=True)
    assert a == b
    for (toks, reason), (ref, _) in zip(b, free):
        if eos in ref:
            cut = ref.index(eos) + 1
            assert toks == ref[:cut] and reason == "stop"
        else:
            assert toks == ref and reason == "length"
    # the same pairs come out of step(), a call later where the step ran ahead
    flat = lambda stream: [pair for out in stream for pair in out]
    assert sorted(flat(stream_a)) == sorted(flat(stream_b))
    per_request = lambda stream, r: [t for rid, t in flat(stream) if rid == r]
    assert all(per_request(stream_b, r) == b[r][0] for r in range(len(prompts)))


def test_running_ahead_through_preemption_and_late_arrivals(tmp_path):
    """A pool too small for all requests at their full lengths (the scheduler preempts and recomputes), and requests
    that arrive while the others decode (the step they join is not a captured one, so the tokens before it are read
    first): the same tokens either way."""
    from cellm_b200 import SamplingParams
    folder = make_model(tmp_path, "tiny_a", dtype="float32")
    prompts = prompts_of(500, (20, 25, 18, 30), seed=3)
    late = [(6, prompts_of(500, (14,), seed=4)[0]), (15, prompts_of(500, (7,), seed=5)[0])]
    params = SamplingParams.greedy(60, stop_eos=False)
    tight = dict(total_blocks=30)          # 4 x (30 + 60) tokens would need 45 pages of 8
    a, _, _, stats_a = run(folder, prompts, params, run_ahead=False, late=late, **tight)
    b, _, _, stats_b = run(folder, prompts, params, run_ahead=True, late=late, **tight)
    assert stats_a["preemptions"] > 0 and stats_b["preemptions"] > 0
    assert a == b and all(len(t) == 60 for t, _ in b)


def test_sampling_with_temperature_reads_every_step(tmp_path):
    """Requests that draw from the distribution need the host's random stream and, with a repeat penalty, the tokens so
    far: their steps do not run ahead, and greedy requests beside them wait with them."""
    from cellm_b200 import Engine, SamplingParams
    folder = make_model(tmp_path, "tiny_a", dtype="float32")
    prompts = prompts_of(500, (5, 9), seed=6)
    eng = Engine(folder, dtype="float32", run_ahead=True, **ENGINE)
    eng.add_request(prompts[0], SamplingParams(temperature=0.8, top_k=20, max_new_tokens=12, seed=3))
    eng.add_request(prompts[1], SamplingParams.greedy(12, stop_eos=False))
    while eng.has_unfinished():
        eng.step()
        assert eng._ahead is None
    ref = Engine(folder, dtype="float32", run_ahead=False, **ENGINE)
    ref.add_request(prompts[0], SamplingParams(temperature=0.8, top_k=20, max_new_tokens=12, seed=3))
    ref.add_request(prompts[1], SamplingParams.greedy(12, stop_eos=False))
    while ref.has_unfinished():
        ref.step()
    assert [eng.output(i).tokens for i in (0, 1)] == [ref.output(i).tokens for i in (0, 1)]
