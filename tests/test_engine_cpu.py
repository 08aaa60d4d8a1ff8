"""The engine's bookkeeping around the step function, on the CPU: kernels are recorders, and the arg-max
"kernel" hands out tokens the test chooses. Requests are admitted, cut into portions, decoded, stopped at
the end-of-sequence token, preempted when pages run out, and everything is given back."""
import ctypes

import pytest
import torch

from launch_recorder import Recorder, zero_model

CONFIG = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": 1000, "hidden_size": 64,
          "num_hidden_layers": 2, "layer_types": ["conv", "full_attention"], "num_attention_heads": 4,
          "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "block_auto_adjust_ff_dim": False,
          "rope_theta": 1e4, "conv_L_cache": 3, "norm_eps": 1e-5, "tie_embedding": True, "max_position_embeddings": 512,
          "eos_token_id": 7}


def engine(monkeypatch, next_token, **kw):
    """An engine on the CPU whose arg-max gives next_token(row, call number)."""
    from cellm_b200 import Engine
    calls = [0]

    def argmax(out, logits, R, V, parts, stream):
        row = (ctypes.c_int * R).from_address(out)
        for r in range(R):
            row[r] = next_token(r, calls[0])
        calls[0] += 1
    rec = Recorder(monkeypatch, hooks={"cellm_argmax": argmax})
    loaded = zero_model(CONFIG)
    eng = Engine(loaded, dtype="bfloat16", device="cpu", use_cuda_graphs=False, **kw)
    monkeypatch.setattr(eng.runner, "_staging", lambda n: torch.empty(max(n, 4096), dtype=torch.int32))
    monkeypatch.setattr(eng.runner, "_uploaded", lambda: None)
    monkeypatch.setattr(eng.runner, "check", lambda: None)          # reads the device error word
    return eng, rec


def test_requests_run_to_their_length_and_everything_is_given_back(monkeypatch):
    from cellm_b200 import SamplingParams
    eng, rec = engine(monkeypatch, lambda r, n: 100 + n, tokens_per_block=8, total_blocks=32, max_num_seqs=3,
                      max_batch_tokens=16, prefill_chunk=8)
    prompts = [list(range(1, 20)), [5, 6, 7], list(range(30, 41)), [9]]
    outs = eng.generate(prompts, SamplingParams.greedy(5, stop_eos=False))
    assert [len(o) for o in outs] == [5, 5, 5, 5]
    st = eng.stats()
    assert st["idle"] and st["free_pages"] == st["total_pages"] and st["free_slots"] == 3
    # every step stayed under the token budget, and portions under their limit
    for args in rec.of("cellm_embed"):
        assert args[4] <= 16


def test_generation_stops_at_the_end_of_sequence_token(monkeypatch):
    from cellm_b200 import SamplingParams
    eng, _ = engine(monkeypatch, lambda r, n: 7 if n == 3 else 50, tokens_per_block=8, total_blocks=16, max_num_seqs=2)
    out = eng.generate([[1, 2, 3]], SamplingParams.greedy(20, stop_eos=True))[0]
    assert out == [50, 50, 50, 7]
    eng2, _ = engine(monkeypatch, lambda r, n: 7 if n == 3 else 50, tokens_per_block=8, total_blocks=16, max_num_seqs=2)
    assert len(eng2.generate([[1, 2, 3]], SamplingParams.greedy(20, stop_eos=False))[0]) == 20


def test_preempted_requests_are_recomputed_and_finish(monkeypatch):
    from cellm_b200 import SamplingParams
    eng, _ = engine(monkeypatch, lambda r, n: 200 + (n % 50), tokens_per_block=4, total_blocks=14, max_num_seqs=4,
                    max_batch_tokens=32, prefill_chunk=16)
    prompts = [list(range(10, 18)) for _ in range(4)]
    outs = eng.generate(prompts, SamplingParams.greedy(24, stop_eos=False))
    assert [len(o) for o in outs] == [24] * 4
    st = eng.stats()
    assert st["preemptions"] > 0 and st["free_pages"] == st["total_pages"]


def test_cancel_and_refusals(monkeypatch):
    from cellm_b200 import SamplingParams
    from cellm_b200.engine import SchedulerError
    eng, _ = engine(monkeypatch, lambda r, n: 11, tokens_per_block=8, total_blocks=8, max_num_seqs=2)
    a = eng.add_request([1, 2, 3], SamplingParams.greedy(30, stop_eos=False))
    b = eng.add_request([4, 5], SamplingParams.greedy(3, stop_eos=False))
    eng.step()
    eng.cancel(a)
    while eng.has_unfinished():
        eng.step()
    assert eng.output(a).finish_reason == "cancelled" and eng.output(b).tokens == [11, 11, 11]
    with pytest.raises(SchedulerError):
        eng.add_request(list(range(60)), SamplingParams.greedy(40))       # more than the pool holds
    with pytest.raises(ValueError):
        eng.add_request([5, 100000], SamplingParams.greedy(4))
    assert eng.stats()["free_pages"] == eng.stats()["total_pages"]


def test_sampling_inputs_follow_the_requests_streams_and_histories(monkeypatch):
    """With temperature, the sampling kernel gets one uniform number per request and step from the request's own
    XorShift64 stream (seeded as the reference mixes session and seed), its top-k and penalty, and the last tokens
    of prompt and output as the repetition window."""
    import numpy as np
    import plain_lfm2 as plain
    from cellm_b200 import Engine, SamplingParams
    from cellm_b200.sampling import session_seed
    seen = []

    def sample(out, logits, R, V, temperature, top_k, u, penalty, recent, W, max_top_k, group_max, stream):
        f = lambda a: list((ctypes.c_float * R).from_address(a))
        rec = np.ctypeslib.as_array((ctypes.c_int * (R * W)).from_address(recent)).reshape(R, W).copy() if W else None
        seen.append((R, f(temperature), list((ctypes.c_int * R).from_address(top_k)), f(u), f(penalty), rec, W, max_top_k))
        row = (ctypes.c_int * R).from_address(out)
        for r in range(R):
            row[r] = 300 + len(seen)
    Recorder(monkeypatch, hooks={"cellm_sample": sample})
    eng = Engine(zero_model(CONFIG), dtype="bfloat16", device="cpu", use_cuda_graphs=False,
                 tokens_per_block=8, total_blocks=16, max_num_seqs=2)
    monkeypatch.setattr(eng.runner, "_staging", lambda n: torch.empty(max(n, 4096), dtype=torch.int32))
    monkeypatch.setattr(eng.runner, "_uploaded", lambda: None)
    monkeypatch.setattr(eng.runner, "check", lambda: None)
    params = SamplingParams(temperature=0.7, top_k=12, seed=99, repeat_penalty=1.2, repeat_window=4, max_new_tokens=3, stop_eos=False)
    outs = eng.generate([[1, 2, 3, 4, 5, 6], [9]], params)
    assert outs == [[301, 302, 303], [301, 302, 303]] and len(seen) == 3
    streams = [plain.XorShift64(session_seed(i, 99)) for i in range(2)]
    history = [[1, 2, 3, 4, 5, 6], [9]]
    for step, (R, temp, top_k, u, penalty, recent, W, max_top_k) in enumerate(seen):
        assert R == 2 and W == 4 and max_top_k == 12 and top_k == [12, 12]
        assert temp == pytest.approx([0.7, 0.7]) and penalty == pytest.approx([1.2, 1.2])
        for r in range(2):
            assert u[r] == pytest.approx(streams[r].next_f32(), abs=1e-7)
            tail = history[r][-4:]
            assert list(recent[r][:len(tail)]) == tail and all(v == -1 for v in recent[r][len(tail):])
            history[r].append(301 + step)


@pytest.mark.parametrize("seed", range(12))
def test_random_requests_through_the_engine(monkeypatch, seed):
    """Random prompts, lengths, sampling modes, pools and budgets; some requests meet the end-of-sequence token,
    some are cancelled under way. Every request ends with a reason, no output is longer than asked for, nothing
    of the engine's per-request state is left behind and all pages and slots come back."""
    import numpy as np
    from cellm_b200 import SamplingParams
    rng = np.random.default_rng(seed)
    page = int(rng.choice([4, 8, 16]))
    n = int(rng.integers(2, 9))
    lens = [int(x) for x in rng.integers(1, 50, n)]
    news = [int(x) for x in rng.integers(1, 25, n)]
    need = [-(-(l + g) // page) for l, g in zip(lens, news)]
    pages = int(max(max(need), sum(need) * rng.uniform(0.3, 1.0)))
    token = lambda r, k: 7 if rng.random() < 0.04 else int(rng.integers(8, 1000))

    def sample(out, logits, R, V, *rest):
        row = (ctypes.c_int * R).from_address(out)
        for r in range(R):
            row[r] = token(r, 0)
    eng, rec = engine(monkeypatch, token, tokens_per_block=page, total_blocks=pages, max_num_seqs=int(rng.integers(1, n + 1)),
                      max_batch_tokens=int(rng.integers(4, 64)), prefill_chunk=int(rng.integers(2, 32)))
    monkeypatch.setitem(rec.hooks, "cellm_sample", sample)
    ids, asked, stop = [], {}, {}
    for l, g in zip(lens, news):
        greedy = rng.random() < 0.5
        stop_eos = bool(rng.random() < 0.5)
        params = SamplingParams.greedy(g, stop_eos=stop_eos) if greedy else SamplingParams(
            temperature=0.8, top_k=int(rng.choice([0, 40])), seed=int(rng.integers(1, 1000)),
            repeat_penalty=float(rng.choice([1.0, 1.1])), max_new_tokens=g, stop_eos=stop_eos)
        rid = eng.add_request([int(x) for x in rng.integers(8, 1000, l)], params)
        ids.append(rid)
        asked[rid], stop[rid] = g, stop_eos
    cancel_at = {rid: int(rng.integers(1, 30)) for rid in ids if rng.random() < 0.2}
    steps = 0
    while eng.has_unfinished():
        for rid, at in cancel_at.items():
            if at == steps and not eng.output(rid).finished:
                eng.cancel(rid)
        eng.step()
        steps += 1
        assert steps < 3000
    for rid in ids:
        out = eng.output(rid)
        assert out.finished and out.finish_reason in ("length", "stop", "cancelled")
        assert len(out.tokens) <= asked[rid]
        if out.finish_reason == "length":
            assert len(out.tokens) == asked[rid]
        if out.finish_reason == "stop":
            assert stop[rid] and out.tokens[-1] == 7 and 7 not in out.tokens[:-1]
        if not stop[rid]:
            assert out.finish_reason != "stop"
    st = eng.stats()
    assert st["idle"] and st["free_pages"] == st["total_pages"] and not eng._samplers


def test_replayer_maps_requests_reuses_pages_and_refuses_more_than_its_pool(monkeypatch):
    """Trace replay on the CPU: names become requests, `end` gives pages and slot back so that later requests get
    them again, a request left out of a step goes on later, and a pool made for --max-tokens holds no more."""
    from cellm_b200.cache.manager import OutOfPages
    from cellm_b200.replay import Replayer
    import traces
    rec = Recorder(monkeypatch)
    loaded = zero_model(CONFIG)
    rp = Replayer(loaded, "bfloat16", max_tokens=128, tokens_per_block=16, max_requests=2, device="cpu")
    monkeypatch.setattr(rp.runner, "_staging", lambda n: torch.empty(max(n, 4096), dtype=torch.int32))
    monkeypatch.setattr(rp.runner, "_uploaded", lambda: None)
    monkeypatch.setattr(rp.runner, "check", lambda: None)
    assert rp.cache.group_pages == [8]
    out = rp.step([{"id": "a", "tokens": list(range(1, 41)), "want": [0, 39]}, {"id": "b", "tokens": [5, 6], "want": []}])
    assert out.shape == (2, 1000) and rp.cache.free_pages(0) == 8 - 3 - 1
    assert rp.step([{"id": "b", "tokens": [7], "want": []}]) is None             # "a" sits this step out
    rp.step([{"id": "a", "tokens": [41], "want": [0]}], end=["a"])
    assert rp.cache.free_pages(0) == 7 and rp.cache.live == 1
    first_pages = set(range(8)) - {int(rp.cache.block_table(rp._ids["b"], 0)[0])}
    rp.step([{"id": "c", "tokens": list(range(60)), "want": [59]}])               # takes pages "a" gave back
    assert set(int(p) for p in rp.cache.block_table(rp._ids["c"], 0)) <= first_pages
    with pytest.raises(OutOfPages):
        rp.step([{"id": "c", "tokens": list(range(60)), "want": []}])             # 120 + 3 tokens > the pool's 128
    rp.step([], end=["b", "c"])
    assert rp.cache.live == 0 and rp.cache.free_pages(0) == 8
    # the traces the GPU tests replay need exactly the pool their own accounting asks for
    reqs = {"x": list(range(70)), "y": list(range(9)), "z": list(range(130))}
    for make in (traces.whole, traces.tail_one_by_one, traces.portions, traces.mixed):
        steps = make(reqs)
        rp2 = Replayer(loaded, "bfloat16", traces.max_live_tokens(steps), 16, 4, device="cpu")
        monkeypatch.setattr(rp2.runner, "_staging", lambda n: torch.empty(max(n, 4096), dtype=torch.int32))
        monkeypatch.setattr(rp2.runner, "_uploaded", lambda: None)
        monkeypatch.setattr(rp2.runner, "check", lambda: None)
        for s in steps:
            rp2.step(s["entries"], s["end"])
        assert rp2.cache.live == 0
