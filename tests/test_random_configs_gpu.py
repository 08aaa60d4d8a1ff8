"""Random LFM2 configurations, requests and cuttings against the plain implementation: 24 fixed seeds,
each a configuration of its own (widths that are and are not multiples of 8, head sizes 16 to 128 in steps
of 16, one to four key/value heads in groups of one to eight, one to five layers in any order of kinds, some
without attention, one to five taps, with and without bias, tied and untied, pages of 4 to 64 tokens), a set
of requests, and the four ways of cutting them with random portion sizes, in 32-bit and in bfloat16, at the
bounds of tolerances.py. Every third seed also generates through the engine under a roomy and a tight pool,
greedy and with temperature, and wants the same tokens from both.

The sizes stay in the range the bounds were stated for (widths up to 200, all heads together at most four times
the width, up to five layers, a few hundred tokens), and the linear weights' spread is 1.2 / sqrt(width), that of
the tiny configurations."""
import numpy as np
import pytest

import plain_lfm2 as plain
import traces
from tolerances import check_close

pytestmark = pytest.mark.gpu
SEEDS = list(range(24))


def random_config(rng):
    H = int(rng.choice([64, 72, 96, 100, 104, 128, 136, 192, 200]))
    while True:     # all heads together up to four times the width (in the family they are as wide as the model)
        hd = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128]))
        nkv = int(rng.choice([1, 2, 3, 4]))
        group = int(rng.choice([1, 2, 3, 4, 8] if hd <= 64 else [1, 2, 4]))
        if nkv * group * hd <= 4 * H:
            break
    L = int(rng.integers(1, 6))
    types = [str(rng.choice(["conv", "full_attention"])) for _ in range(L)]
    if rng.random() < 0.85 and "full_attention" not in types:
        types[int(rng.integers(0, L))] = "full_attention"
    cfg = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": int(rng.integers(50, 3000)),
           "hidden_size": H, "num_hidden_layers": L, "layer_types": types, "num_attention_heads": nkv * group,
           "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": int(rng.choice([64, 128, 130, 192, 200, 256, 320, 333, 512])),
           "block_auto_adjust_ff_dim": bool(rng.random() < 0.3), "block_multiple_of": int(rng.choice([8, 32, 64])),
           "block_ffn_dim_multiplier": float(rng.choice([1.0, 1.3])),
           "rope_theta": float(rng.choice([1e4, 5e4, 1e6])), "conv_L_cache": int(rng.choice([1, 2, 3, 3, 4, 5])),
           "conv_bias": bool(rng.random() < 0.4), "norm_eps": float(rng.choice([1e-5, 1e-6])),
           "tie_embedding": bool(rng.random() < 0.6), "max_position_embeddings": 4096}
    page = int(rng.choice([4, 8, 16, 16, 32, 64]))
    lens = [int(x) for x in rng.integers(1, 260, int(rng.integers(2, 7)))]
    return cfg, page, lens


def write_model(tmp_path, cfg, seed):
    from cellm_b200.weights import InitSpec, write_random_model
    init = InitSpec(linear_std=1.2 / cfg["hidden_size"] ** 0.5, embedding_std=0.1, conv_tap_std=0.3, bias_std=0.05, norm_jitter=0.1)
    return write_random_model(str(tmp_path / "m"), cfg, seed=seed, dtype="bfloat16", init=init)


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration_in_every_cutting(tmp_path, seed):
    from cellm_b200.replay import Replayer
    rng = np.random.default_rng(seed)
    cfg, page, lens = random_config(rng)
    folder = write_model(tmp_path, cfg, seed)
    c, w = plain.load_folder(folder)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate(lens)}
    ref = {r: plain.forward(c, w, t).numpy() for r, t in reqs.items()}
    cuts = {"whole": traces.whole(reqs), "tail": traces.tail_one_by_one(reqs, tail=int(rng.integers(1, 40))),
            "portions": traces.portions(reqs, sizes=tuple(int(x) for x in rng.integers(2, 70, 7))),
            "mixed": traces.mixed(reqs, prompt_frac=float(rng.uniform(0.2, 0.95)),
                                  portion_sizes=tuple(int(x) for x in rng.integers(2, 40, 5)),
                                  max_live=int(rng.integers(2, 5)), seed=seed)}
    for dtype in ("float32", "bfloat16"):
        for name, steps in cuts.items():
            rp = Replayer(folder, dtype, traces.max_live_tokens(steps, round_to=max(64, page)), page, 4)
            got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
            for r, t in reqs.items():
                check_close(traces.as_matrix(got[r], len(t)), ref[r], dtype, f"seed {seed} {cfg} page {page}: {dtype} {name} {r}")
            assert rp.cache.live == 0


@pytest.mark.parametrize("seed", SEEDS[::3])
def test_random_configuration_generates_the_same_under_a_tight_pool(tmp_path, seed):
    from cellm_b200 import Engine, SamplingParams
    rng = np.random.default_rng(1000 + seed)
    cfg, page, lens = random_config(rng)
    lens = [min(n, 120) for n in lens][:5]
    gen = int(rng.integers(4, 40))
    folder = write_model(tmp_path, cfg, seed)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lens]
    need = [-(-(n + gen) // page) for n in lens]
    for params in (SamplingParams.greedy(gen, stop_eos=False),
                   SamplingParams(temperature=0.9, top_k=int(rng.choice([0, 5, 40])), seed=7 + seed,
                                  repeat_penalty=float(rng.choice([1.0, 1.1])), max_new_tokens=gen, stop_eos=False)):
        big = Engine(folder, dtype="float32", tokens_per_block=page, total_blocks=sum(need) + 4, max_num_seqs=len(lens),
                     max_batch_tokens=int(rng.integers(8, 200)), prefill_chunk=int(rng.integers(2, 64)))
        ref = big.generate(prompts, params)
        tight = max(max(need), sum(need) * int(rng.integers(30, 80)) // 100)
        small = Engine(folder, dtype="float32", tokens_per_block=page, total_blocks=tight,
                       max_num_seqs=int(rng.integers(1, len(lens) + 1)),
                       max_batch_tokens=int(rng.integers(8, 200)), prefill_chunk=int(rng.integers(2, 64)))
        out = small.generate(prompts, params)
        st = small.stats()
        assert st["free_pages"] == st["total_pages"], f"pages lost: {st}"
        assert [len(o) for o in out] == [gen] * len(lens)
        assert out == ref, f"seed {seed} temperature {params.temperature} preemptions {st['preemptions']}"
