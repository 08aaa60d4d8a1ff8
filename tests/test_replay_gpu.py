"""Replays the same requests whole, with the last tokens one by one, in
portions of changing size, and mixed with other requests so that pages are
used again, in 32-bit and in bfloat16, and compares all with the plain
implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_lfm2 as plain
import traces
from tiny_configs import CONFIGS, make_model
from tolerances import K_SELF, check_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LENGTHS = {"tiny_a": [1, 7, 33, 64, 100, 45, 130], "tiny_b": [5, 50, 200, 77, 2, 140]}
PAGE = {"tiny_a": 8, "tiny_b": 16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    d = tmp_path_factory.mktemp("models")
    out = {}
    for name in CONFIGS:
        folder = make_model(d, name)
        cfg, w = plain.load_folder(folder)
        rng = np.random.default_rng(5)
        reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate(LENGTHS[name])}
        ref = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
        out[name] = (folder, reqs, ref)
    return out


def run_trace(folder, dtype, steps, page, max_tokens=None, use_graphs=True):
    from cellm_b200.replay import Replayer
    rp = Replayer(folder, dtype, max_tokens or traces.max_live_tokens(steps), page, 4, use_graphs=use_graphs)
    outs = [rp.step(s["entries"], s["end"]) for s in steps]
    decode_steps = sum(all(len(e["tokens"]) == 1 and e["want"] == [0] for e in s["entries"]) for s in steps)
    assert (len(rp.runner._graphs) > 0) == (use_graphs and decode_steps > 0), "decode steps did not take the asked path"
    assert rp.cache.live == 0
    assert all(rp.cache.free_pages(g) == rp.cache.group_pages[g] for g in range(len(rp.cache.group_pages)))
    return traces.collect(steps, outs)


FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions, "mixed": traces.mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_matches_plain(models, name, dtype):
    folder, reqs, ref = models[name]
    results = {}
    for fam, make in FAMILIES.items():
        steps = make(reqs)
        got = run_trace(folder, dtype, steps, PAGE[name])
        results[fam] = got
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} {fam} {rid}")
    for fam in ("tail", "portions", "mixed"):
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(results[fam][rid], len(toks)), traces.as_matrix(results["whole"][rid], len(toks)),
                        dtype, f"{name} {dtype} {fam} vs whole {rid}", k=K_SELF[dtype])
    # Decode steps above were replayed as CUDA graphs (block tables padded to the graph's width, the number of key
    # splits planned from that width), as serving replays them; launched kernel by kernel they must give the same.
    for fam in ("tail", "mixed"):
        got = run_trace(folder, dtype, FAMILIES[fam](reqs), PAGE[name], use_graphs=False)
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} {fam} no graphs {rid}")
            check_close(traces.as_matrix(got[rid], len(toks)), traces.as_matrix(results[fam][rid], len(toks)),
                        dtype, f"{name} {dtype} {fam}: kernel by kernel vs graphs {rid}", k=K_SELF[dtype])


def test_mixed_trace_reuses_pages(models):
    """The mixed trace's pool is so small that later requests get pages that
    earlier ones gave back."""
    folder, reqs, _ = models["tiny_a"]
    steps = traces.mixed(reqs)
    need = traces.max_live_tokens(steps)
    assert need < sum(-(-len(t) // 64) * 64 for t in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    """bin/trace_run as a user calls it: steps on standard input, files out."""
    folder, reqs, ref = models["tiny_b"]
    steps = traces.mixed(reqs, seed=3)
    out_dir = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out_dir), "--max-tokens", str(traces.max_live_tokens(steps))],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    V = CONFIGS["tiny_b"]["vocab_size"]
    outs = []
    for s in steps:
        f = out_dir / f"{s['step']}.f32"
        n_want = sum(len(e["want"]) for e in s["entries"])
        outs.append(np.fromfile(f, dtype="<f4").reshape(n_want, V) if n_want else None)
    got = traces.collect(steps, outs)
    for rid, toks in reqs.items():
        check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"trace_run {dtype} {rid}")
