"""The command lines on the GPU, as a user calls them: a model folder (or a configuration for random
weights) goes in, generated tokens and the reference tools' report lines come out
(tools/infer/src/main.rs:432-536, tools/bench/src/main.rs:162-194)."""
import json
import os
import re
import subprocess
import sys

import pytest

import plain_lfm2 as plain
from tiny_configs import TINY_A, TINY_B, make_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_tool(tool, *args):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", tool), *map(str, args)], capture_output=True, text=True,
                       timeout=900, env={**os.environ, "PYTHONUNBUFFERED": "1"})
    assert p.returncode == 0, f"{tool} {args}:\n{p.stdout[-2000:]}\n{p.stderr[-3000:]}"
    return p.stdout


def greedy_margin_ok(cfg, w, prompt, ref, k=2e-3):
    """Every greedy choice along `ref` has a clear margin in the plain model."""
    toks = list(prompt)
    for t in ref:
        lg = plain.forward(cfg, w, toks)[-1]
        top = lg.topk(2).values
        if float(top[0] - top[1]) < k * (1 + float(lg.abs().max())):
            return False
        toks.append(t)
    return True


def test_infer_with_random_weights_greedy_in_32_bit(tmp_path):
    cfg_path = tmp_path / "tiny_b.json"
    cfg_path.write_text(json.dumps(TINY_B))
    prompt = [5, 17, 3, 999, 250, 41, 8, 77, 600, 12, 1]
    out = run_tool("infer", "--random", cfg_path, "--weights-seed", 4, "--tokens", ",".join(map(str, prompt)), "--gen", 8,
                   "--temperature", 0, "--dtype", "float32", "--stop-eos", "false", "--tokens-per-block", 8)
    folder = re.search(r"written to (\S+)", out).group(1)
    assert re.search(r"^Startup: .*KV cache: blocks=4 tokens_per_block=8$", out, re.M)      # ceil((11 + 8 + 8) / 8)
    assert re.search(r"^Prefill: 11 tokens in ", out, re.M) and re.search(r"^Decode: 7 tokens in .*tok/s\)$", out, re.M)
    tokens = [int(t) for t in re.search(r"^tokens: ([\d,]+)$", out, re.M).group(1).split(",")]
    cfg, w = plain.load_folder(folder)
    ref = plain.generate(cfg, w, prompt, 8)
    if tokens != ref:
        i = next(j for j in range(8) if tokens[j] != ref[j])
        assert not greedy_margin_ok(cfg, w, prompt, ref[:i + 1]), f"token {i}: {tokens} vs {ref}"
    assert len(tokens) == 8


def test_infer_samples_as_the_plain_model_with_the_same_seed(tmp_path):
    """Temperature, top-k, repeat penalty and --seed through the tool; --seq gives the prompt 0..seq-1."""
    folder = make_model(tmp_path, "tiny_a", dtype="float32")
    out = run_tool("infer", "--model", folder, "--seq", 9, "--gen", 12, "--temperature", 0.7, "--top-k", 20, "--seed", 99,
                   "--repeat-penalty", 1.1, "--repeat-window", 16, "--dtype", "float32", "--stop-eos", "false")
    tokens = [int(t) for t in re.search(r"^tokens: ([\d,]+)$", out, re.M).group(1).split(",")]
    cfg, w = plain.load_folder(folder)
    ref = plain.generate(cfg, w, list(range(9)), 12, temperature=0.7, top_k=20, seed=99, repeat_penalty=1.1, repeat_window=16)
    assert len(tokens) == 12
    # a draw within rounding of a boundary of the distribution may differ, and everything after it; the first tokens must not
    assert tokens[:4] == ref[:4], f"{tokens} vs {ref}"


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_bench_tool_reports_prefill_and_decode(tmp_path, dtype):
    folder = make_model(tmp_path, "tiny_a")
    out = run_tool("bench", "--model", folder, "--seq", 16, "--gen", 9, "--batch", 3, "--dtype", dtype, "--tokens-per-block", 8)
    assert re.search(r"^KV cache: blocks=15 tokens_per_block=8$", out, re.M)       # 3 * ceil((16 + 9 + 8) / 8)
    assert re.search(r"^Prefill: 48 tokens in \d+\.\d+s$", out, re.M)
    m = re.search(r"^Decode: (\d+) tokens in \d+\.\d+s \((\d+\.\d+) tok/s\)$", out, re.M)
    assert m and int(m.group(1)) == 3 * 8 and float(m.group(2)) > 0


def test_kernel_timing_tool_times_the_decode_kernels_alone():
    """Small sizes: the tool runs the kernels it names through the wrappers serving uses and prints a line for each."""
    out = run_tool("kernel_timing", "attention-decode", "--batch", 2, "--context", 700, "--pieces", 1, 4, 8, "--heads", 8,
                   "--kv-heads", 2)
    lines = re.findall(r"^attention_decode batch 2 context 700 pieces +(\d+): +(\d+\.\d+) us", out, re.M)
    assert [int(p) for p, _ in lines] == [1, 4, 8] and all(float(us) > 0 for _, us in lines)
    out = run_tool("kernel_timing", "product-chain", "--tokens", 5, "--hidden", 256, "--ff", 512)
    assert len(re.findall(r"^5 tokens, .*: +\d+\.\d+ us a link", out, re.M)) == 4


def test_bench_py_prints_its_line():
    """The measurement script itself, shortened: one JSON line with the keys its readers take."""
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "4", "--warmup", "3", "--no-points"],
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "prefill", "roofline", "clocks"):
        assert key in rec, key
    assert rec["n_gpus"] == 1 and rec["steps"] == 4 and rec["value"] > 0 and rec["gpu_launches"] > 0
    assert rec["e2e"]["value"] > 0 and rec["e2e"]["h2d_bytes_per_step"] > 0 and rec["e2e"]["d2h_bytes_per_step"] > 0
    assert rec["prefill"]["tokens"] == 2048 and 0 < rec["prefill"]["frac"] < 1.2 and 0 < rec["roofline"]["frac"] < 1.2
    assert len(rec["config"]) <= 20 and all(not isinstance(v, (list, dict)) for v in rec["config"].values())
