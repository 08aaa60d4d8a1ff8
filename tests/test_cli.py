"""The command lines' option handling, on the CPU: names, defaults and the small
helpers, without loading a model."""
import json
import os
import subprocess
import sys

import pytest

from cellm_b200.cli.common import default_blocks, parse_tokens
from cellm_b200.config.presets import LFM2_SHAPES, shape

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_parse_tokens_and_default_blocks():
    assert parse_tokens("1, 2,3") == [1, 2, 3] and parse_tokens("7") == [7]
    with pytest.raises(SystemExit):
        parse_tokens(" , ")
    with pytest.raises(ValueError):
        parse_tokens("1,x")
    # tools/infer/src/main.rs:381-384: ceil((seq + gen + 8) / tokens_per_block), per request
    assert default_blocks(8, 8, 16) == 2 and default_blocks(16, 32, 16) == 4 and default_blocks(16, 32, 16, batch=3) == 12


@pytest.mark.parametrize("tool,options", [
    ("infer", ["--model", "--tokens", "--seq", "--gen", "--temperature", "--top-k", "--seed", "--repeat-penalty",
               "--repeat-window", "--max-layers", "--tokens-per-block", "--total-blocks", "--stop-eos", "--dtype", "--random",
               "--tokenizer", "--prompt"]),
    ("bench", ["--model", "--seq", "--gen", "--top-k", "--batch", "--tokens-per-block", "--total-blocks", "--dtype"]),
    ("workload", ["continuous", "long-context", "--shape", "--requests", "--prompt-min", "--prompt-max", "--gen",
                  "--long-prompt", "--prefill-chunk", "--max-batch-tokens", "--total-blocks"]),
    ("trace_run", ["--model", "--dtype", "--out", "--max-tokens"]),
    ("kernel_timing", ["attention-decode", "product-chain"]),
])
def test_tools_offer_their_options(tool, options):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", tool), "--help"], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    for o in options:
        assert o in p.stdout, f"{tool} --help does not name {o}"


def test_infer_wants_a_model():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer")], capture_output=True, text=True, timeout=120)
    assert p.returncode != 0 and "--model" in (p.stderr + p.stdout)


def test_bench_py_refuses_more_than_one_gpu_and_names_the_missing_reference():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert p.returncode == 2 and len(p.stdout.strip().splitlines()) == 1
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True, text=True, timeout=120)
    line = json.loads(p.stdout)
    assert p.returncode == 0 and line["impl"] == "reference" and "unavailable" in line


def test_shapes_of_the_family():
    from cellm_b200.config import config_from_dict
    want = {"lfm2-1.2b": (16, 8192, 6), "lfm2-2.6b": (30, 7168, 8), "lfm2-700m": (16, 6912, 6)}
    for name, (layers, ff, attn) in want.items():
        cfg, plan = config_from_dict(shape(name))
        assert len(plan.order) == layers and cfg.ff_dim == ff
        assert sum(1 for t in cfg.layer_types if t != "conv") == attn
    assert shape("LFM2-1.2B") == LFM2_SHAPES["lfm2-1.2b"]
    with pytest.raises(ValueError, match="known"):
        shape("lfm2-9b")
