#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM2 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: LFM2-1.2B layer sizes, random bfloat16 weights, 8 requests with
2,048-token random prompts in a cache sized for 8,192 tokens per request. A
"step" is one decode step of the whole batch. One JSON line is printed:
`value` = decoded tokens a second timed on the device, `e2e` = the same through
the Python entry point with host tokens in and out (Engine.step(): every step uploads
its index arrays from pinned memory and every step's tokens are read on the host; with
EngineConfig.run_ahead, the default, a step's tokens are read after the next step has been
launched, which takes them from the device), `prefill` = one 2,048-token
prompt, `roofline` = the bytes a decode step has to read over its time,
`points` = decoding at batch 1 and 64.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from cellm_b200.config.presets import LFM2_SHAPES  # noqa: E402

# The benchmark's model: layers of LFM2-1.2B's sizes.
LFM2_1P2B = LFM2_SHAPES["lfm2-1.2b"]
CONTEXT_LEN = 8192
PROMPT_LEN = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except (ValueError, KeyError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons through NVML while a region is timed (read-only)."""

    def __init__(self, period=0.05):
        super().__init__(daemon=True)
        self.period, self.samples, self.reasons, self.max_mhz = period, [], set(), None
        self._stop = threading.Event()
        self.active = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
        while not self._stop.is_set():
            if self.active.is_set():
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def param_count(plan_tensors) -> int:
    return sum(int(t.numel()) for t in plan_tensors)


def decode_setup(loaded, batch, total_blocks, rng):
    """An engine with `batch` requests that have all finished their 2,048-token prompts."""
    import torch
    from cellm_b200 import Engine, SamplingParams
    eng = Engine(loaded, dtype="bfloat16", tokens_per_block=PAGE, total_blocks=total_blocks, max_num_seqs=batch,
                 max_batch_tokens=max(4096, batch), prefill_chunk=2048)
    V = eng.plan.vocab_size
    params = SamplingParams.greedy(CONTEXT_LEN - PROMPT_LEN, stop_eos=False)
    ids = [eng.add_request(rng.integers(0, V, PROMPT_LEN).tolist(), params) for _ in range(batch)]
    while any(eng.scheduler.info(r)["state"] != "decoding" for r in ids):
        eng.step()
    torch.cuda.synchronize()
    return eng, ids


def time_decode(eng, ids, steps, warmup, rng, sampler=None):
    """(device ms per step, e2e ms per step, launches per step, h2d bytes, d2h bytes, context at the end)."""
    import torch
    from cellm_b200 import ops
    from cellm_b200.engine import StepEntry
    from cellm_b200.ops._lib import LAUNCHES
    B = len(ids)
    # end to end through the entry point: host tokens in, host tokens out
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    if sampler:
        sampler.active.set()
    import gc
    gc.collect()
    gc.disable()            # a collection inside the timed steps would be charged to one of them
    t0 = time.perf_counter()
    for _ in range(steps):
        out = eng.step()
        assert len(out) == B
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    gc.enable()
    # device-timed: the step function and the arg-max on given tokens, no read back
    V = eng.plan.vocab_size
    toks = rng.integers(0, V, (warmup + steps, B))
    def device_step(i):
        # the step function and the arg-max of its logits (inside the step's graph where there is one)
        logits = eng.runner.run([StepEntry(r, [int(toks[i, b])], [0]) for b, r in enumerate(ids)])
        return eng.runner.last_argmax if eng.runner.last_argmax is not None else ops.argmax(logits)
    for i in range(warmup):
        device_step(i)
    torch.cuda.synchronize()
    l0 = LAUNCHES[0]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(warmup, warmup + steps):
        device_step(i)
    e1.record()
    torch.cuda.synchronize()
    if sampler:
        sampler.active.clear()
    dev_ms = e0.elapsed_time(e1) / steps
    launches = (LAUNCHES[0] - l0) // steps
    ctx = eng.cache.tokens(ids[0])
    width = (ctx + PAGE - 1) // PAGE
    n_groups = len(eng.cache.paged_keys)
    h2d = 4 * (3 * B + (B + 1) + 2 * B + B + n_groups * B * width)
    d2h = 4 * B
    eng.runner.check()
    return dev_ms, e2e_ms, launches, h2d, d2h, ctx


def time_prefill(loaded, rng, reps=5, warmup=3):
    import torch
    from cellm_b200.cache import CacheManager
    from cellm_b200.engine import StepEntry, StepRunner
    cfg, plan, model = loaded
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in plan.order], PAGE, PROMPT_LEN // PAGE + 1, 1,
                         model.dtype, model.device)
    runner = StepRunner(model, cache)
    toks = rng.integers(0, plan.vocab_size, PROMPT_LEN).tolist()
    times = []
    for i in range(warmup + reps):
        cache.add(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.run([StepEntry(i, toks, [PROMPT_LEN - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.release(i)
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    runner.check()
    return sorted(times)[len(times) // 2]


def profile_region(loaded, args, rng) -> int:
    """One decode step of the batch (launched kernel by kernel, no graph) or one
    prefill (2,048 tokens unless --profile-tokens says fewer) between cudaProfilerStart and cudaProfilerStop."""
    import torch
    from cellm_b200.engine import StepEntry
    if args.profile_region == "decode":
        eng, ids = decode_setup(loaded, args.batch, args.batch * CONTEXT_LEN // PAGE, rng)
        eng.runner.use_graphs = False
        V = eng.plan.vocab_size
        step = lambda: eng.runner.run([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in ids])
    else:
        from cellm_b200.cache import CacheManager
        from cellm_b200.engine import StepRunner
        cfg, plan, model = loaded
        cache = CacheManager(model.cache_needs(), [e.cache_of for e in plan.order], PAGE, 4 * (PROMPT_LEN // PAGE + 1), 4,
                             model.dtype, model.device)
        runner = StepRunner(model, cache)
        n_tok = max(1, min(args.profile_tokens, PROMPT_LEN))
        toks = rng.integers(0, plan.vocab_size, n_tok).tolist()
        counter = [0]

        def step():
            cache.add(counter[0])
            runner.run([StepEntry(counter[0], toks, [n_tok - 1])])
            counter[0] += 1
    for _ in range(max(args.warmup, 1)):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"profiled one {args.profile_region} step")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 runs")
    ap.add_argument("--profile-region", choices=["decode", "prefill"], default=None,
                    help="for a profiler started with --profile-from-start off: run the set-up, then one eager "
                         "decode step (or one prefill) between cudaProfilerStart/Stop, print no bench line")
    ap.add_argument("--profile-tokens", type=int, default=PROMPT_LEN,
                    help="with --profile-region prefill: the prompt's length (the bench line's prefill is always 2,048)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "jeffasante/cellm is a Rust workspace (no setup.py/pyproject.toml; pip: 'not installable') "
                          "and no Rust toolchain exists offline; its GPU path is Apple Metal"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch
    from cellm_b200 import write_random_model
    from cellm_b200.models import load_model
    from cellm_b200.weights import InitSpec

    rng = np.random.default_rng(0)
    pk, pk_src = peaks()
    t_setup = time.time()
    with tempfile.TemporaryDirectory(prefix="cellm_bench_") as d:
        # the benchmark's weights: N(0, 0.02), norm weights 1
        write_random_model(d, LFM2_1P2B, seed=0, dtype="bfloat16", init=InitSpec(norm_jitter=0.0))
        loaded = load_model(d, "bfloat16", "cuda:0")
    cfg, plan, model = loaded
    n_layers = cfg.num_hidden_layers
    weight_bytes = 0
    seen = set()
    for blk in model.blocks:
        for part in (blk.mixer, blk.feed_forward):
            for v in vars(part).values():
                w = getattr(v, "weight", None)
                if isinstance(w, torch.Tensor) and w.data_ptr() not in seen:
                    seen.add(w.data_ptr())
                    weight_bytes += w.numel() * w.element_size()
    weight_bytes += model.head.weight.numel() * model.head.weight.element_size()
    print(f"[bench] model ready in {time.time() - t_setup:.1f}s, matrix weights {weight_bytes / 1e9:.3f} GB", file=sys.stderr)

    if args.profile_region:
        return profile_region(loaded, args, rng)

    sampler = ClockSampler()
    sampler.start()
    B = args.batch
    eng, ids = decode_setup(loaded, B, B * CONTEXT_LEN // PAGE, rng)
    dev_ms, e2e_ms, launches, h2d, d2h, ctx = time_decode(eng, ids, args.steps, args.warmup, rng, sampler)
    kv_bytes_tok = eng.cache.bytes_per_token()
    run_ahead = bool(eng.config.run_ahead)
    for r in ids:
        eng.cancel(r)
    del eng
    torch.cuda.empty_cache()

    # bytes a decode step has to read: every weight once, and the cache of the live requests
    mean_ctx = ctx - args.steps / 2
    step_bytes = weight_bytes + B * mean_ctx * kv_bytes_tok
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9

    sampler.active.set()
    pf_ms = time_prefill(loaded, rng)
    sampler.active.clear()
    H, ff, V = cfg.hidden_size, cfg.ff_dim, cfg.vocab_size
    A, KV = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    lin = len(cfg.conv_layers) * (3 * H * H + H * H) + len(cfg.attention_layers) * ((A + 2 * KV) * H + H * A) \
        + n_layers * 3 * ff * H
    flops = 2 * PROMPT_LEN * lin + len(cfg.attention_layers) * 4 * A * PROMPT_LEN * PROMPT_LEN / 2 + 2 * V * H
    pf_frac = flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)

    points = {}
    if not args.no_points:
        for b in (1, 64):
            e, r = decode_setup(loaded, b, b * CONTEXT_LEN // PAGE, rng)
            n_steps = max(8, args.steps // 2)
            ms, _, _, _, _, c_end = time_decode(e, r, n_steps, args.warmup, rng)
            points[f"decode_b{b}"] = round(b / (ms * 1e-3), 1)
            # the same roofline as the main run's: weights once and the live requests' cache, over the step's time
            b_bytes = weight_bytes + b * (c_end - n_steps / 2) * kv_bytes_tok
            points[f"decode_b{b}_ms"] = round(ms, 4)
            points[f"decode_b{b}_hbm_frac"] = round(b_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            for x in r:
                e.cancel(x)
            del e
            torch.cuda.empty_cache()
    sampler.stop()

    value = B / (dev_ms * 1e-3)
    line = {
        "metric": "LFM2-1.2B decode tok/s @bs 8 (device-timed), with prefill tok/s @2048 and % of roofline",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random-init weights N(0,0.02)",
        "impl": "ours",
        "config": {"model": "LFM2-1.2B shape", "layers": n_layers, "layers_of_config": 16, "hidden": H,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "ff_dim": ff, "vocab": V, "conv_L_cache": cfg.conv_L_cache, "attn_layers": len(cfg.attention_layers),
                   "global_batch": B, "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN, "decode_ctx_end": int(ctx),
                   "kv_page": PAGE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: %.2f GB of weights read every step" % (weight_bytes / 1e9),
                   "peaks": pk_src},
        "e2e": {"value": round(B / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "tokens_read": "every step's, one step late: the next step is launched first" if run_ahead
                               else "every step's, before the next step is planned"},
        "gpu_launches": int(launches * args.steps),
        "prefill": {"value": round(PROMPT_LEN / (pf_ms * 1e-3), 1), "tokens": PROMPT_LEN, "ms": round(pf_ms, 3),
                    "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_src},
        "points": points,
        "clocks": sampler.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
