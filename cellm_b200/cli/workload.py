"""`workload`: serving workloads through the engine's scheduler with random
weights of a named LFM2 shape, timed end to end (host tokens in and out).

  continuous    many requests with prompts of random length arrive at once and
                are served by the continuous scheduler until each has its tokens
  long-context  one long prompt is fed in portions beside decoding requests
                that were already running

The reference's bench tool times one prompt and one decode loop
(tools/bench/src/main.rs:177, :194); these two have no counterpart there.
"""
from __future__ import annotations

import argparse
import json
import tempfile
import time


def _load(shape_name: str, dtype: str):
    from ..config.presets import shape
    from ..models import load_model
    from ..weights import InitSpec, write_random_model
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, shape(shape_name), seed=0, dtype="bfloat16", init=InitSpec(norm_jitter=0.0))
        return load_model(d, dtype, "cuda:0")


def continuous(args) -> dict:
    import numpy as np
    import torch
    from .. import Engine, SamplingParams
    loaded = _load(args.shape, args.dtype)
    rng = np.random.default_rng(args.seed)
    V = loaded[1].vocab_size
    lens = rng.integers(args.prompt_min, args.prompt_max + 1, args.requests).tolist()
    page = args.tokens_per_block
    need = sum(-(-(n + args.gen) // page) for n in lens)
    pages = args.total_blocks or need + 8
    eng = Engine(loaded, dtype=args.dtype, tokens_per_block=page, total_blocks=pages, max_num_seqs=args.requests,
                 max_batch_tokens=args.max_batch_tokens, prefill_chunk=args.prefill_chunk, run_ahead=not args.no_run_ahead)
    prompts = [rng.integers(0, V, n).tolist() for n in lens]
    eng.generate([p[:64] for p in prompts[:2]], SamplingParams.greedy(4, stop_eos=False))     # warm-up: loads the kernels
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(prompts, SamplingParams.greedy(args.gen, stop_eos=False))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.stats()
    return {"workload": "continuous", "shape": args.shape, "dtype": args.dtype, "requests": args.requests,
            "prompt_tokens": int(sum(lens)), "generated_tokens": sum(len(o) for o in outs), "seconds": round(dt, 3),
            "generated_tok_s": round(sum(len(o) for o in outs) / dt, 1),
            "total_tok_s": round((sum(lens) + sum(len(o) for o in outs)) / dt, 1),
            "pages": pages, "pages_needed_at_once": need, "preemptions": st["preemptions"], "steps": st["steps_run"]}


def long_context(args) -> dict:
    import numpy as np
    import torch
    from .. import Engine, SamplingParams
    loaded = _load(args.shape, args.dtype)
    rng = np.random.default_rng(args.seed)
    V = loaded[1].vocab_size
    page = args.tokens_per_block
    ctxs = rng.integers(args.prompt_min, args.prompt_max + 1, args.requests).tolist()
    steps_long = -(-args.long_prompt // args.prefill_chunk)
    gen = steps_long + 64           # the streams outlast the long prompt
    need = sum(-(-(n + gen) // page) for n in ctxs) + -(-(args.long_prompt + 8) // page)
    eng = Engine(loaded, dtype=args.dtype, tokens_per_block=page, total_blocks=args.total_blocks or need + 8,
                 max_num_seqs=args.requests + 1, max_batch_tokens=args.prefill_chunk + args.requests,
                 prefill_chunk=args.prefill_chunk, run_ahead=not args.no_run_ahead)
    params = SamplingParams.greedy(gen, stop_eos=False)
    streams = [eng.add_request(rng.integers(0, V, n).tolist(), params) for n in ctxs]
    while any(eng.scheduler.info(r)["state"] != "decoding" for r in streams):
        eng.step()                  # the streams' own prompts are not part of the measurement
    torch.cuda.synchronize()
    before = sum(len(eng.output(r).tokens) for r in streams)
    t0 = time.perf_counter()
    long_id = eng.add_request(rng.integers(0, V, args.long_prompt).tolist(), SamplingParams.greedy(1, stop_eos=False))
    n_steps = 0
    while not eng.output(long_id).finished:
        eng.step()
        n_steps += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    decoded = sum(len(eng.output(r).tokens) for r in streams) - before
    for r in streams:
        eng.cancel(r)
    return {"workload": "long-context", "shape": args.shape, "dtype": args.dtype, "long_prompt": args.long_prompt,
            "portion": args.prefill_chunk, "streams": args.requests, "stream_contexts": [int(min(ctxs)), int(max(ctxs))],
            "seconds": round(dt, 3), "steps": n_steps, "prompt_tok_s": round(args.long_prompt / dt, 1),
            "decoded_beside": decoded, "decode_tok_s_beside": round(decoded / dt, 1),
            "ms_per_step": round(1e3 * dt / max(n_steps, 1), 2)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="workload", description=__doc__.split("\n\n")[0])
    ap.add_argument("workload", choices=["continuous", "long-context"])
    ap.add_argument("--shape", default=None, help="lfm2-1.2b | lfm2-2.6b | lfm2-700m (default: 2.6b / 700m by workload)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--requests", type=int, default=None, help="requests (continuous: 32) or decoding streams (long-context: 16)")
    ap.add_argument("--prompt-min", type=int, default=None)
    ap.add_argument("--prompt-max", type=int, default=None)
    ap.add_argument("--gen", type=int, default=256, help="tokens generated per request (continuous)")
    ap.add_argument("--long-prompt", type=int, default=32768, help="tokens of the long prompt (long-context)")
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--max-batch-tokens", type=int, default=4096)
    ap.add_argument("--tokens-per-block", type=int, default=16)
    ap.add_argument("--total-blocks", type=int, default=None, help="pages (default: what all requests need at once)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-run-ahead", action="store_true",
                    help="read every step's tokens before the next step is planned (EngineConfig.run_ahead = False)")
    args = ap.parse_args(argv)
    cont = args.workload == "continuous"
    args.shape = args.shape or ("lfm2-2.6b" if cont else "lfm2-700m")
    args.requests = args.requests or (32 if cont else 16)
    args.prompt_min = args.prompt_min or (128 if cont else 1024)
    args.prompt_max = args.prompt_max or (4096 if cont else 8192)
    print(json.dumps(continuous(args) if cont else long_context(args)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
