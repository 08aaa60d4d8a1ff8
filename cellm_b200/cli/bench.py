"""`bench`: prefill then greedy decode, timed, with the options and output
lines of the reference's tool (tools/bench/src/main.rs:27-63, :177, :194),
plus --batch for several equal requests at once."""
from __future__ import annotations

import argparse
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bench", description="Prefill / decode timing for an LFM2 model folder")
    from .common import add_model_options, default_blocks, resolve_model
    add_model_options(ap)
    ap.add_argument("--seq", type=int, default=16, help="prompt length (token ids 0..seq-1)")
    ap.add_argument("--gen", type=int, default=32, help="number of generated tokens")
    ap.add_argument("--top-k", type=int, default=40, help="kept for the reference's interface; decoding is greedy")
    ap.add_argument("--batch", type=int, default=1, help="equal requests run together")
    args = ap.parse_args(argv)

    import torch
    from .. import Engine, SamplingParams
    folder = resolve_model(args)
    blocks = args.total_blocks or default_blocks(args.seq, args.gen, args.tokens_per_block, args.batch)
    eng = Engine(folder, dtype=args.dtype, tokens_per_block=args.tokens_per_block, total_blocks=blocks,
                 max_num_seqs=args.batch, max_batch_tokens=max(2048, args.batch))
    eng.max_layers = args.max_layers
    V = eng.plan.vocab_size
    print(f"KV cache: blocks={blocks} tokens_per_block={args.tokens_per_block}")
    params = SamplingParams.greedy(args.gen, stop_eos=False)
    for b in range(args.batch):
        eng.add_request([(i + b) % V for i in range(args.seq)], params)
    torch.cuda.synchronize()
    t0 = time.time()
    produced = 0
    while produced < args.batch and eng.has_unfinished():
        produced += len(eng.step())
    torch.cuda.synchronize()
    t1 = time.time()
    print(f"Prefill: {args.seq * args.batch} tokens in {t1 - t0:.2f}s")
    n = 0
    while eng.has_unfinished():
        n += len(eng.step())
    torch.cuda.synchronize()
    t2 = time.time()
    print(f"Decode: {n} tokens in {t2 - t1:.2f}s ({n / max(t2 - t1, 1e-9):.2f} tok/s)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
