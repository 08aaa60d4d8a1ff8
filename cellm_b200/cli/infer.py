"""`infer`: generate from one prompt, with the options of the reference's tool
of that name (tools/infer/src/main.rs:40-135). Token ids in, token ids out; a
tokenizer.json may be given to work on text."""
from __future__ import annotations

import argparse
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="infer", description="Inference for an LFM2 model folder on one B200")
    from .common import add_model_options, default_blocks, parse_tokens, resolve_model
    add_model_options(ap)
    ap.add_argument("--tokenizer", help="path to a HuggingFace tokenizer.json (needed with --prompt)")
    ap.add_argument("--prompt", help="prompt text (uses the tokenizer to encode and decode)")
    ap.add_argument("--seq", type=int, default=8, help="prompt length (token ids 0..seq-1 unless --tokens)")
    ap.add_argument("--gen", type=int, default=8, help="number of generated tokens")
    ap.add_argument("--temperature", type=float, default=0.8, help="sampling temperature (0 = greedy)")
    ap.add_argument("--top-k", type=int, default=40, help="sample from the top K tokens (0 = all)")
    ap.add_argument("--seed", type=int, default=None, help="RNG seed for sampling")
    ap.add_argument("--repeat-penalty", type=float, default=1.05, help="repetition penalty (1.0 disables)")
    ap.add_argument("--repeat-window", type=int, default=64, help="recent token window for the penalty")
    ap.add_argument("--tokens", help="comma-separated token ids (overrides --seq)")
    ap.add_argument("--stop-eos", type=lambda s: s.lower() not in ("0", "false", "no"), default=True,
                    help="stop when the EOS token is produced")
    args = ap.parse_args(argv)

    from .. import Engine, SamplingParams
    t0 = time.time()
    folder = resolve_model(args)
    tok = None
    if args.prompt is not None:
        if not args.tokenizer:
            raise SystemExit("--prompt needs --tokenizer")
        from tokenizers import Tokenizer
        tok = Tokenizer.from_file(args.tokenizer)
        prompt = tok.encode(args.prompt).ids
    elif args.tokens:
        prompt = parse_tokens(args.tokens)
    else:
        prompt = list(range(args.seq))
    blocks = args.total_blocks or default_blocks(len(prompt), args.gen, args.tokens_per_block)
    eng = Engine(folder, dtype=args.dtype, tokens_per_block=args.tokens_per_block, total_blocks=blocks, max_num_seqs=1)
    eng.max_layers = args.max_layers
    print(f"Startup: {time.time() - t0:.2f}s  KV cache: blocks={blocks} tokens_per_block={args.tokens_per_block}")
    seed = args.seed if args.seed is not None else (time.time_ns() & 0xFFFFFFFFFFFF)   # seed from the clock, as the reference
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, seed=seed,
                            repeat_penalty=args.repeat_penalty, repeat_window=args.repeat_window,
                            max_new_tokens=args.gen, stop_eos=args.stop_eos)
    rid = eng.add_request(prompt, params)
    t1 = time.time()
    out: list[int] = []
    first = None
    while eng.has_unfinished():
        for _, t in eng.step():
            if first is None:
                first = time.time()
                print(f"Prefill: {len(prompt)} tokens in {first - t1:.2f}s")
            out.append(t)
    t2 = time.time()
    n_dec = max(len(out) - 1, 0)
    if first is not None and n_dec:
        print(f"Decode: {n_dec} tokens in {t2 - first:.2f}s ({n_dec / max(t2 - first, 1e-9):.2f} tok/s)")
    print("tokens:", ",".join(str(t) for t in out))
    if tok is not None:
        print(tok.decode(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
