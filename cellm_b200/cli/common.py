"""Shared pieces of the command lines."""
from __future__ import annotations

import json
import tempfile


def parse_tokens(s: str) -> list[int]:
    """Comma-separated token ids (tools/infer/src/main.rs:1047-1060)."""
    out = [int(p.strip()) for p in s.split(",") if p.strip()]
    if not out:
        raise SystemExit("--tokens parsed to empty list")
    return out


def resolve_model(args) -> str:
    """The model folder: --model, or a folder of random weights made from --random."""
    if args.model:
        return args.model
    if not args.random:
        raise SystemExit("give --model DIR or --random CONFIG.json")
    from ..weights import write_random_model
    with open(args.random) as f:
        cfg = json.load(f)
    folder = tempfile.mkdtemp(prefix="cellm_random_")
    write_random_model(folder, cfg, args.weights_seed, "float32" if args.dtype in ("float32", "fp32") else "bfloat16")
    print(f"random weights (seed {args.weights_seed}) written to {folder}")
    return folder


def add_model_options(ap) -> None:
    ap.add_argument("--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="CONFIG.json", help="make a model with random weights from this configuration")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"],
                    help="bfloat16: serving kernels; float32: the whole model in true 32-bit")
    ap.add_argument("--max-layers", type=int, default=None, help="run only the first N layers (debug)")
    ap.add_argument("--tokens-per-block", type=int, default=16, help="tokens per KV block")
    ap.add_argument("--total-blocks", type=int, default=None, help="total KV blocks (default: from seq+gen)")


def default_blocks(seq: int, gen: int, tokens_per_block: int, batch: int = 1) -> int:
    """tools/infer/src/main.rs:381-384: ceil((seq + gen + 8) / tokens_per_block), per request."""
    return batch * ((seq + gen + 8 + tokens_per_block - 1) // tokens_per_block)
