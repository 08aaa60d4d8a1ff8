"""`kernel_timing`: kernels of the decode step timed alone, as chains in a CUDA graph, on random data.
The executor's rules (how many pieces the keys of a request are cut into, how a product's K is split) were set
from these timings; the tool repeats them on the GPU at hand.

  attention-decode   the decode attention at a batch and context for several counts of pieces; the caches of
                     the timed calls rotate so that L2 does not hold them
  product-chain      chains of the decode step's products and norms with a layer's sizes (--hidden, --ff),
                     each link reading the one before it; 16 different weight matrices in turn

The reference has no counterpart (its kernels are timed through tools/bench only).
"""
from __future__ import annotations

import argparse


def _time_graph(run, per: int, reps: int = 10) -> float:
    """Microseconds per item: `run` launches `per` items; it is captured once and replayed."""
    import torch
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps / per * 1e3


def attention_decode(args) -> int:
    import torch
    from ..ops.attention import attention_decode as kernel
    dev = "cuda:0"
    nh, nkv, hd, ps, B, ctx = args.heads, args.kv_heads, args.head_dim, args.tokens_per_block, args.batch, args.context
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    pages_req = (ctx + 1 + ps - 1) // ps
    kv_bytes = B * (ctx + 1) * nkv * hd * 2 * 2
    n_caches = max(2, min(24, int(300e6 // kv_bytes) + 1))          # more than L2 holds
    caches = [(torch.randn(B * pages_req, nkv, ps, hd, device=dev).bfloat16(),
               torch.randn(B * pages_req, nkv, ps, hd, device=dev).bfloat16()) for _ in range(n_caches)]
    width = -(-pages_req // 32) * 32
    bt = torch.full((B, width), -1, dtype=torch.int32, device=dev)
    for b in range(B):
        bt[b, :pages_req] = torch.arange(b * pages_req, (b + 1) * pages_req, dtype=torch.int32, device=dev)
    q = torch.randn(B, nh * hd, device=dev).bfloat16()
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    blocks = (ctx + 1 + 63) // 64
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for pieces in args.pieces or [1, 2, 4, 8, 9, 16, 18, 24, 32, 48, 64, 72]:
        if pieces > blocks or pieces * B * nkv > 16 * sms:
            continue

        def run():
            for k, v in caches:
                kernel(q, k, v, cu, lens, bt, B, nh, hd ** -0.5, 0, err, pieces)
        us = _time_graph(run, n_caches, 5)
        print(f"attention_decode batch {B} context {ctx} pieces {pieces:3d}: {us:8.2f} us  {kv_bytes / us / 1e3:6.0f} GB/s", flush=True)
    if err.item() != 0:
        raise RuntimeError(f"device error word {err.item()}")
    return 0


def product_chain(args) -> int:
    import torch
    from .. import ops
    from ..ops import gemm_bf16 as tc
    dev = "cuda:0"
    H, FF, M, L = args.hidden, args.ff, args.tokens, 16
    gen = torch.Generator(device=dev).manual_seed(0)
    mk = lambda n, k: [(torch.randn(n, k, device=dev, generator=gen) * 0.02).bfloat16() for _ in range(L)]
    w13, w2, w_in, w_out = mk(2 * FF, H), mk(H, FF), mk(3 * H, H), mk(H, H)
    gain = torch.ones(H, device=dev).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    xs = torch.randn(M, H, device=dev, generator=gen)
    first = (torch.randn(M, H, device=dev, generator=gen) * 0.01).bfloat16()

    def product(a, w, epilogue=0):
        bn, split = tc.plan_tiles(a.shape[0], w.shape[0], a.shape[1], sms)
        if epilogue and bn == 64:
            bn = 128
        return tc.gemm_tcgen05(a, w, torch.bfloat16, bn, split, err, epilogue, True)

    def norms():
        pend = first
        for _ in range(L):
            pend = ops.add_rmsnorm(xs, pend, gain, 1e-5, torch.bfloat16)

    def out_proj():
        y = first
        for i in range(L):
            y = product(y, w_out[i])

    def mixer():
        pend = first
        for i in range(L):
            y = ops.add_rmsnorm(xs, pend, gain, 1e-5, torch.bfloat16)
            pend = product(product(y, w_in[i])[:, :H], w_out[i])

    def feed_forward():
        pend = first
        for i in range(L):
            y = ops.add_rmsnorm(xs, pend, gain, 1e-5, torch.bfloat16)
            pend = product(product(y, w13[i], 1), w2[i])

    stream = lambda nbytes: nbytes / 6.5562e6          # microseconds at 6,556 GB/s
    for name, run, nbytes in (("add_rmsnorm", norms, 0), ("out_proj", out_proj, H * H * 2),
                              ("norm + in_proj + out_proj", mixer, 4 * H * H * 2),
                              ("norm + w1|w3 + w2", feed_forward, 3 * FF * H * 2)):
        us = _time_graph(run, L)
        print(f"{M} tokens, {name}: {us:6.2f} us a link" + (f" ({stream(nbytes):.1f} us of streaming)" if nbytes else ""), flush=True)
    if err.item() != 0:
        raise RuntimeError(f"device error word {err.item()}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_timing", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    a = sub.add_parser("attention-decode")
    a.add_argument("--batch", type=int, default=8)
    a.add_argument("--context", type=int, default=2048)
    a.add_argument("--pieces", type=int, nargs="*", default=None)
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=64)
    a.add_argument("--tokens-per-block", type=int, default=16)
    c = sub.add_parser("product-chain")
    c.add_argument("--tokens", type=int, default=8)
    c.add_argument("--hidden", type=int, default=2048)
    c.add_argument("--ff", type=int, default=8192)
    args = ap.parse_args(argv)
    return attention_decode(args) if args.what == "attention-decode" else product_chain(args)


if __name__ == "__main__":
    raise SystemExit(main())
