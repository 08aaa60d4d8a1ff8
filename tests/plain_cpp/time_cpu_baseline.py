#!/usr/bin/env python3
"""The timed CPU baseline: the plain C++ restatement of jeffasante/cellm's CPU LFM path
(crates/cellm-model/src/lfm.rs:263-763, non-Metal branches), in 32-bit as the reference computes, one
token at a time on one core, on a model of a given shape with random weights.

This is NOT a run of the reference (a Rust workspace; no Rust toolchain exists on this machine): it is this
repository's own restatement of the reference's formulas and loop structure (scalar inner products, a cache
that grows by one token), and every line it prints says so. It gives the only context beside the roofline
for the GPU engine's numbers.

    python tests/plain_cpp/time_cpu_baseline.py [--shape lfm2-1.2b] [--prompt 4] [--gen 4]

prints one JSON line: prefill and decode tokens a second of the restatement on this host's CPU.
"""
import argparse
import ctypes
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="lfm2-1.2b", help="a shape of cellm_b200.config.presets, or a config.json")
    ap.add_argument("--prompt", type=int, default=4)
    ap.add_argument("--gen", type=int, default=4)
    args = ap.parse_args()
    import numpy as np
    import torch
    import plain_lfm2 as plain
    from cellm_b200.config.presets import shape
    from cellm_b200.weights import write_random_model
    config = json.load(open(args.shape)) if os.path.isfile(args.shape) else shape(args.shape)
    cxx = shutil.which("g++") or shutil.which("c++")
    with tempfile.TemporaryDirectory(prefix="cpu_baseline_") as d:
        so = os.path.join(d, "libplain.so")
        subprocess.run([cxx, "-O3", "-march=native", "-std=c++17", "-fPIC", "-shared", "-o", so,
                        os.path.join(HERE, "plain_lfm2.cc")], check=True)
        lib = ctypes.CDLL(so)
        folder = write_random_model(os.path.join(d, "m"), config, seed=0, dtype="bfloat16")
        from safetensors.torch import load_file
        cfg = json.load(open(os.path.join(folder, "config.json")))
        w = {k: v.to(torch.float32).contiguous() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}

        class Config(ctypes.Structure):
            _fields_ = [(n, ctypes.c_int) for n in ("vocab", "hidden", "layers", "heads", "kv_heads", "head_dim", "ff", "taps")] + \
                       [("eps", ctypes.c_double), ("theta", ctypes.c_double)]
        types = plain.layer_types(cfg)
        L = cfg["num_hidden_layers"]
        c = Config(cfg["vocab_size"], cfg["hidden_size"], L, cfg["num_attention_heads"], cfg["num_key_value_heads"],
                   plain.head_dim(cfg), plain.feed_forward_size(cfg), int(cfg.get("conv_L_cache", 3)),
                   plain.norm_eps(cfg), float(cfg.get("rope_theta", 1e6)))
        p = lambda name: w[name].data_ptr() if name in w else None
        tied = cfg.get("tie_embedding", cfg.get("tie_word_embeddings", True))
        ptrs = [p("model.embed_tokens.weight"), p("model.embedding_norm.weight"), None if tied else p("lm_head.weight")]
        for l in range(L):
            q = f"model.layers.{l}."
            ptrs += [p(q + n) for n in ("operator_norm.weight", "ffn_norm.weight", "feed_forward.w1.weight", "feed_forward.w2.weight",
                                        "feed_forward.w3.weight", "conv.in_proj.weight", "conv.conv.weight", "conv.conv.bias",
                                        "conv.out_proj.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                        "self_attn.v_proj.weight", "self_attn.out_proj.weight", "self_attn.q_layernorm.weight",
                                        "self_attn.k_layernorm.weight")]
        arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
        kinds = (ctypes.c_int * L)(*[0 if t == "conv" else 1 for t in types])
        rng = np.random.default_rng(0)
        lib.plain_lfm2_forward_f32.restype = ctypes.c_int

        def run(n):
            ids = rng.integers(0, cfg["vocab_size"], n).tolist()
            out = np.empty((n, cfg["vocab_size"]), dtype=np.float32)
            t0 = time.perf_counter()
            rc = lib.plain_lfm2_forward_f32(ctypes.byref(c), arr, kinds, (ctypes.c_int * n)(*ids), n, out.ctypes.data_as(ctypes.c_void_p))
            assert rc == 0 and np.isfinite(out).all()
            return time.perf_counter() - t0
        run(1)                                  # pages the weights in
        t_prompt = run(args.prompt)
        t_all = run(args.prompt + args.gen)     # the restatement keeps no cache between calls: the prompt is fed again
        t_gen = max(t_all - t_prompt, 1e-9)
    print(json.dumps({
        "what": "plain C++ restatement of jeffasante/cellm's CPU LFM path in 32-bit, one core, one token at a time; NOT a run of the reference",
        "shape": args.shape, "layers": L, "host_cpu_threads_used": 1,
        "prefill_tokens": args.prompt, "prefill_tok_s": round(args.prompt / t_prompt, 3),
        "decode_tokens": args.gen, "decode_tok_s": round(args.gen / t_gen, 3)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
