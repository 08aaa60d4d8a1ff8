"""Plain, slow LFM2 for tests: whole sequences, no cache, one function per part.

This file rests on the formulas of jeffasante/cellm's CPU LFM path (the Rust
model code cannot be compiled on a machine without a Rust toolchain, so there
is no run of the original behind these functions). Each function cites the
lines of the reference that it restates. Three things the reference lacks are
defined here and marked "(addition)": the convolution bias, the untied
lm_head, and the feed-forward size adjustment.

It shares no code with the package: it reads tensors with the `safetensors`
library, works on whole sequences with torch on the CPU (float64 by default),
and keeps no cache of any kind. A second restatement, token by token in C++
(tests/plain_cpp/plain_lfm2.cc), is compared with this one in test_plain.py.
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------
# configuration (plain dict from config.json)
# --------------------------------------------------------------------------

def feed_forward_size(cfg: dict) -> int:
    """(addition) Width of the SwiGLU hidden layer.

    The reference takes the width from the converted weights
    (tools/convert_lfm.py:150-159). With `block_auto_adjust_ff_dim` the
    config's `intermediate_size` is first cut to two thirds, scaled by
    `block_ffn_dim_multiplier`, then rounded up to `block_multiple_of`.
    """
    ff = int(cfg["intermediate_size"])
    if cfg.get("block_auto_adjust_ff_dim", False):
        ff = int(2 * ff / 3)
        mult = cfg.get("block_ffn_dim_multiplier", None)
        if mult is not None:
            ff = int(mult * ff)
        m = int(cfg.get("block_multiple_of", 256))
        ff = m * ((ff + m - 1) // m)
    return ff


def layer_types(cfg: dict) -> list[str]:
    """crates/cellm-model/src/lfm.rs:95-114 (list from the config);
    `full_attn_idxs` is the older spelling of the same information."""
    if "layer_types" in cfg and cfg["layer_types"] is not None:
        return list(cfg["layer_types"])
    idx = set(cfg["full_attn_idxs"])
    return ["full_attention" if i in idx else "conv" for i in range(cfg["num_hidden_layers"])]


def head_dim(cfg: dict) -> int:
    """crates/cellm-model/src/lfm.rs:130-142: header value, else H / heads."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def norm_eps(cfg: dict) -> float:
    return float(cfg.get("norm_eps", cfg.get("rms_norm_eps", 1e-5)))


def load_folder(folder: str):
    """config.json as a dict and all tensors as float64 CPU tensors."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return cfg, {k: v.to(torch.float64) for k, v in tensors.items()}


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """crates/cellm-model/src/lfm.rs:817-890: row gather, no scaling."""
    if int(ids.max()) >= table.shape[0] or int(ids.min()) < 0:
        raise ValueError("token id out of range")
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """crates/cellm-kernels/src/cpu_kernels.rs:17-34 over the last axis:
    ms = sum(x^2)/n; out = x / sqrt(ms + eps) * w; the weight is used as is
    (crates/cellm-model/src/lfm.rs:337 passes w_add_one = false)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(ms + eps)) * w


def rope_rotate_half(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """crates/cellm-kernels/src/cpu_kernels.rs:264-277 with rotary_dim =
    head_dim (crates/cellm-model/src/lfm.rs:553-559). x: [T, heads, hd]."""
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=x.dtype)
    inv_freq = theta ** (-(2.0 * i) / hd)
    ang = pos.to(x.dtype)[:, None] * inv_freq[None, :]          # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)


def short_conv_mixer(xn, w_in, w_conv, w_out, bias=None):
    """crates/cellm-model/src/lfm.rs:350-417 for a whole sequence.

    xn [T,H]; w_in [3H,H]; w_conv [H,1,ks] or [H,ks]; w_out [H,H].
    bcx = W_in xn, split B | C | x (:363-365); bx = B*x (:368-371); the state
    holds the last ks columns of bx with zeros before the first token, and
    tap ks-1 meets the current token (:388-398); y = C*conv (:402-405);
    out = W_out y (:408-414). (addition) `bias` [H] is added to conv.
    """
    T, H = xn.shape
    wc = w_conv.reshape(H, -1)
    ks = wc.shape[1]
    bcx = xn @ w_in.T
    B, C, xt = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    bx = B * xt
    hist = torch.cat([torch.zeros(ks - 1, H, dtype=xn.dtype), bx], dim=0)
    conv = torch.zeros(T, H, dtype=xn.dtype)
    for k in range(ks):
        conv = conv + hist[k:k + T] * wc[:, k][None, :]
    if bias is not None:
        conv = conv + bias[None, :]
    return (C * conv) @ w_out.T


def attention_mixer(xn, wq, wk, wv, wo, q_norm_w, k_norm_w, *, n_heads, n_kv, hd, eps,
                    theta, window=0, pos0=0, kv_from=None):
    """crates/cellm-model/src/lfm.rs:418-601 for a whole sequence.

    q,k,v projections without bias (:446-483); RMSNorm of each q and k head
    over hd (:486-543); rotate-half RoPE at the token's position (:553-559);
    head h reads key/value head h // (n_heads / n_kv) and scores are
    q.k / sqrt(hd) over every earlier token and itself
    (crates/cellm-cache/src/kvcache.rs:753-787), softmax with the maximum
    taken off (:1206-1227). `window` > 0 (not an LFM2 option; it serves the
    engine's windowed cache group) keeps only the last `window` keys.
    `kv_from` = (k, v) of another layer replaces this layer's own keys.
    Returns (out, (k, v)).
    """
    T = xn.shape[0]
    pos = torch.arange(pos0, pos0 + T)
    q = (xn @ wq.T).reshape(T, n_heads, hd)
    q = rope_rotate_half(rms_norm(q, q_norm_w, eps), pos, theta)
    if kv_from is None:
        k = (xn @ wk.T).reshape(T, n_kv, hd)
        v = (xn @ wv.T).reshape(T, n_kv, hd)
        k = rope_rotate_half(rms_norm(k, k_norm_w, eps), pos, theta)
    else:
        k, v = kv_from
    g = n_heads // n_kv
    out = torch.zeros(T, n_heads, hd, dtype=xn.dtype)
    scale = 1.0 / math.sqrt(hd)
    ti = torch.arange(T)
    allowed = ti[None, :] <= ti[:, None]
    if window and window > 0:
        allowed = allowed & (ti[None, :] > ti[:, None] - window)
    for h in range(n_heads):
        kh, vh = k[:, h // g], v[:, h // g]
        s = (q[:, h] @ kh.T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h] = p @ vh
    return out.reshape(T, n_heads * hd) @ wo.T, (k, v)


def swiglu(m, w1, w3, w2):
    """crates/cellm-model/src/lfm.rs:631-662: g = W1 m, u = W3 m,
    g*sigmoid(g)*u, then W2."""
    g = m @ w1.T
    u = m @ w3.T
    return (g * (1.0 / (1.0 + torch.exp(-g))) * u) @ w2.T


# --------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------

def forward(cfg: dict, w: dict, ids, order=None, window=0, hidden_out=None, rows=None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence (crates/cellm-model/src/lfm.rs:
    263-763: pre-norm block :333-347, residual :610-612, ffn_norm :615-629,
    residual :665-667, embedding_norm :670-687, tied output :689-757).

    `order` is the list of layers to run, each item `layer` or
    `(layer, cache_of)` where cache_of is the index in `order` of an earlier
    attention item whose keys and values this item reads instead of its own.
    (addition) an untied `lm_head.weight` is used when `tie_embedding` is false.
    `rows`: form the logits of these positions only ([len(rows), V]).
    """
    dt = next(iter(w.values())).dtype
    ids = torch.as_tensor(ids)
    types = layer_types(cfg)
    H = cfg["hidden_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim(cfg)
    eps = norm_eps(cfg)
    theta = float(cfg.get("rope_theta", 1e6))
    x = embedding(w["model.embed_tokens.weight"], ids).to(dt)
    if order is None:
        order = list(range(cfg["num_hidden_layers"]))
    kv_of_item = {}
    for item_index, item in enumerate(order):
        l, cache_of = (item, None) if isinstance(item, int) else item
        p = f"model.layers.{l}."
        xn = rms_norm(x, w[p + "operator_norm.weight"], eps)
        if types[l] == "conv":
            mix = short_conv_mixer(xn, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"],
                                   w[p + "conv.out_proj.weight"], w.get(p + "conv.conv.bias"))
        elif types[l] in ("full_attention", "attention"):
            mix, kv = attention_mixer(
                xn, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                w[p + "self_attn.v_proj.weight"], w[p + "self_attn.out_proj.weight"],
                w[p + "self_attn.q_layernorm.weight"], w[p + "self_attn.k_layernorm.weight"],
                n_heads=nh, n_kv=nkv, hd=hd, eps=eps, theta=theta, window=window,
                kv_from=None if cache_of is None else kv_of_item[cache_of])
            kv_of_item[item_index] = kv
        else:
            raise ValueError(f"unknown layer type {types[l]!r}")
        x = x + mix
        m = rms_norm(x, w[p + "ffn_norm.weight"], eps)
        x = x + swiglu(m, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                       w[p + "feed_forward.w2.weight"])
    if hidden_out is not None:
        hidden_out.append(x)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    xf = rms_norm(x, w["model.embedding_norm.weight"], eps)
    tied = cfg.get("tie_embedding", cfg.get("tie_word_embeddings", True))
    head = w["model.embed_tokens.weight"] if tied else w["lm_head.weight"]
    return xf @ head.T


# --------------------------------------------------------------------------
# sampling, as tools/infer does it
# --------------------------------------------------------------------------

class XorShift64:
    """tools/infer/src/main.rs:1025-1045: shifts 13, 7, 17; next_f32 is the
    top 24 bits over 2^24. Seed 0 becomes 1 (`seed.max(1)`)."""

    def __init__(self, seed: int):
        self.s = max(int(seed) & 0xFFFFFFFFFFFFFFFF, 1)

    def next_u64(self) -> int:
        x = self.s
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        self.s = x
        return x

    def next_f32(self) -> float:
        return float(self.next_u64() >> 40) / float(1 << 24)


def top_k_candidates(logits: torch.Tensor, k: int):
    """crates/cellm-model/src/lfm.rs:806-815: non-finite to -inf, stable sort
    by logit descending (equal logits keep ascending ids), first k.
    (addition) k <= 0 keeps the whole vocabulary in the order of the ids."""
    v = logits.to(torch.float32).clone()
    v[~torch.isfinite(v)] = float("-inf")
    if k and k > 0:
        order = torch.sort(v, descending=True, stable=True).indices[:k]
    else:
        order = torch.arange(v.numel())
    return [(int(i), float(v[i])) for i in order]


def select_next(cands, temperature, repeat_penalty, repeat_window, recent, rng) -> int:
    """tools/infer/src/main.rs:958-1016 in float32 steps."""
    import numpy as np

    if temperature <= 0.0:
        return max(cands, key=lambda c: (c[1], -c[0]))[0]
    ids = [c[0] for c in cands]
    scores = np.array([c[1] for c in cands], dtype=np.float32)
    if repeat_penalty > 1.0 and repeat_window > 0 and len(recent) > 0:
        tail = set(recent[-repeat_window:])
        for i, t in enumerate(ids):
            if t in tail:
                scores[i] = np.float32(scores[i] / np.float32(repeat_penalty))
    mx = scores.max()
    wts = np.exp((scores - mx) / np.float32(temperature)).astype(np.float32)
    total = np.float32(0.0)
    for x in wts:
        total = np.float32(total + x)
    if total == 0.0:
        return ids[0]
    r = np.float32(np.float32(rng.next_f32()) * total)
    acc = np.float32(0.0)
    for i, x in enumerate(wts):
        acc = np.float32(acc + x)
        if r <= acc:
            return ids[i]
    return ids[-1]


def generate(cfg, w, prompt, n_new, temperature=0.0, top_k=0, seed=1,
             repeat_penalty=1.0, repeat_window=64, stop_eos=False):
    """Whole-sequence recomputation for every new token (no cache)."""
    toks = list(prompt)
    rng = XorShift64(seed)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, toks)[-1]
        nxt = select_next(top_k_candidates(logits, top_k), temperature, repeat_penalty,
                          repeat_window, toks, rng)
        out.append(nxt)
        toks.append(nxt)
        if stop_eos and cfg.get("eos_token_id") is not None and nxt == cfg["eos_token_id"]:
            break
    return out
