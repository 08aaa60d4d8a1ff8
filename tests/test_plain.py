"""The plain implementation checked against itself: each part's defining
property, so that it can serve as the reference for the engine."""
import math

import numpy as np
import torch

import plain_lfm2 as plain
from tiny_configs import make_model


def test_rms_norm_and_rope_properties():
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.rand(12, dtype=torch.float64) + 0.5
    y = plain.rms_norm(x, w, 0.0)
    assert torch.allclose((y / w).pow(2).mean(-1), torch.ones(5, dtype=torch.float64))
    q = torch.randn(6, 3, 8, dtype=torch.float64)
    pos = torch.arange(10, 16)
    r = plain.rope_rotate_half(q, pos, 100.0)
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1))                     # a rotation
    assert torch.allclose(plain.rope_rotate_half(q, torch.zeros(6, dtype=torch.long), 100.0), q)
    # the score of a rotated pair depends on the distance only
    k = torch.randn(6, 3, 8, dtype=torch.float64)
    a = (plain.rope_rotate_half(q[:1], torch.tensor([7]), 100.0) * plain.rope_rotate_half(k[:1], torch.tensor([3]), 100.0)).sum()
    b = (plain.rope_rotate_half(q[:1], torch.tensor([14]), 100.0) * plain.rope_rotate_half(k[:1], torch.tensor([10]), 100.0)).sum()
    assert abs(float(a - b)) < 1e-9
    # pairing (i, i + half) with angle pos * theta^(-2i/d): one hand-computed element
    d, p, th = 8, 5, 100.0
    ang = p * th ** (-2 * 1 / d)
    h = q[0, 0]
    assert abs(float(plain.rope_rotate_half(q[:1], torch.tensor([p]), th)[0, 0, 1]) - float(h[1] * math.cos(ang) - h[5] * math.sin(ang))) < 1e-12


def test_short_conv_is_causal_and_equals_the_token_loop():
    torch.manual_seed(0)
    T, H, ks = 9, 6, 4
    xn = torch.randn(T, H, dtype=torch.float64)
    w_in, w_c = torch.randn(3 * H, H, dtype=torch.float64), torch.randn(H, 1, ks, dtype=torch.float64)
    w_out, bias = torch.randn(H, H, dtype=torch.float64), torch.randn(H, dtype=torch.float64)
    y = plain.short_conv_mixer(xn, w_in, w_c, w_out, bias)
    # the reference's one-token loop with a shifting state (crates/cellm-model/src/lfm.rs:388-398)
    state = torch.zeros(ks, H, dtype=torch.float64)
    for t in range(T):
        bcx = w_in @ xn[t]
        bx = bcx[:H] * bcx[2 * H:]
        state = torch.cat([state[1:], bx[None]])
        conv = (state * w_c.reshape(H, ks).T).sum(0) + bias
        assert torch.allclose(w_out @ (bcx[H:2 * H] * conv), y[t])
    y2 = plain.short_conv_mixer(torch.cat([xn[:5], torch.randn(4, H, dtype=torch.float64)]), w_in, w_c, w_out, bias)
    assert torch.allclose(y2[:5], y[:5])


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(1)
    T, H, nh, nkv, hd = 12, 16, 4, 2, 8
    xn = torch.randn(T, H, dtype=torch.float64)
    mk = lambda *s: torch.randn(*s, dtype=torch.float64) * 0.3
    wq, wk, wv, wo = mk(nh * hd, H), mk(nkv * hd, H), mk(nkv * hd, H), mk(H, nh * hd)
    qn, kn = torch.rand(hd, dtype=torch.float64) + 0.5, torch.rand(hd, dtype=torch.float64) + 0.5
    kw = dict(n_heads=nh, n_kv=nkv, hd=hd, eps=1e-5, theta=1e4)
    out, (k, v) = plain.attention_mixer(xn, wq, wk, wv, wo, qn, kn, **kw)
    out2, _ = plain.attention_mixer(torch.cat([xn[:7], mk(5, H)]), wq, wk, wv, wo, qn, kn, **kw)
    assert torch.allclose(out[:7], out2[:7])                                   # later tokens do not matter
    assert torch.allclose(out[0], (v[0].repeat_interleave(nh // nkv, 0).reshape(-1)) @ wo.T)   # first token sees itself only
    win, _ = plain.attention_mixer(xn, wq, wk, wv, wo, qn, kn, window=3, **kw)
    assert torch.allclose(win[:3], out[:3]) and not torch.allclose(win[5], out[5])
    tail, _ = plain.attention_mixer(xn[3:], wq, wk, wv, wo, qn, kn, window=3, pos0=3, **kw)
    assert torch.allclose(tail[2:], win[5:], atol=1e-12)                       # a window forgets what lies before it


def test_forward_prefix_property_and_order_list(tmp_path):
    folder = make_model(tmp_path, "tiny_b")
    cfg, w = plain.load_folder(folder)
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"], 30).tolist()
    full = plain.forward(cfg, w, ids)
    assert full.shape == (30, 1000)
    assert torch.allclose(plain.forward(cfg, w, ids[:11]), full[:11], atol=1e-12)
    assert torch.equal(plain.forward(cfg, w, ids, order=list(range(6))), full)
    twice = plain.forward(cfg, w, ids, order=[0, 1, 2, 2, 3, (4, 2), 5])
    assert not torch.allclose(twice, full)


def test_sampler_follows_select_next():
    rng = plain.XorShift64(1234)
    seq = [rng.next_u64() for _ in range(3)]
    x = 1234
    for v in seq:      # shifts 13, 7, 17 (tools/infer/src/main.rs:1031-1037)
        x ^= (x << 13) & (2 ** 64 - 1); x ^= x >> 7; x ^= (x << 17) & (2 ** 64 - 1)
        assert v == x
    assert plain.XorShift64(0).s == 1
    logits = torch.tensor([0.1, 2.0, float("nan"), 2.0, -1.0, 1.5])
    c = plain.top_k_candidates(logits, 3)
    assert [i for i, _ in c] == [1, 3, 5]                                       # ties keep ascending ids, nan is -inf
    assert plain.select_next(c, 0.0, 1.0, 64, [], rng) == 1
    assert [i for i, _ in plain.top_k_candidates(logits, 0)] == [0, 1, 2, 3, 4, 5]
    counts = {1: 0, 3: 0, 5: 0}
    for _ in range(3000):
        counts[plain.select_next(c, 1.0, 1.0, 64, [], rng)] += 1
    p = torch.softmax(torch.tensor([2.0, 2.0, 1.5]), 0)
    assert abs(counts[1] / 3000 - float(p[0])) < 0.04 and abs(counts[5] / 3000 - float(p[2])) < 0.04
    pen = {1: 0, 3: 0, 5: 0}
    for _ in range(3000):
        pen[plain.select_next(c, 1.0, 2.0, 4, [9, 9, 1], rng)] += 1             # token 1 was seen: its score halves
    assert pen[1] < counts[1] * 0.7


def _cpp_forward(lib, cfg, w, ids):
    """Logits of the C++ restatement (tests/plain_cpp/plain_lfm2.cc) for tensors `w` (float64)."""
    import ctypes

    class Config(ctypes.Structure):
        _fields_ = [(n, ctypes.c_int) for n in ("vocab", "hidden", "layers", "heads", "kv_heads", "head_dim", "ff", "taps")] + \
                   [("eps", ctypes.c_double), ("theta", ctypes.c_double)]
    types = plain.layer_types(cfg)
    L = cfg["num_hidden_layers"]
    c = Config(cfg["vocab_size"], cfg["hidden_size"], L, cfg["num_attention_heads"], cfg["num_key_value_heads"],
               plain.head_dim(cfg), plain.feed_forward_size(cfg), int(cfg.get("conv_L_cache", 3)),
               plain.norm_eps(cfg), float(cfg.get("rope_theta", 1e6)))
    keep = []

    def p(name):
        t = w.get(name)
        if t is None:
            return None
        t = t.to(torch.float64).contiguous()
        keep.append(t)
        return t.data_ptr()
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
    ids_c = (ctypes.c_int * len(ids))(*ids)
    out = np.empty((len(ids), cfg["vocab_size"]), dtype=np.float64)
    lib.plain_lfm2_forward.restype = ctypes.c_int
    rc = lib.plain_lfm2_forward(ctypes.byref(c), arr, kinds, ids_c, len(ids), out.ctypes.data_as(ctypes.c_void_p))
    assert rc == 0
    return out


def test_cpp_restatement_agrees_with_the_python_one(tmp_path):
    """Two restatements of the reference's formulas, written apart (whole sequences in
    torch; token by token with a growing cache in C++), give the same logits on both
    tiny configurations: a slip in reading the reference would have to be made twice."""
    import ctypes
    import os
    import shutil
    import subprocess
    cxx = shutil.which("g++") or shutil.which("c++")
    assert cxx, "a host C++ compiler is needed"
    so = str(tmp_path / "libplain_cpp.so")
    src = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_cpp", "plain_lfm2.cc")
    subprocess.run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-o", so, src], check=True)
    lib = ctypes.CDLL(so)
    for name in ("tiny_a", "tiny_b"):
        cfg, w = plain.load_folder(make_model(tmp_path, name))
        ids = np.random.default_rng(3).integers(0, cfg["vocab_size"], 41).tolist()
        a = plain.forward(cfg, w, ids).numpy()
        b = _cpp_forward(lib, cfg, w, ids)
        assert np.abs(a - b).max() < 1e-10 * (1 + np.abs(a).max()), name
