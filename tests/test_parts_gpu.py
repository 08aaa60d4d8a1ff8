"""Each part of a layer alone against the plain implementation's function for
it, then arrangements of parts: a run order that names a layer twice and lets
a layer read another's cache, the first tokens of a sequence, and a model
stored in 32-bit run in both modes."""
import numpy as np
import pytest
import torch

import plain_lfm2 as plain
import traces
from tiny_configs import CONFIGS, make_model
from tolerances import check_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = [torch.float32, torch.bfloat16]
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


def one_sequence_ctx(T, dtype, ctx_len=0, slot=0):
    from cellm_b200.parts import StepContext
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return StepContext(T=T, B=1, dtype=dtype, device=torch.device(DEV), token_ids=i32([0] * T),
                       positions=i32(list(range(ctx_len, ctx_len + T))), seq_of_token=i32([0] * T),
                       cu_seqlens=i32([0, T]), ctx_lens=i32([ctx_len]), slot_ids=i32([slot]),
                       err=torch.zeros(1, dtype=torch.int32, device=DEV), q_lens=[T], ctx_lens_host=[ctx_len],
                       max_q_len=T, max_total_len=ctx_len + T)


def rnd(*shape, scale=1.0, dtype=torch.float32):
    return (torch.randn(*shape, device=DEV) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DT)
def test_rms_norm_part_adds_what_is_pending(dtype):
    from cellm_b200.parts import Residual
    from cellm_b200.parts.norm import RMSNorm
    w = (torch.rand(72, device=DEV) + 0.5).to(dtype)
    part = RMSNorm({"dim": 72, "eps": 1e-4}, {"weight": w}, dtype)
    x = torch.randn(5, 72, device=DEV)
    d = rnd(5, 72, dtype=dtype)
    res = Residual(x.clone())
    res.add(d)
    y = part.forward(res)
    assert res.pending is None
    check_close(res.x.cpu(), (x.double() + d.double()).cpu(), "float32", "stream")
    check_close(y.float().cpu(), plain.rms_norm((x.double() + d.double()).cpu(), w.double().cpu(), 1e-4), NAME[dtype], "norm")


@pytest.mark.parametrize("dtype", DT)
def test_swiglu_part(dtype):
    from cellm_b200.parts.swiglu import SwiGLU
    H, ff = 40, 104
    w = {"w1": rnd(ff, H, scale=0.3, dtype=dtype), "w3": rnd(ff, H, scale=0.3, dtype=dtype), "w2": rnd(H, ff, scale=0.3, dtype=dtype)}
    part = SwiGLU({"hidden_size": H, "ff_dim": ff}, w, dtype)
    assert set(SwiGLU.weight_specs({"hidden_size": H, "ff_dim": ff})) == {"w1", "w2", "w3"}
    m = rnd(9, H, dtype=dtype)
    ref = plain.swiglu(m.double().cpu(), w["w1"].double().cpu(), w["w3"].double().cpu(), w["w2"].double().cpu())
    check_close(part.forward(m, one_sequence_ctx(9, dtype)).float().cpu(), ref, NAME[dtype])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("taps,bias", [(3, False), (4, True)])
def test_short_conv_part_in_two_portions(dtype, taps, bias):
    from cellm_b200.parts import CacheBinding
    from cellm_b200.parts.short_conv import ShortConvMixer
    H = 40
    params = {"hidden_size": H, "taps": taps, "bias": bias}
    w = {"in_proj": rnd(3 * H, H, scale=0.3, dtype=dtype), "conv": rnd(H, 1, taps, scale=0.5, dtype=dtype),
         "out_proj": rnd(H, H, scale=0.3, dtype=dtype)}
    if bias:
        w["conv_bias"] = rnd(H, scale=0.3, dtype=dtype)
    need = ShortConvMixer.cache_need(params)
    assert need.shape == (taps - 1, H) and need.dtype == torch.float32
    part = ShortConvMixer(params, w, dtype)
    state = torch.zeros(2, taps - 1, H, device=DEV)
    xn = rnd(11, H, dtype=dtype)
    cache = CacheBinding(need=need, state=state, num_slots=2)
    y = torch.cat([part.forward(xn[:2], one_sequence_ctx(2, dtype, 0, slot=1), cache),
                   part.forward(xn[2:], one_sequence_ctx(9, dtype, 2, slot=1), cache)])
    c = {k: v.double().cpu() for k, v in w.items()}
    ref = plain.short_conv_mixer(xn.double().cpu(), c["in_proj"], c["conv"], c["out_proj"], c.get("conv_bias"))
    check_close(y.float().cpu(), ref, NAME[dtype])
    assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (3, 1, 32, 0), (4, 4, 64, 7)])
def test_attention_part_in_two_portions(dtype, nh, nkv, hd, window):
    from cellm_b200.config import PartSpec
    from cellm_b200.parts import CacheBinding
    from cellm_b200.parts.attention import AttentionMixer
    H, ps, theta, eps = 48, 8, 5e4, 1e-5
    params = {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "scale": hd ** -0.5, "window": window,
              "qk_norm": PartSpec("rms_norm", {"dim": hd, "eps": eps}),
              "position": PartSpec("rope", {"head_dim": hd, "rotary_dim": hd, "theta": theta, "layout": "half"})}
    w = {"q_proj": rnd(nh * hd, H, scale=0.3, dtype=dtype), "k_proj": rnd(nkv * hd, H, scale=0.3, dtype=dtype),
         "v_proj": rnd(nkv * hd, H, scale=0.3, dtype=dtype), "out_proj": rnd(H, nh * hd, scale=0.3, dtype=dtype),
         "q_norm": (torch.rand(hd, device=DEV) + 0.5).to(dtype), "k_norm": (torch.rand(hd, device=DEV) + 0.5).to(dtype)}
    part = AttentionMixer(params, w, dtype)
    need = AttentionMixer.cache_need(params)
    assert (need.num_kv_heads, need.head_dim, need.window) == (nkv, hd, window)
    pages = 6
    kp = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    bt = torch.tensor([[4, 1, 5, 0]], dtype=torch.int32, device=DEV)
    cache = CacheBinding(need=need, k=kp, v=vp, block_table=bt, page_size=ps, num_pages=pages)
    xn = rnd(27, H, dtype=dtype)
    y = torch.cat([part.forward(xn[:13], one_sequence_ctx(13, dtype, 0), cache),
                   part.forward(xn[13:], one_sequence_ctx(14, dtype, 13), cache)])
    c = {k: v.double().cpu() for k, v in w.items()}
    ref, _ = plain.attention_mixer(xn.double().cpu(), c["q_proj"], c["k_proj"], c["v_proj"], c["out_proj"], c["q_norm"],
                                   c["k_norm"], n_heads=nh, n_kv=nkv, hd=hd, eps=eps, theta=theta, window=window)
    check_close(y.float().cpu(), ref, NAME[dtype])
    assert float(kp[2].float().abs().max()) == 0.0 and float(kp[3].float().abs().max()) == 0.0     # pages it was not given


def test_rope_part_describes_itself():
    from cellm_b200.config import ConfigError
    from cellm_b200.parts.rope import RotaryEmbedding
    r = RotaryEmbedding({"head_dim": 32, "rotary_dim": 16, "theta": 100.0, "layout": "interleaved"}, DEV)
    rot, inter, inv = r.rotation()
    assert rot == 16 and inter and inv.dtype == torch.float32 and tuple(inv.shape) == (8, 2)
    exact = 100.0 ** (-(2.0 * torch.arange(8, dtype=torch.float64)) / 16)
    assert float((inv.cpu().double().sum(1) - exact).abs().max()) < 1e-15
    with pytest.raises(ConfigError):
        RotaryEmbedding({"head_dim": 32, "rotary_dim": 34, "theta": 100.0}, DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_names_a_layer_twice_and_shares_a_cache(tmp_path, dtype):
    """Order [0, 1, 2, 2, 3, {4 reading the cache of the first 2}, 5]: layer 2 runs
    twice with a cache for each run; layer 4 computes no keys of its own."""
    from cellm_b200.replay import Replayer
    order = [0, 1, 2, 2, 3, {"layer": 4, "cache_of": 2}, 5]
    folder = make_model(tmp_path, "tiny_b", overrides={"layer_order": order})
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(3)
    reqs = {"a": rng.integers(0, 1000, 50).tolist(), "b": rng.integers(0, 1000, 21).tolist()}
    plain_order = [0, 1, 2, 2, 3, (4, 2), 5]
    ref = {r: plain.forward(cfg, w, t, order=plain_order).numpy() for r, t in reqs.items()}
    for make in (traces.whole, traces.portions, traces.mixed):
        steps = make(reqs)
        rp = Replayer(folder, dtype, traces.max_live_tokens(steps), 16, 4)
        assert len(rp.cache.k_pools) == 1 and rp.cache.k_pools[0].shape[0] == 3      # two runs of layer 2, and layer 5
        got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
        for r, t in reqs.items():
            check_close(traces.as_matrix(got[r], len(t)), ref[r], dtype, f"{make.__name__} {r}")


def test_a_conv_layer_cannot_borrow_a_cache(tmp_path):
    from cellm_b200.config import ConfigError
    from cellm_b200.replay import Replayer
    folder = make_model(tmp_path, "tiny_b", overrides={"layer_order": [0, {"layer": 1, "cache_of": 0}, 2, 3, 4, 5]})
    with pytest.raises(ConfigError, match="cannot read another item's cache"):
        Replayer(folder, "float32", 64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_first_tokens_of_a_sequence(tmp_path, name, dtype):
    """Sequences of one, two and three tokens, and a long one fed one token at a
    time from the very start: history before the first token is zero, the first
    token attends to itself alone."""
    from cellm_b200.replay import Replayer
    folder = make_model(tmp_path, name)
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(8)
    rp = Replayer(folder, dtype, 256, 8, 4)
    for n in (1, 2, 3):
        toks = rng.integers(0, cfg["vocab_size"], n).tolist()
        out = rp.step([{"id": f"s{n}", "tokens": toks, "want": list(range(n))}], [f"s{n}"])
        check_close(out, plain.forward(cfg, w, toks).numpy(), dtype, f"{n} tokens")
    toks = rng.integers(0, cfg["vocab_size"], 12).tolist()
    outs = [rp.step([{"id": "one", "tokens": [t], "want": [0]}], []) for t in toks]
    check_close(np.concatenate(outs), plain.forward(cfg, w, toks).numpy(), dtype, "token by token from the start")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_stored_in_32_bit(tmp_path, dtype):
    """Tensors stored in 32-bit stay 32-bit: in the bfloat16 mode the matrices then
    run the 32-bit product on widened activations."""
    from cellm_b200.replay import Replayer
    folder = make_model(tmp_path, "tiny_a", dtype="float32")
    cfg, w = plain.load_folder(folder)
    toks = np.random.default_rng(9).integers(0, 512, 40).tolist()
    rp = Replayer(folder, dtype, 64, 8)
    assert rp.model.embedding.weight.dtype == torch.float32
    out = rp.step([{"id": "a", "tokens": toks, "want": list(range(40))}], ["a"])
    check_close(out, plain.forward(cfg, w, toks).numpy(), dtype)


def test_max_layers_runs_a_prefix(tmp_path):
    from cellm_b200.engine import StepEntry
    from cellm_b200.replay import Replayer
    folder = make_model(tmp_path, "tiny_b")
    cfg, w = plain.load_folder(folder)
    toks = np.random.default_rng(1).integers(0, 1000, 20).tolist()
    rp = Replayer(folder, "float32", 64)
    rp.cache.add(0)
    out = rp.runner.run([StepEntry(0, toks, list(range(20)))], max_layers=3).cpu().numpy()
    check_close(out, plain.forward(cfg, w, toks, order=[0, 1, 2]).numpy(), "float32")
