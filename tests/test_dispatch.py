"""Which kernels a step of a given shape launches, and with which tile shapes, on the CPU: the
entry points are replaced by recorders (launch_recorder.py), the model has LFM2-1.2B's layer sizes
(one convolution layer, one attention layer) and zero weights."""
import pytest
import torch

from launch_recorder import Recorder, run_step, zero_model

WIDE = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": 65536, "hidden_size": 2048,
        "num_hidden_layers": 2, "layer_types": ["conv", "full_attention"], "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 12288, "block_auto_adjust_ff_dim": True,
        "block_multiple_of": 256, "rope_theta": 1e6, "conv_L_cache": 3, "norm_eps": 1e-5, "tie_embedding": True,
        "max_position_embeddings": 128000}
H, FF, V = 2048, 8192, 65536
# positions of the arguments in the entry points' signatures
G_M, G_N, G_K, G_OUT, G_BN, G_SPLIT, G_EPI, G_WS = 3, 4, 5, 9, 10, 11, 12, 14


def test_decode_step(monkeypatch):
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(WIDE)
    run_step(model, plan, [1] * 8, [2048] * 8)
    assert rec.names() == [
        "cellm_embed",
        "cellm_add_rmsnorm", "cellm_gemm_conv_tcgen05", "cellm_gemm_tcgen05",                     # conv mixer: in_proj + conv, out_proj
        "cellm_add_rmsnorm", "cellm_gemm_tcgen05", "cellm_gemm_tcgen05",                          # feed-forward: w1|w3 + SwiGLU, w2
        "cellm_add_rmsnorm", "cellm_gemm_rope_tcgen05", "cellm_attention_decode", "cellm_gemm_tcgen05",     # q/k/v + norm + rotation + cache write
        "cellm_add_rmsnorm", "cellm_gemm_tcgen05", "cellm_gemm_tcgen05",
        "cellm_add_rmsnorm", "cellm_gemm_tcgen05"]                                                # final norm on the wanted rows, head
    gemms = rec.of("cellm_gemm_tcgen05")
    assert [(g[G_M], g[G_N], g[G_K]) for g in gemms] == [(8, H, H), (8, 2 * FF, H), (8, H, FF), (8, H, H),
                                                          (8, 2 * FF, H), (8, H, FF), (8, V, H)]
    assert all(g[G_BN] == -16 for g in gemms)                      # swapped tiles of 16 tokens
    assert [g[G_EPI] for g in gemms] == [0, 1, 0, 0, 1, 0, 0]
    rope = rec.of("cellm_gemm_rope_tcgen05")[0]
    assert (rope[3], rope[4]) == (8, H) and rope[7] == -16 and 1 <= rope[8] <= 8 and (rope[19], rope[20]) == (32, 8)
    assert all(1 <= g[G_SPLIT] <= 8 and g[G_WS] is None for g in gemms[:-1])      # the K split stays inside a cluster
    assert gemms[-1][G_SPLIT] == 1 and gemms[-1][G_OUT] == 0       # the head has tiles to spare; 32-bit logits
    conv = rec.of("cellm_gemm_conv_tcgen05")[0]
    assert (conv[3], conv[4], conv[5], conv[8], conv[13]) == (8, 49 * 128, H, H, 3) and conv[9] == -16
    dec = rec.of("cellm_attention_decode")[0]
    assert (dec[11], dec[12]) == (8, 8) and 2 <= dec[20] <= 8 and dec[1] is None      # keys split over the CTAs of a cluster


def test_decode_attention_pieces_by_batch_and_context(monkeypatch):
    """How many pieces the keys of a request are cut into: one cluster of up to 8 for short contexts, a multiple
    of 8 (clusters of eight, a piece per cluster through the workspace) where few requests have long contexts,
    and what fills four CTAs an SM otherwise."""
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(WIDE)
    for lens, want in (([2048], 8), ([4096], 32), ([8192], 64), ([32768], 72), ([8192] * 2, 32), ([32768] * 8, 9),
                       ([2048] * 64, 1)):
        rec.calls.clear()
        run_step(model, plan, [1] * len(lens), lens)
        dec = rec.of("cellm_attention_decode")[0]
        assert dec[20] == want, (lens, dec[20])
        assert (dec[1] is not None) == (want > 8)                  # a workspace only beyond one cluster


def test_decode_step_without_the_fused_decode_kernels(monkeypatch):
    from cellm_b200.runtime import program
    monkeypatch.setitem(program.OPTIONS, "fused_rope", False)
    monkeypatch.setitem(program.OPTIONS, "fused_conv", False)
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(WIDE)
    run_step(model, plan, [1] * 3, [10, 500, 4000])
    names = rec.names()
    assert "cellm_gemm_rope_tcgen05" not in names and "cellm_qk_norm_rope" in names
    assert "cellm_short_conv" in names and "cellm_gemm_conv_tcgen05" not in names
    assert rec.of("cellm_short_conv")[0][15] == 1                  # the one-launch form for single tokens
    assert [(g[G_M], g[G_N]) for g in rec.of("cellm_gemm_tcgen05")][:2] == [(3, 3 * H), (3, H)]


def test_prompt_step(monkeypatch):
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(WIDE)
    run_step(model, plan, [2048], [0])
    names = rec.names()
    assert "cellm_gemm_conv_tcgen05" not in names and "cellm_attention_decode" not in names
    assert names.count("cellm_attention_tc") == 1 and names.count("cellm_short_conv") == 1
    gemms = rec.of("cellm_gemm_tcgen05")
    body, head = gemms[:-1], gemms[-1]
    assert all(g[G_M] == 2048 and 128 <= g[G_BN] <= 256 and g[G_SPLIT] == 1 for g in body)     # plain tiles, persistent kernel
    assert [g[G_BN] for g in body] == [240, 240, 256, 240, 176, 240, 256, 240]                  # widths that fill the waves of 148 SMs
    assert [g[G_EPI] for g in body] == [0, 0, 1, 0, 0, 0, 1, 0]
    assert (head[G_M], head[G_N]) == (1, V) and head[G_BN] == -16                               # one wanted row
    assert rec.of("cellm_short_conv")[0][15] == 2048


def test_mixed_step(monkeypatch):
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(WIDE)
    run_step(model, plan, [1, 40, 1, 300], [77, 16, 500, 0])
    names = rec.names()
    assert names.count("cellm_attention_flash") + names.count("cellm_attention_tc") == 1
    assert "cellm_attention_decode" not in names and "cellm_attention_plain" not in names
    assert "cellm_gemm_conv_tcgen05" not in names                  # a portion of several tokens: product, then convolution
    gemms = rec.of("cellm_gemm_tcgen05")
    assert all(g[G_M] == 342 for g in gemms[:-1]) and gemms[-1][G_M] == 4
    for g in gemms[:-1]:
        if g[G_SPLIT] > 1 and g[G_BN] > 0:
            assert g[G_WS] is not None                             # plain tiles with a K split go through the workspace


def test_32_bit_model_runs_no_tensor_core_kernel(monkeypatch):
    rec = Recorder(monkeypatch)
    small = dict(WIDE, vocab_size=1000, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                 intermediate_size=512, block_auto_adjust_ff_dim=False)
    cfg, plan, model = zero_model(small, torch.float32)
    run_step(model, plan, [1, 9], [5, 0])
    names = set(rec.names())
    assert names == {"cellm_embed", "cellm_add_rmsnorm", "cellm_gemm_plain", "cellm_short_conv", "cellm_qk_norm_rope",
                     "cellm_attention_plain", "cellm_swiglu"}


def test_widths_off_the_tensor_core_kernels_rules_take_the_plain_product(monkeypatch):
    rec = Recorder(monkeypatch)
    odd = dict(WIDE, vocab_size=777, hidden_size=100, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
               intermediate_size=130, block_auto_adjust_ff_dim=False)
    cfg, plan, model = zero_model(odd)
    run_step(model, plan, [1, 1], [3, 40])
    names = rec.names()
    assert "cellm_gemm_conv_tcgen05" not in names                  # in_proj has K = 100
    assert "cellm_attention_plain" in names and "cellm_swiglu" in names       # heads of 16; a feed-forward of 130
    plain_k = sorted({g[5] for g in rec.of("cellm_gemm_plain")})
    assert plain_k == [100, 130]                                   # the width and the feed-forward: no multiples of 8
    assert {g[G_K] for g in rec.of("cellm_gemm_tcgen05")} == {80}  # out_proj of the attention: 5 heads of 16


def test_patches_are_put_back():
    assert torch.zeros(1).is_cuda is False


def test_step_runner_builds_the_step_and_runs_it(monkeypatch):
    """The step function itself on the CPU (pinned staging and events replaced by stand-ins): entries are
    checked, pages reserved, the index arrays laid out, the model run on exactly the given tokens, lengths
    committed."""
    from cellm_b200.cache.manager import CacheManager
    from cellm_b200.engine.step import StepEntry, StepRunner
    rec = Recorder(monkeypatch)
    small = dict(WIDE, vocab_size=1000, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                 intermediate_size=512, block_auto_adjust_ff_dim=False)
    cfg, plan, model = zero_model(small)
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in plan.order], 16, 8, 2, model.dtype, "cpu")
    runner = StepRunner(model, cache, use_graphs=False)
    monkeypatch.setattr(runner, "_staging", lambda n: torch.empty(max(n, 4096), dtype=torch.int32))
    monkeypatch.setattr(runner, "_uploaded", lambda: None)
    cache.add(7)
    cache.add(9)
    logits = runner.run([StepEntry(7, [1, 2, 3], [0, 2]), StepEntry(9, [5], [])])
    assert tuple(logits.shape) == (2, 1000) and cache.tokens(7) == 3 and cache.tokens(9) == 1
    embed = rec.of("cellm_embed")[0]
    assert embed[4] == 4                                            # four tokens in the step
    rec.calls.clear()
    assert runner.run([StepEntry(7, [4], [])]) is None and cache.tokens(7) == 4        # nothing wanted: no head product
    assert rec.names()[-1] != "cellm_gemm_tcgen05" or rec.of("cellm_gemm_tcgen05")[-1][G_N] != 1000
    with pytest.raises(ValueError, match="twice"):
        runner.run([StepEntry(7, [1], [0]), StepEntry(7, [2], [0])])
    with pytest.raises(ValueError, match="vocabulary"):
        runner.run([StepEntry(9, [1000], [0])])
    from cellm_b200.cache.manager import OutOfPages
    with pytest.raises(OutOfPages):
        runner.run([StepEntry(9, list(range(200)), [])])            # 8 pages of 16 tokens do not hold it
    assert cache.tokens(9) == 1                                     # and nothing was committed
