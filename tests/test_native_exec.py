"""The runtime's executor against the Python parts, on the CPU: both are run with the kernels' entry
points replaced by recorders, and must launch the same kernels with the same arguments (addresses compared
by what they name: a weight, a cache, an index array, or the launch that wrote them)."""
import ctypes

import numpy as np
import pytest
import torch

from launch_recorder import Names, Recorder, canonical, run_step, zero_model
from test_dispatch import WIDE


def test_tile_planning_is_the_same_in_both_languages():
    from cellm_b200.engine.native_exec import _runtime
    from cellm_b200.ops.gemm_bf16 import plan_tiles
    rt = _runtime()
    rng = np.random.default_rng(0)
    out = (ctypes.c_longlong * 2)()
    cases = [(int(m), int(n), int(k)) for m, n, k in zip(rng.integers(1, 5000, 3000), rng.integers(8, 70000, 3000),
                                                          rng.integers(8, 9000, 3000))]
    cases += [(m, n, k) for m in (1, 8, 16, 17, 64, 65, 128, 129, 342, 512, 2048) for n in (2048, 3072, 6144, 6272, 16384, 65536)
              for k in (2048, 8192)]
    for sms in (148, 132, 16):
        for m, n, k in cases:
            rt.cellm_exec_plan_tiles(m, n, k, sms, out)
            assert (out[0], out[1]) == plan_tiles(m, n, k, sms), (m, n, k, sms)


def both_ways(monkeypatch, config, q_lens, ctx_lens, dtype=torch.bfloat16, page=16, max_layers=None):
    """The canonical launch lists of the Python parts and of the executor for one step."""
    from cellm_b200.engine.native_exec import ENTRY_POINTS, NativeForward
    from cellm_b200.ops import _lib, gemm_bf16
    import importlib
    attention = importlib.import_module("cellm_b200.ops.attention")
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(config, dtype)
    step = run_step(model, plan, q_lens, ctx_lens, page, prepare_only=True)
    names = Names()
    names.add_model(model)
    for label, t in step.named_tensors():
        names.add(label, t)

    def with_workspaces(n):
        for label, t in (("gemm_ws", gemm_bf16._WORKSPACE.get(torch.device("cpu"))), ("attn_ws", attention._WORKSPACE.get(torch.device("cpu"))),
                         ("counters", gemm_bf16._COUNTERS.get(torch.device("cpu")))):
            n.add(label, t)
        return n
    before = _lib.LAUNCHES[0]
    step.run(model.forward, max_layers)
    launches_python = _lib.LAUNCHES[0] - before
    python_calls = list(rec.calls)
    python_list = canonical(python_calls, _lib._SIGNATURES, with_workspaces(names))

    native_calls = []
    thunks = []
    for library, name in ENTRY_POINTS:
        sig = _lib._SIGNATURES[library][name]

        def record(*args, _name=name):
            native_calls.append((_name, args))
            return 0
        thunks.append(ctypes.CFUNCTYPE(ctypes.c_int, *sig)(record))
    native = NativeForward(model, [ctypes.cast(t, ctypes.c_void_p).value for t in thunks], sms=148)
    step2 = run_step(model, plan, q_lens, ctx_lens, page, prepare_only=True)
    names2 = Names()
    names2.add_model(model)
    for label, t in step2.named_tensors():
        names2.add(label, t)
    step2.run(native.forward, max_layers)
    for label, t in (("gemm_ws", native._gemm_ws), ("attn_ws", native._attn_ws), ("counters", gemm_bf16._COUNTERS.get(torch.device("cpu")))):
        names2.add(label, t)
    native_list = canonical(native_calls, _lib._SIGNATURES, names2)
    return python_list, native_list, native.last_launches, launches_python


SHAPES = {"decode8": ([1] * 8, [2048] * 8), "decode64": ([1] * 64, [100 + 7 * i for i in range(64)]), "prompt": ([2048], [0]),
          "short prompt": ([128], [0]), "portion after a context": ([512], [1536]), "mixed": ([1, 40, 1, 300], [77, 16, 500, 0]),
          "two tokens each": ([2, 2, 2], [5, 700, 64])}


@pytest.mark.parametrize("shape", list(SHAPES))
def test_the_executor_launches_what_the_python_parts_launch(monkeypatch, shape):
    same(*both_ways(monkeypatch, WIDE, *SHAPES[shape]))


def same(a, b, launches_native, launches_python):
    assert len(a) == len(b), f"{len(a)} launches from Python, {len(b)} from the executor"
    for i, (x, y) in enumerate(zip(a, b)):
        assert x == y, f"launch {i}: python {x} vs executor {y}"
    assert launches_native == launches_python          # kernels, counting the second kernels some entry points launch


SMALL = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": 1000, "hidden_size": 256,
         "num_hidden_layers": 3, "layer_types": ["conv", "full_attention", "full_attention"], "num_attention_heads": 4,
         "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512, "block_auto_adjust_ff_dim": False,
         "rope_theta": 1e4, "conv_L_cache": 3, "norm_eps": 1e-6, "tie_embedding": True, "max_position_embeddings": 4096}
VARIANTS = {
    "32-bit": (SMALL, dict(dtype=torch.float32)),
    "untied head, bias, four taps": (dict(SMALL, tie_embedding=False, conv_bias=True, conv_L_cache=4), {}),
    "one tap": (dict(SMALL, conv_L_cache=1), {}),
    "five taps (no fused convolution)": (dict(SMALL, conv_L_cache=5), {}),
    "width off the tensor-core rules": (dict(SMALL, hidden_size=100, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
                                             intermediate_size=130), {}),
    "heads of 128": (dict(SMALL, head_dim=128), {}),
    "heads of 48": (dict(SMALL, head_dim=48), {}),
    "sixteen heads on one": (dict(SMALL, num_attention_heads=16, num_key_value_heads=1), {}),
    "pages of 8": (SMALL, dict(page=8)),
    "pages of 4": (SMALL, dict(page=4)),
    "first two layers only": (SMALL, dict(max_layers=2)),
    "a layer run twice on another's cache": (dict(SMALL, layer_order=[0, 1, {"layer": 2, "cache_of": 1}, 2]), {}),
    "feed-forward off the fused kernel's sizes": (dict(SMALL, intermediate_size=200), {}),
}
STEPS = [([1, 1, 1], [5, 300, 64]), ([70], [0]), ([1, 33, 2], [100, 0, 17]), ([400, 300], [0, 200])]


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_the_executor_follows_the_python_parts_in_other_models(monkeypatch, variant):
    config, kw = VARIANTS[variant]
    for q_lens, ctx_lens in STEPS:
        same(*both_ways(monkeypatch, config, q_lens, ctx_lens, **kw))


@pytest.mark.parametrize("rope,conv", [("1", "1"), ("1", "0"), ("0", "0")])
def test_the_executor_follows_the_fused_decode_kernels_switches(monkeypatch, rope, conv):
    monkeypatch.setenv("CELLM_B200_FUSED_ROPE", rope)
    monkeypatch.setenv("CELLM_B200_FUSED_CONV", conv)
    for q_lens, ctx_lens in (([1] * 8, [2048] * 8), ([1], [9]), ([1, 5], [3, 3])):
        same(*both_ways(monkeypatch, WIDE, q_lens, ctx_lens))


def test_prompt_kernel_policy_is_read_at_every_step(monkeypatch):
    """Tests lower the threshold of the tcgen05 prompt attention; the executor must see it too."""
    import importlib
    attention = importlib.import_module("cellm_b200.ops.attention")
    monkeypatch.setitem(attention.TC_POLICY, "min_ctas", 0)
    monkeypatch.setitem(attention.TC_POLICY, "min_fill", 0.0)
    a, b, n1, n2 = both_ways(monkeypatch, SMALL, [70, 3], [0, 40])
    same(a, b, n1, n2)
    assert any(row[0] == "cellm_attention_tc" for row in b)


def test_models_with_other_parts_are_left_to_python(monkeypatch):
    from cellm_b200.engine.native_exec import NativeForward, unsupported
    from cellm_b200.parts.norm import RMSNorm
    Recorder(monkeypatch)
    cfg, plan, model = zero_model(SMALL)
    assert unsupported(model) is None

    class OtherNorm(RMSNorm):
        pass
    model.blocks[1].mixer_norm.__class__ = OtherNorm
    assert "norm" in unsupported(model)
    with pytest.raises(ValueError, match="does not run this model"):
        NativeForward(model, [0] * 13, sms=148)


def test_random_models_and_steps(monkeypatch):
    """Two hundred random models (head sizes, groups, widths that do and do not fit the tensor-core rules, one to
    five taps, bias, tied or not, 32-bit now and then) and steps (single tokens, a few tokens each, prompt
    portions, one long prompt; pages of 4 to 64), with and without the rotation in the product."""
    for seed in range(200):
        rng = np.random.default_rng(seed)
        hd = int(rng.choice([16, 32, 48, 64, 64, 64, 128]))
        nkv = int(rng.choice([1, 2, 4, 8]))
        nh = nkv * int(rng.choice([1, 2, 4, 8] if hd <= 64 else [1, 2]))
        layers = int(rng.integers(1, 4))
        config = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": int(rng.choice([500, 1000, 40000])),
                  "hidden_size": int(rng.choice([64, 100, 256, 512, 1024, 2048])), "num_hidden_layers": layers,
                  "layer_types": [str(rng.choice(["conv", "full_attention"])) for _ in range(layers)],
                  "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd,
                  "intermediate_size": int(rng.choice([128, 130, 512, 2048, 8192])), "block_auto_adjust_ff_dim": False,
                  "rope_theta": 1e4, "conv_L_cache": int(rng.choice([1, 2, 3, 4, 5])), "conv_bias": bool(rng.random() < 0.3),
                  "norm_eps": 1e-5, "tie_embedding": bool(rng.random() < 0.5), "max_position_embeddings": 100000}
        B, kind = int(rng.integers(1, 70)), rng.random()
        if kind < 0.35:
            q_lens = [1] * B
        elif kind < 0.6:
            q_lens = [int(x) for x in rng.integers(1, 5, B)]
        elif kind < 0.8:
            q_lens = [int(x) for x in rng.integers(1, 400, min(B, 6))]
        else:
            q_lens = [int(rng.integers(64, 4000))]
        ctx_lens = [int(x) for x in rng.integers(0, 3000, len(q_lens))]
        dtype = torch.float32 if rng.random() < 0.15 else torch.bfloat16
        with monkeypatch.context() as m:
            m.setenv("CELLM_B200_FUSED_ROPE", "1" if rng.random() < 0.5 else "0")
            try:
                same(*both_ways(m, config, q_lens, ctx_lens, dtype=dtype, page=int(rng.choice([4, 8, 16, 32, 64]))))
            except AssertionError as e:
                raise AssertionError(f"seed {seed}: {config} {q_lens} {ctx_lens}: {e}") from None
