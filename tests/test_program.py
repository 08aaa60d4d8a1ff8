"""The model as a program of the native executor, on the CPU (kernels' entry points replaced by recorders):
parts emit their own records, a part without a record is called back in Python between native ones, a
built-in part's own forward() launches what its record launches inside the program, and the executor's
decisions (tile shapes, kernels) hold the properties the kernels rely on."""
import numpy as np
import pytest
import torch

from launch_recorder import Recorder, run_step, zero_model
from test_dispatch import WIDE

SMALL = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": 1000, "hidden_size": 256,
         "num_hidden_layers": 3, "layer_types": ["conv", "full_attention", "full_attention"], "num_attention_heads": 4,
         "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512, "block_auto_adjust_ff_dim": False,
         "rope_theta": 1e4, "conv_L_cache": 3, "norm_eps": 1e-6, "tie_embedding": True, "max_position_embeddings": 4096}


def test_every_built_in_part_emits_its_own_record(monkeypatch):
    from cellm_b200.runtime import records as R
    from cellm_b200.runtime.program import Program
    Recorder(monkeypatch)
    cfg, plan, model = zero_model(SMALL)
    prog = Program(model)
    assert prog.all_native
    assert [r.kind for r in prog.prologue] == [R.EMBED] and [r.kind for r in prog.epilogue] == [R.RMS_NORM, R.HEAD]
    kinds = [[r.kind for r in layer] for layer in prog.layers]
    assert kinds == [[R.RMS_NORM, R.SHORT_CONV, R.RMS_NORM, R.SWIGLU]] + [[R.RMS_NORM, R.ATTENTION, R.RMS_NORM, R.SWIGLU]] * 2
    # each record names the part it came from, and the part keeps it: the same record serves the part's own forward()
    for layer, block in zip(prog.layers, model.blocks):
        assert [r.part for r in layer] == [block.mixer_norm, block.mixer, block.feed_forward_norm, block.feed_forward]
        assert layer[1] is block.mixer.record() and layer[3] is block.feed_forward.record()


def test_tile_planning_properties():
    """What the kernels rely on: swapped tiles of 16, 32 or 64 tokens up to 64 tokens, a K split of at most 8 there
    (one thread-block cluster) and never more slices than four K blocks each allow; plain tiles of 64, 128 or 256."""
    from cellm_b200.runtime.program import plan_tiles
    rng = np.random.default_rng(0)
    cases = [(int(m), int(n), int(k)) for m, n, k in zip(rng.integers(1, 5000, 2000), rng.integers(8, 70000, 2000),
                                                          rng.integers(8, 9000, 2000))]
    cases += [(m, n, k) for m in (1, 8, 16, 17, 64, 65, 128, 129, 342, 512, 2048) for n in (2048, 3072, 6144, 6272, 16384, 65536)
              for k in (2048, 8192)]
    for sms in (148, 132, 16):
        for m, n, k in cases:
            bn, split = plan_tiles(m, n, k, sms)
            kblocks = (k + 63) // 64
            assert split >= 1 and (split == 1 or split <= kblocks // 4)
            if m <= 64:
                assert bn == -(16 if m <= 16 else 32 if m <= 32 else 64) and split <= 8
            elif bn < 0:
                assert bn == -64 and m <= 128 and split <= 8
            else:
                assert (bn == 64 or (128 <= bn <= 256 and bn % 16 == 0)) and split <= 16
                assert split == 1 or bn in (64, 128, 256)     # the widths between are for unsplit products
    # a prompt of 2,048 tokens on 148 SMs: the q/k/v product (3,072 columns) in 16 x 18 tiles of 176 columns (two full
    # waves less a few), the products of 2,048 columns in 16 x 9 tiles of 240 (one wave)
    assert plan_tiles(2048, 3072, 2048, 148) == (176, 1) and plan_tiles(2048, 2048, 8192, 148) == (240, 1)
    # the sizes of LFM2-1.2B's decode step at 8 requests: every product fills most of the 148 SMs
    for n, k in ((2048, 2048), (3072, 2048), (16384, 2048), (2048, 8192), (6272, 2048)):
        bn, split = plan_tiles(8, n, k, 148)
        assert bn == -16 and 100 <= ((n + 127) // 128) * split <= 2 * 148


def part_calls(rec, start):
    return [(n, a) for n, a in rec.calls[start:]]


@pytest.mark.parametrize("q_lens,ctx_lens", [([1, 1, 1], [5, 300, 64]), ([70], [0]), ([1, 33, 2], [100, 0, 17])])
def test_a_parts_own_forward_launches_what_its_record_launches_in_the_program(monkeypatch, q_lens, ctx_lens):
    """Kernel names and every size argument agree (addresses differ: the part alone works on its caller's tensors)."""
    from cellm_b200.ops import _lib
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(SMALL)
    step = run_step(model, plan, q_lens, ctx_lens, prepare_only=True)
    step.run(model.forward)
    whole = list(rec.calls)
    sig_of = {n: s for lib_sigs in _lib._SIGNATURES.values() for n, s in lib_sigs.items()}
    sizes = lambda calls: [(n, tuple(v for t, v in zip(sig_of[n], a) if t is not _lib.P)) for n, a in calls]
    alone = []
    x = torch.zeros((sum(q_lens), 256), dtype=torch.bfloat16)
    for i, block in enumerate(model.blocks):
        for part, args in ((block.mixer, (x, step.ctx, step.bindings[i])), (block.feed_forward, (x, step.ctx))):
            before = len(rec.calls)
            out = part.forward(*args)
            assert tuple(out.shape) == tuple(x.shape) and out.dtype == x.dtype
            alone.append(rec.calls[before:])
    in_program = [c for c in sizes(whole) if c[0] not in ("cellm_embed", "cellm_add_rmsnorm")][:-1]      # without norms and head
    assert [c for part in alone for c in sizes(part)] == in_program


def test_a_part_without_a_record_is_called_back_between_native_parts(monkeypatch):
    """A norm and a mixer defined here, with forward() only: the executor runs the native records around them and
    calls the interpreter for these two, with the registers they are to work on."""
    from cellm_b200.parts import Mixer, Norm
    from cellm_b200.runtime import records as R
    from cellm_b200.runtime.program import Program
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(SMALL)
    seen = []

    class MyNorm(Norm):
        graph_safe = True

        def forward(self, residual, rows=None):
            seen.append(("norm", tuple(residual.x.shape), residual.pending is not None, len(rec.calls)))
            residual.pending = None
            return torch.full((residual.x.shape[0] if rows is None else rows.numel(), 256), 2.0, dtype=torch.bfloat16)

    class MyMixer(Mixer):
        graph_safe = True

        def forward(self, x, ctx, cache):
            seen.append(("mixer", float(x[0, 0]), cache.state is not None, len(rec.calls)))
            return torch.ones_like(x)
    model.blocks[0].feed_forward_norm = MyNorm()
    model.blocks[0].mixer = MyMixer()
    prog = Program(model)
    assert [r.kind for r in prog.layers[0]] == [R.RMS_NORM, R.PYTHON, R.PYTHON, R.SWIGLU] and len(prog.python_parts) == 2
    model.program = prog
    run_step(model, plan, [3, 1], [0, 9])
    # embedding and first norm ran natively before the mixer was called; the norm after it saw the mixer's output waiting
    assert seen[0][0] == "mixer" and seen[0][2] and seen[0][3] == 2
    assert seen[1] == ("norm", (4, 256), True, 2)
    names = rec.names()
    assert names[:2] == ["cellm_embed", "cellm_add_rmsnorm"] and names[2] == "cellm_gemm_tcgen05"     # the feed-forward reads MyNorm's output
    assert names.count("cellm_short_conv") + names.count("cellm_gemm_conv_tcgen05") == 0               # the native mixer is gone
    # the feed-forward's first product read the tensor MyNorm returned: an address outside the step's arena
    arena = prog._arena
    a_ptr = rec.of("cellm_gemm_tcgen05")[0][1]
    assert not arena.data_ptr() <= a_ptr < arena.data_ptr() + arena.numel()


def test_an_exception_in_a_python_part_comes_out_of_forward(monkeypatch):
    from cellm_b200.parts import FeedForward
    Recorder(monkeypatch)
    cfg, plan, model = zero_model(SMALL)

    class Broken(FeedForward):
        def forward(self, x, ctx):
            raise KeyError("from the part")
    model.blocks[1].feed_forward = Broken()
    with pytest.raises(KeyError, match="from the part"):
        run_step(model, plan, [2], [0])


def test_options_are_read_at_every_step(monkeypatch):
    """Tests lower the threshold of the tcgen05 prompt attention and switch the fused decode kernels off."""
    from cellm_b200.runtime import program
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(SMALL)
    run_step(model, plan, [70, 3], [0, 40])
    assert "cellm_attention_tc" not in rec.names()
    monkeypatch.setitem(program.OPTIONS, "attention_tc_min_ctas", 0)
    monkeypatch.setitem(program.OPTIONS, "attention_tc_min_fill", 0.0)
    rec.calls.clear()
    run_step(model, plan, [70, 3], [0, 40])
    assert "cellm_attention_tc" in rec.names()


VARIANTS = {
    "32-bit": (SMALL, dict(dtype=torch.float32)),
    "untied head, bias, four taps": (dict(SMALL, tie_embedding=False, conv_bias=True, conv_L_cache=4), {}),
    "five taps (no fused convolution)": (dict(SMALL, conv_L_cache=5), {}),
    "width off the tensor-core rules": (dict(SMALL, hidden_size=100, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
                                             intermediate_size=130), {}),
    "heads of 128": (dict(SMALL, head_dim=128), {}),
    "heads of 48": (dict(SMALL, head_dim=48), {}),
    "a layer run twice on another's cache": (dict(SMALL, layer_order=[0, 1, {"layer": 2, "cache_of": 1}, 2]), {}),
}


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_other_models_walk_through(monkeypatch, variant):
    """Every model runs the same order of parts; which kernels serve them follows the sizes."""
    config, kw = VARIANTS[variant]
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(config, kw.get("dtype", torch.bfloat16))
    for q_lens, ctx_lens in (([1, 1, 1], [5, 300, 64]), ([70], [0]), ([400, 300], [0, 200])):
        rec.calls.clear()
        logits = run_step(model, plan, q_lens, ctx_lens)
        assert tuple(logits.shape) == (len(q_lens), config["vocab_size"]) and logits.dtype == torch.float32
        names = rec.names()
        assert names[0] == "cellm_embed" and names.count("cellm_add_rmsnorm") == 2 * len(plan.order) + 1
        attn = [n for n in names if n.startswith("cellm_attention")]
        assert len(attn) == sum(1 for e in plan.order if plan.layers[e.layer].mixer.kind == "attention")
        if variant == "a layer run twice on another's cache":
            # the item that borrows a cache forms queries only: no keys or values are written for it
            writes = [a[17] for a in rec.of("cellm_qk_norm_rope")] + [a[20] for a in rec.of("cellm_gemm_rope_tcgen05")]
            assert sorted(writes) == [0, 2, 2]


def test_max_layers_runs_the_first_items_only(monkeypatch):
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(SMALL)
    step = run_step(model, plan, [5], [0], prepare_only=True)
    step.run(model.forward, 2)
    assert rec.names().count("cellm_add_rmsnorm") == 2 * 2 + 1
