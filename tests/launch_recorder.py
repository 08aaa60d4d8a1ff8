"""Runs the package's Python side of a step without a GPU: the kernels' entry points are replaced by
recorders, so that a test can see which kernels a step of a given shape would launch and with which
sizes. Weights are zeros on the CPU; nothing is computed."""
import importlib

import numpy as np
import torch


class Recorder:
    def __init__(self, monkeypatch, sms: int = 148, hooks: dict | None = None):
        """Patches (through `monkeypatch`, so that everything is put back) the look-up of the compiled
        entry points, by the Python wrappers and by the native executor alike, the checks that operands lie on a
        GPU, the stream and SM queries. `hooks`: entry point name -> function of its arguments, run in the
        kernel's place (to leave something in an output)."""
        import ctypes
        self.hooks = hooks = dict(hooks or {})
        from cellm_b200.ops import _lib, _state, basic, gemm_bf16
        from cellm_b200.runtime import program, records
        gemm = importlib.import_module("cellm_b200.ops.gemm")
        attention = importlib.import_module("cellm_b200.ops.attention")
        self.calls: list[tuple[str, tuple]] = []
        sigs = _lib._SIGNATURES

        def stand_in(name, sig):
            def call(*args):
                assert len(args) == len(sig), f"{name}: {len(args)} arguments for a signature of {len(sig)}"
                self.calls.append((name, args))
                if name in hooks:
                    hooks[name](*args)
                return 0
            return call

        def fn(library, name):
            return stand_in(name, sigs[library][name])
        for m in (_lib, basic, gemm, gemm_bf16, attention):
            for attr, value in (("fn", fn), ("require_cuda", lambda *a: None), ("stream_of", lambda t: 0)):
                if hasattr(m, attr):
                    monkeypatch.setattr(m, attr, value)
        # the executor's table of entry points: C call-backs into the same recorders
        self._thunks = [ctypes.CFUNCTYPE(ctypes.c_int, *sigs[library][name])(stand_in(name, sigs[library][name]))
                        for library, name in records.ENTRY_POINTS]
        self.entries = [ctypes.cast(t, ctypes.c_void_p).value for t in self._thunks]
        monkeypatch.setattr(program, "entry_points", lambda dtype: self.entries)
        monkeypatch.setattr(program, "sm_count", lambda device: sms)
        monkeypatch.setattr(program, "_BARE", {})
        monkeypatch.setattr(gemm_bf16, "_sms", lambda device: sms)
        monkeypatch.setitem(_state._ERR, torch.device("cpu"), torch.zeros(1, dtype=torch.int32))
        monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
        monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True), raising=False)
        gemm_bf16.plan_tiles.cache_clear()

    def names(self) -> list[str]:
        return [n for n, _ in self.calls]

    def of(self, name: str) -> list[tuple]:
        return [a for n, a in self.calls if n == name]


def zero_model(config: dict, dtype=torch.bfloat16):
    """(typed config, plan, DecoderModel) with all-zero weights on the CPU."""
    from cellm_b200 import parts  # noqa: F401  (registers the built-in parts)
    from cellm_b200.config import config_from_dict
    from cellm_b200.models.decoder import DecoderModel
    from cellm_b200.weights.loader import expected_tensors
    cfg, plan = config_from_dict(config)
    tensors = {n: torch.zeros(ts.shape, dtype=dtype) for n, ts in expected_tensors(plan).items()}
    return cfg, plan, DecoderModel(plan, tensors, dtype, "cpu")


class Step:
    """The context, cache bindings and wanted rows of one step on the CPU."""

    def __init__(self, model, plan, q_lens, ctx_lens, page: int = 16):
        from cellm_b200.cache.manager import CacheManager
        from cellm_b200.ops._state import error_word           # the engine's steps carry the device's one error word
        from cellm_b200.parts.base import StepContext
        B, T = len(q_lens), sum(q_lens)
        width = max((c + q + page - 1) // page for c, q in zip(ctx_lens, q_lens)) + 1
        self.cache = cache = CacheManager(model.cache_needs(), [e.cache_of for e in plan.order], page, B * width + 4, B + 1,
                                          model.dtype, "cpu")
        i32 = lambda x: torch.tensor(x, dtype=torch.int32)
        self.tables = [torch.full((B, width), -1, dtype=torch.int32) for _ in cache.paged_keys]
        for b in range(B):
            cache.add(b)
            cache.reserve(b, ctx_lens[b] + q_lens[b])
            for g, t in enumerate(self.tables):
                cache.block_table(b, g, t[b].numpy())
        cu = [0] + [int(v) for v in np.cumsum(q_lens)]
        self.ctx = StepContext(T=T, B=B, dtype=model.dtype, device=torch.device("cpu"), token_ids=i32(list(range(T))),
                               positions=i32([c + j for c, q in zip(ctx_lens, q_lens) for j in range(q)]),
                               seq_of_token=i32([b for b, q in enumerate(q_lens) for _ in range(q)]), cu_seqlens=i32(cu),
                               ctx_lens=i32(list(ctx_lens)), slot_ids=i32([cache.slot(b) for b in range(B)]),
                               err=error_word("cpu"), q_lens=list(q_lens), ctx_lens_host=list(ctx_lens),
                               max_q_len=max(q_lens), max_total_len=max(c + q for c, q in zip(ctx_lens, q_lens)))
        self.rows = i32([c - 1 for c in cu[1:]])
        self.bindings = cache.bindings(self.tables)

    def run(self, forward, max_layers=None):
        return forward(self.ctx, self.bindings, self.rows, max_layers)

    def named_tensors(self):
        c = self.ctx
        yield from (("ids", c.token_ids), ("positions", c.positions), ("seq_of_token", c.seq_of_token), ("cu_seqlens", c.cu_seqlens),
                    ("ctx_lens", c.ctx_lens), ("slot_ids", c.slot_ids), ("err", c.err), ("rows", self.rows))
        for g, t in enumerate(self.tables):
            yield f"block_table{g}", t
        for g, (k, v) in enumerate(zip(self.cache.k_pools, self.cache.v_pools)):
            yield f"k_pool{g}", k
            yield f"v_pool{g}", v
        for g, st in enumerate(self.cache.states):
            yield f"state{g}", st


def run_step(model, plan, q_lens, ctx_lens, page: int = 16, prepare_only: bool = False):
    """One step of entries with `q_lens` new tokens after `ctx_lens` cached ones; logits wanted at each entry's
    last token. `prepare_only`: return the Step without running it."""
    step = Step(model, plan, q_lens, ctx_lens, page)
    return step if prepare_only else step.run(model.forward)


# ---- comparing the launches of two runs -------------------------------------------------------------------------
OUTPUTS = {"cellm_add_rmsnorm": (0, 4)}          # arguments a kernel writes (default: the first)
WRITE_ONLY = {"cellm_add_rmsnorm": (4,)}         # of these, the ones whose old content does not matter (default: the first)


class Names:
    """Names for the addresses a launch may carry: tensors known by name (weights, caches, the step's index
    arrays, workspaces) and, for everything else, the launch that wrote the address last."""

    def __init__(self):
        self.ranges: list[tuple[int, int, str]] = []

    def add(self, name: str, t) -> None:
        if t is not None and t.numel():
            self.ranges.append((t.data_ptr(), t.data_ptr() + t.numel() * t.element_size(), name))

    def add_model(self, model) -> None:
        def scan(obj, path, depth=0):
            if isinstance(obj, torch.Tensor):
                self.add(path, obj)
            elif depth < 4 and hasattr(obj, "__dict__"):
                for k, v in vars(obj).items():
                    scan(v, f"{path}.{k}", depth + 1)
        for i, b in enumerate(model.blocks):
            scan(b, f"L{i}")
        scan(model.final_norm, "final_norm")
        scan(model.head, "head")
        scan(model.embedding, "embedding")

    def of(self, address):
        if not address:
            return None
        for lo, hi, name in self.ranges:
            if lo <= address < hi:
                return name if address == lo else f"{name}+{address - lo}"
        return None


def canonical(calls, signatures: dict, names: Names) -> list:
    """The launches with every address replaced by its name, or by the index of the launch that wrote it."""
    import numpy as np
    from cellm_b200.ops import _lib
    sig_of = {n: s for lib_sigs in signatures.values() for n, s in lib_sigs.items()}
    writer: dict[int, int] = {}
    out = []
    for index, (name, args) in enumerate(calls):
        row = [name]
        for position, (t, v) in enumerate(zip(sig_of[name], args)):
            if t is _lib.P:
                known = names.of(v)
                if known is not None or not v:
                    row.append(known)
                elif position in WRITE_ONLY.get(name, (0,)):
                    row.append("new")
                else:
                    row.append(f"written by {writer.get(v, '?')}")
            elif t is _lib.F:
                row.append(float(np.float32(v)))
            else:
                row.append(int(v))
        for o in OUTPUTS.get(name, (0,)):
            if args[o] and names.of(args[o]) is None:
                writer[args[o]] = index
        out.append(row)
    return out
