"""A model as a program for the native executor (csrc/runtime/executor.cc), and its runs.

The model's parts emit one op record each (embedding; for every layer whatever
its block arrangement emits; final norm and head). `Program.forward` hands a
step to the executor, which walks the records and launches the kernels in one
foreign call, with the decisions below the parts (kernel, tile shape, K split)
taken there. A part without a native record is run by `_python_op`, which the
executor calls for that part alone with the registers it works on.

This is the only forward walker: generation, trace replay and the captured
decode graphs all go through it, and a built-in part's own forward() runs the
part's single record through `run_part`.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_longlong, c_void_p
from typing import Optional

import torch

from ..cache.native import CacheError, last_error, lib
from ..ops import _lib as klib
from ..ops._state import MAX_COUNTERS, STATIC_WEIGHTS_FLAG, counters, error_word, sm_count
from . import records as R

# Switches of the executor's decisions, read at every run (tests change them to drive small cases through kernels
# that serving reaches only at large sizes). fused_conv / fused_rope: decode steps run in_proj + short convolution,
# and the q/k/v product + head norms + rotation + cache write, as one kernel each. attention_tc_*: prompt attention
# goes to the tcgen05 kernel from this many CTAs (None: an eighth of the SMs) and this share of its tiles' rows in use.
OPTIONS = {"fused_conv": True, "fused_rope": True, "attention_tc_min_ctas": None, "attention_tc_min_fill": 0.5}

_bound = False


def runtime():
    """The runtime library with the executor's functions typed; checks the structs' layout once."""
    global _bound
    l = lib()
    if not _bound:
        l.cellm_exec_sizeof.argtypes, l.cellm_exec_sizeof.restype = [ctypes.c_int], c_longlong
        l.cellm_exec_need.argtypes, l.cellm_exec_need.restype = [c_void_p, c_void_p, POINTER(R.I64)], ctypes.c_int
        l.cellm_exec_forward.argtypes, l.cellm_exec_forward.restype = [c_void_p, c_void_p], ctypes.c_int
        l.cellm_exec_part.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int, POINTER(R.I64)]
        l.cellm_exec_part.restype = ctypes.c_int
        l.cellm_exec_plan_tiles.argtypes = [R.I64, R.I64, R.I64, R.I64, POINTER(R.I64)]
        l.cellm_exec_plan_tiles.restype = ctypes.c_int
        for which, cls in enumerate(R.LAYOUT_CHECKED):
            if l.cellm_exec_sizeof(which) != ctypes.sizeof(cls):
                raise RuntimeError(f"native executor: {cls.__name__} is {ctypes.sizeof(cls)} bytes here and "
                                   f"{l.cellm_exec_sizeof(which)} in the runtime")
        _bound = True
    return l


def plan_tiles(M: int, N: int, K: int, sms: int) -> tuple[int, int]:
    """(bn, split_k) of a product of M tokens by N weight rows over K, as the executor plans it: bn > 0 plain
    tiles of 128 x bn, bn < 0 swapped tiles of 128 weight rows x -bn tokens."""
    out = (R.I64 * 2)()
    runtime().cellm_exec_plan_tiles(M, N, K, sms, out)
    return int(out[0]), int(out[1])


def entry_points(act_dtype: torch.dtype) -> list:
    """Addresses of the compiled kernels' C symbols in the order of the executor's table; loads (and if need be
    compiles) the libraries this element type calls into, and leaves the others' entries empty."""
    from ..csrc import build as _build
    out = []
    for library, name in R.ENTRY_POINTS:
        if act_dtype == torch.float32 and library in R.BF16_ONLY_LIBRARIES:
            out.append(None)
        else:
            out.append(ctypes.cast(getattr(_build.load(library), name), c_void_p).value)
    return out


# calls of each kernel entry point by the executor since the process began (tests read which kernels served a run)
CALLS: dict = {name: 0 for _, name in R.ENTRY_POINTS}


def _count_calls(s) -> None:
    for (_, name), n in zip(R.ENTRY_POINTS, s.calls):
        if n:
            CALLS[name] += int(n)


def _kernel_error(message: str) -> Exception:
    """A kernel's refusal of its arguments (negative status) is a ValueError, as from the kernel's own wrapper;
    anything else a RuntimeError."""
    import re
    m = re.search(r"status (-?\d+)", message)
    if m and int(m.group(1)) < 0:
        return ValueError(f"native executor: {message} ({klib._ERRORS.get(int(m.group(1)), 'refused')})")
    return RuntimeError(f"native executor: {message}")


def _ops_array(recs: list) -> tuple:
    arr = (R.ExecOp * max(len(recs), 1))(*[r.op for r in recs])
    return R.ExecOps(len(recs), arr), arr


class Program:
    def __init__(self, model=None, entries: Optional[list] = None, sms: Optional[int] = None, *,
                 dtype=None, device=None, hidden: int = 0):
        """`model`: a DecoderModel (None: a program without records, for `run_part` alone, over activations of
        `dtype` and width `hidden` on `device`). `entries`: addresses for the executor's table in the order of
        records.ENTRY_POINTS (default: the compiled libraries' symbols). `sms`: the SM count the tile planning
        assumes (default: the device's)."""
        self.model = model
        self.device = torch.device(model.device if model is not None else device)
        self.dtype = model.dtype if model is not None else dtype
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the executor runs bfloat16 or float32 activations, not {self.dtype}")
        self._rt = runtime()
        self.python_parts: list = []        # (role, part) of the Python records, by token
        self.prologue, self.layers, self.epilogue, order = [], [], [], []
        if model is not None:
            em = R.Emitter(self.dtype, self.python_parts)
            model.embedding.emit(em)
            self.prologue = em.records
            for block in model.blocks:
                em = R.Emitter(self.dtype, self.python_parts)
                block.emit(em)
                self.layers.append(em.records)
            em = R.Emitter(self.dtype, self.python_parts)
            model.final_norm.emit(em)
            model.head.emit(em)
            self.epilogue = em.records
            order = [e.layer for e in model.plan.order]
        self._keep = []
        p = R.ExecProgram()
        p.n_layers, p.n_order = len(self.layers), len(order)
        p.H, p.V = (model.plan.hidden_size, model.plan.vocab_size) if model is not None else (int(hidden), 0)
        p.act_dtype = klib.tag(self.dtype)
        p.sms = sms if sms is not None else sm_count(self.device)
        p.static_flag, p.max_counters = STATIC_WEIGHTS_FLAG, MAX_COUNTERS
        p.prologue, a = _ops_array(self.prologue)
        p.epilogue, b = _ops_array(self.epilogue)
        per_layer = [_ops_array(recs) for recs in self.layers]
        layer_arr = (R.ExecOps * max(len(per_layer), 1))(*[x[0] for x in per_layer])
        order_arr = (R.I64 * max(len(order), 1))(*order)
        p.layers, p.order = layer_arr, order_arr
        self._callback = R.PythonOpFn(self._python_op)
        p.python = self._callback
        for i, addr in enumerate(entries if entries is not None else entry_points(self.dtype)):
            p.fns[i] = addr
        self._keep += [a, b, per_layer, layer_arr, order_arr]
        self.program = p
        self._arena = self._gemm_ws = self._attn_ws = None
        self._live = None               # (ctx, bindings, logit rows, logits, arena, tensors of Python parts) of the running step
        self._raised: Optional[BaseException] = None
        self.last_launches = 0

    @property
    def all_native(self) -> bool:
        return not self.python_parts

    # ---------------------------------------------------------------------------------------------- running
    def _grow(self, name: str, n: int, dtype) -> torch.Tensor:
        if torch.cuda.is_current_stream_capturing():
            # a captured launch keeps its pointers: give it memory of the graph's own pool
            return torch.empty(max(n, 1), dtype=dtype, device=self.device)
        t = getattr(self, name)
        if t is None or t.numel() < n:
            t = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            setattr(self, name, t)
        return t

    def _options(self) -> None:
        p = self.program
        p.fused_conv, p.fused_rope = int(OPTIONS["fused_conv"]), int(OPTIONS["fused_rope"])
        p.tc_min_ctas = -1 if OPTIONS["attention_tc_min_ctas"] is None else int(OPTIONS["attention_tc_min_ctas"])
        p.tc_min_fill = float(OPTIONS["attention_tc_min_fill"])

    def _step(self, ctx, bindings, n_items: int, logit_rows, stream) -> tuple:
        items = (R.ExecItem * max(n_items, 1))()
        for it, b in zip(items, bindings[:n_items]):
            it.writes = int(b.writes)
            if b.k is not None:
                it.k, it.v, it.block_table = b.k.data_ptr(), b.v.data_ptr(), b.block_table.data_ptr()
                it.bt_stride, it.num_pages, it.page_size = b.block_table.stride(0), b.k.shape[0], b.page_size
            if b.state is not None:
                it.state = b.state.data_ptr() if b.state.numel() else None
                it.slot_stride, it.n_slots = b.state.stride(0), b.state.shape[0]
        s = R.ExecStep()
        nrows = 0 if logit_rows is None else int(logit_rows.numel())
        s.T, s.B, s.R, s.max_q_len, s.max_total_len, s.n_order = ctx.T, ctx.B, nrows, ctx.max_q_len, ctx.max_total_len, n_items
        s.ids, s.positions, s.seq_of_token = ctx.token_ids.data_ptr(), ctx.positions.data_ptr(), ctx.seq_of_token.data_ptr()
        s.cu_seqlens, s.ctx_lens, s.slot_ids = ctx.cu_seqlens.data_ptr(), ctx.ctx_lens.data_ptr(), ctx.slot_ids.data_ptr()
        s.rows = logit_rows.data_ptr() if nrows else None
        q_lens = (R.I64 * ctx.B)(*ctx.q_lens)
        s.q_lens, s.items = q_lens, items
        s.err = ctx.err.data_ptr()
        s.stream = klib.stream_of(ctx.err) if stream is None else stream
        s.counters = counters(self.device).data_ptr()
        return s, (items, q_lens)

    def _buffers(self, s, need) -> torch.Tensor:
        arena = self._grow("_arena", need[0] + 256, torch.uint8)
        s.arena, s.arena_bytes = arena.data_ptr(), arena.numel()
        if need[1]:
            ws = self._grow("_gemm_ws", need[1], torch.float32)
            s.gemm_ws, s.gemm_ws_floats = ws.data_ptr(), ws.numel()
        if need[2]:
            ws = self._grow("_attn_ws", need[2], torch.float32)
            s.attn_ws, s.attn_ws_floats = ws.data_ptr(), ws.numel()
        return arena

    def forward(self, ctx, bindings, logit_rows: Optional[torch.Tensor], max_layers: Optional[int] = None,
                stream: Optional[int] = None) -> Optional[torch.Tensor]:
        """Runs the step's T tokens through the layers; float32 logits [R, vocab] for the rows in `logit_rows`
        (None: no logits are formed). `max_layers` runs only the first items of the run order."""
        p = self.program
        self._options()
        n_order = p.n_order if max_layers is None else min(int(max_layers), p.n_order)
        s, keep = self._step(ctx, bindings, n_order, logit_rows, stream)
        need = (R.I64 * 3)()
        if self._rt.cellm_exec_need(ctypes.byref(p), ctypes.byref(s), need) != 0:
            raise CacheError(last_error())
        arena = self._buffers(s, need)
        logits = torch.empty((s.R, p.V), dtype=torch.float32, device=self.device) if s.R else None
        s.logits = logits.data_ptr() if s.R else None
        self._live, self._raised = (ctx, bindings, logit_rows, logits, arena, {}), None
        try:
            rc = self._rt.cellm_exec_forward(ctypes.byref(p), ctypes.byref(s))
        finally:
            self._live = None
        if self._raised is not None:
            raise self._raised
        if rc != 0:
            raise _kernel_error(last_error())
        self.last_launches = int(s.launches)
        klib.count_launch(self.last_launches)
        _count_calls(s)
        return logits

    def run_part(self, record: R.Record, x: torch.Tensor, ctx, binding=None, out: Optional[torch.Tensor] = None,
                 rows: Optional[int] = None) -> torch.Tensor:
        """One record by itself. A mixer or feed-forward record: x [T, H] in, a new [T, H] out, both of the
        activations' element type (this is what a built-in part's own forward() runs). A LINEAR or ATTEND record:
        x in, `out` (given) written. `ctx` may be None for a record that reads no index array (`rows` tokens then)."""
        if x.dtype != self.dtype or not x.is_contiguous():
            if record.kind != R.LINEAR:
                x = x.to(self.dtype).contiguous()
        p = self.program
        self._options()
        from ..parts.base import CacheBinding
        if ctx is not None:
            s, keep = self._step(ctx, [binding if binding is not None else CacheBinding()], 1, None, None)
        else:
            s, keep = R.ExecStep(), (R.ExecItem * 1)()
            s.T, s.items, s.n_order = int(rows), keep, 1
            s.err, s.stream = error_word(self.device).data_ptr(), klib.stream_of(x)
            s.counters = counters(self.device).data_ptr()
        need = (R.I64 * 3)()
        op = ctypes.byref(record.op)
        if self._rt.cellm_exec_part(ctypes.byref(p), ctypes.byref(s), op, x.data_ptr(), None, 1, need) != 0:
            raise ValueError(f"native executor: {last_error()}")
        self._buffers(s, need)
        if out is None:
            out = torch.empty((s.T, p.H), dtype=self.dtype, device=x.device)
        if self._rt.cellm_exec_part(ctypes.byref(p), ctypes.byref(s), op, x.data_ptr(), out.data_ptr(), 0, need) != 0:
            raise _kernel_error(last_error())
        klib.count_launch(int(s.launches))
        _count_calls(s)
        return out

    # ------------------------------------------------------------------------------------- Python parts
    def _view(self, address: int, shape, dtype) -> torch.Tensor:
        """The tensor behind an address the executor names: a buffer of the step's arena, or what a Python part
        left earlier in this step."""
        ctx, bindings, rows, logits, arena, mine = self._live
        t = mine.get(address)
        if t is not None:
            return t
        off = address - arena.data_ptr()
        n = 1
        for d in shape:
            n *= d
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if not 0 <= off <= arena.numel() - nbytes:
            raise RuntimeError("native executor: a register points outside the step's memory")
        return arena[off:off + nbytes].view(dtype).view(shape)

    def _own(self, t: Optional[torch.Tensor], shape) -> Optional[int]:
        """Keeps a Python part's output alive for the rest of the step; returns its address for a register."""
        if t is None:
            return None
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"a part returned {tuple(t.shape)} where {tuple(shape)} was wanted")
        if t.dtype != self.dtype or not t.is_contiguous():
            t = t.to(self.dtype).contiguous()
        self._live[5][t.data_ptr()] = t
        return t.data_ptr()

    def _python_op(self, token: int, regs_ptr) -> int:
        """Called by the executor for a Python record: runs the part's own forward() on the registers.
        embedding: x = forward(ids, ctx). norm: y = forward(residual[, rows]). mixer / feed_forward: pending =
        forward(y, ctx[, cache]). block: forward(residual, ctx, cache). head: logits = forward(y)."""
        try:
            from .. import ops
            from ..parts.base import Residual
            role, part = self.python_parts[token]
            regs = regs_ptr.contents
            ctx, bindings, rows, logits, arena, mine = self._live
            T, H = ctx.T, self.program.H
            x = self._view(regs.x, (T, H), torch.float32)
            pending = self._view(regs.pending, (T, H), self.dtype) if regs.pending else None
            n_y = T if regs.phase != 2 else int(rows.numel())
            if role == "embedding":
                x.copy_(part.forward(ctx.token_ids, ctx))
            elif role in ("norm", "block"):
                res = Residual(x)
                res.pending = pending
                if role == "norm":
                    y = part.forward(res, rows=rows if regs.phase == 2 else None)
                    regs.y = self._own(y, (n_y, H))
                else:
                    part.forward(res, ctx, bindings[regs.item])
                    regs.y = None
                if res.x is not x:
                    x.copy_(res.x)
                regs.pending = self._own(res.pending, (T, H))
            elif role in ("mixer", "feed_forward"):
                if not regs.y:
                    raise RuntimeError("a part wants activations before any norm has left some")
                y = self._view(regs.y, (T, H), self.dtype)
                out = part.forward(y, ctx, bindings[regs.item]) if role == "mixer" else part.forward(y, ctx)
                if pending is not None:
                    ops.residual_add(x, pending)
                regs.pending = self._own(out, (T, H))
            elif role == "head":
                logits.copy_(part.forward(self._view(regs.y, (n_y, H), self.dtype)))
            else:
                raise RuntimeError(f"unknown role {role!r} of a Python record")
            return 0
        except BaseException as e:          # carried across the foreign call and raised by forward()
            self._raised = e
            return 1


_BARE: dict = {}
# Entry points for programs that parts make for themselves (None: the compiled libraries'); tests that run the
# parts without a GPU put recording stand-ins here.
PART_ENTRIES: dict = {"entries": None, "sms": None}


def part_program(dtype: torch.dtype, device, hidden: int) -> Program:
    """The program a part runs its own record in when its forward() is called by itself (a Python block
    arrangement, a test of the part alone): no records of its own, activations of `dtype` and width `hidden`."""
    key = (dtype, torch.device(device), int(hidden), id(PART_ENTRIES["entries"]), PART_ENTRIES["sms"])
    prog = _BARE.get(key)
    if prog is None:
        prog = _BARE[key] = Program(None, PART_ENTRIES["entries"], PART_ENTRIES["sms"], dtype=dtype, device=device, hidden=hidden)
    return prog
