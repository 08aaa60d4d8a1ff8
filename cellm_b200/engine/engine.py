"""The engine: requests in, tokens out, over one model on one GPU.

Its calls mirror the reference engine's
(crates/cellm-sdk/src/lib.rs:227-502: create_session / submit_tokens /
step_decode / cancel_session / stats), with one difference in kind: a step
here is one batch over all live requests, not one token of one session.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..models import load_model
from ..sampling import RequestSampler, SamplingParams, sample_rows, session_seed
from .scheduler import Scheduler
from .step import StepRunner


@dataclass
class RequestOutput:
    request_id: int
    tokens: list[int] = field(default_factory=list)
    finished: bool = False
    finish_reason: str = ""


class Engine:
    def __init__(self, model, config: Optional[EngineConfig] = None, **overrides):
        """`model`: a folder with config.json and model.safetensors, or the
        (config, plan, model) triple that `cellm_b200.models.load_model` returned
        (several engines may share one loaded model). Keyword arguments override
        fields of EngineConfig (dtype, total_blocks, ...)."""
        self.config = config or EngineConfig()
        for k, v in overrides.items():
            if not hasattr(self.config, k):
                raise TypeError(f"EngineConfig has no field {k!r}")
            setattr(self.config, k, v)
        self.config.__post_init__()
        c = self.config
        if isinstance(model, (str, bytes)) or hasattr(model, "__fspath__"):
            model = load_model(model, c.dtype, c.device)
        self.model_config, self.plan, self.model = model
        if self.model.dtype != c.dtype:
            raise ValueError(f"the loaded model computes in {self.model.dtype}, the engine was asked for {c.dtype}")
        self.cache = CacheManager(self.model.cache_needs(), [e.cache_of for e in self.plan.order],
                                  c.tokens_per_block, c.total_blocks, c.max_num_seqs, c.dtype, c.device)
        self.runner = StepRunner(self.model, self.cache, use_graphs=c.use_cuda_graphs)
        self.runner.capture_after = c.capture_after
        self.scheduler = Scheduler(self.cache, c.max_batch_tokens, c.prefill_chunk, self.plan.max_positions)
        self._samplers: dict[int, RequestSampler] = {}
        self._outputs: dict[int, RequestOutput] = {}
        self._next_id = 0
        self._prompt_len: dict[int, int] = {}
        # the step whose tokens are still on the device: (requests in row order, where each token goes among its
        # request's tokens, pinned buffer, rows, event after the copy), and how many such tokens each request has
        self._ahead = None
        self._pending: dict[int, int] = {}
        self._check_due = False
        self.max_layers: Optional[int] = None     # run only the first layers (tools/infer --max-layers)
        # Called after every step's forward pass with (ids of the requests whose logits were formed, in row
        # order; the float32 logits [rows, vocab] on the device, valid until the next step): for inspection.
        self.on_logits = None

    # -------------------------------------------------------------- requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    seed: Optional[int] = None) -> int:
        """Queues a prompt (token ids); returns the request's id. The request's
        random stream starts from `seed` (default: params.seed)."""
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        V = self.plan.vocab_size
        if not prompt:
            raise ValueError("a prompt needs at least one token")
        bad = [t for t in prompt if not 0 <= t < V]
        if bad:
            raise ValueError(f"token id {bad[0]} outside the vocabulary of {V}")
        if params.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        rid = self._next_id
        self._next_id += 1
        self.scheduler.add_request(rid, prompt, params.max_new_tokens)
        self._samplers[rid] = RequestSampler(params, params.seed if seed is None else seed, prompt)
        self._outputs[rid] = RequestOutput(rid)
        self._prompt_len[rid] = len(prompt)
        return rid

    def cancel(self, request_id: int) -> None:
        self.scheduler.cancel(request_id)
        self._finish(request_id)

    def _finish(self, rid: int) -> None:
        self._check_due = True       # the device error word is read once per finished request, not per step
        out = self._outputs[rid]
        out.finished = True
        out.finish_reason = self.scheduler.info(rid)["finish_reason"]
        self.scheduler.forget(rid)
        self._samplers.pop(rid, None)
        self._prompt_len.pop(rid, None)
        self._pending.pop(rid, None)

    def has_unfinished(self) -> bool:
        return self._ahead is not None or not self.scheduler.stats()["idle"]

    # ------------------------------------------------------------------ step
    def step(self) -> list[tuple[int, int]]:
        """Plans and runs one batch; returns (request, new token) pairs. A captured decode step of greedy requests
        leaves its tokens on the device (EngineConfig.run_ahead): they are returned by the next call, which has
        launched its own step before it reads them. Otherwise the pairs are this step's."""
        produced: list[tuple[int, int]] = []
        before, self._ahead = self._ahead, None
        rows, preempted, admitted, n_entries = self.scheduler.schedule_rows()
        for rid, slot in admitted:
            self.cache.zero_slot(slot)
        if n_entries == 0 or preempted:
            for rid in list(self._outputs):
                if not self._outputs[rid].finished and self.scheduler.has(rid) and not self._pending.get(rid) \
                        and self.scheduler.info(rid)["state"] == "finished":
                    self._finish(rid)     # the scheduler gave the request up (cannot fit)
        if n_entries == 0:
            if before is not None:
                produced += self._settle(before)
            return produced
        logits = self.runner.run_planned(self.scheduler, self.max_layers)
        self.scheduler.step_done()
        ahead = bool(rows) and self._tokens_may_stay(rows)
        if ahead:
            # every row has a token, value to come; the scheduler counts it now (a request may end by its length)
            self.scheduler.append_pending_rows(len(rows))
            where = []
            for rid in rows:
                where.append(self._prompt_len[rid] + len(self._outputs[rid].tokens) + self._pending.get(rid, 0))
                self._pending[rid] = self._pending.get(rid, 0) + 1
            self._ahead = (list(rows), where) + self.runner.tokens_to_host()
        if before is not None:
            produced += self._settle(before)          # the step before this one: its tokens come first
        if rows and not ahead:
            if self.on_logits is not None:
                self.on_logits(list(rows), logits)
            live = [not self._outputs[r].finished for r in rows]      # a token just read may have ended a request of this step
            samplers = [self._samplers.get(r) for r in rows]
            if all(live):
                tokens = sample_rows(logits, samplers, self.runner.last_argmax)
            else:
                tokens = self._sample_live(logits, samplers, live)
            self.runner.check_rarely()
            eos = self.plan.eos_token_id
            stops = [ok and s.params.stop_eos and eos is not None and tok == eos for ok, s, tok in zip(live, samplers, tokens)]
            finished = self.scheduler.append_rows([tok if ok else -2 for ok, tok in zip(live, tokens)], stops)
            for rid, ok, s, tok, fin in zip(rows, live, samplers, tokens, finished):
                if not ok:
                    continue
                s.history.append(tok)
                self._outputs[rid].tokens.append(tok)
                produced.append((rid, tok))
                if fin:
                    self._finish(rid)
        if self._check_due:
            self._check_due = False
            self.runner.check()
        return produced

    def _tokens_may_stay(self, rows) -> bool:
        """The step just launched was a captured decode step and every one of its tokens is an arg-max."""
        if not self.config.run_ahead or self.on_logits is not None or self.runner.last_argmax is None:
            return False
        if self.runner.last_argmax.numel() != len(rows):
            return False
        return all(self._samplers[r].params.temperature <= 0.0 for r in rows)

    def _sample_live(self, logits, samplers, live) -> list[int]:
        """sample_rows for the rows whose requests still run; -2 elsewhere."""
        import torch
        keep = [i for i, ok in enumerate(live) if ok]
        out = [-2] * len(live)
        if keep:
            idx = torch.tensor(keep, dtype=torch.long, device=logits.device)
            for i, tok in zip(keep, sample_rows(logits.index_select(0, idx), [samplers[i] for i in keep], None)):
                out[i] = tok
        return out

    def _settle(self, ahead) -> list[tuple[int, int]]:
        """Reads the tokens a step left on the device and gives them to the scheduler and the outputs."""
        rows, where, buf, n, event = ahead
        event.synchronize()
        values = buf[:n].tolist()
        self.runner.check_rarely()
        eos = self.plan.eos_token_id
        ids, index, tokens, stops = [], [], [], []
        for rid, at, tok in zip(rows, where, values):
            if rid in self._pending:
                self._pending[rid] -= 1
            if self._outputs[rid].finished:
                continue              # ended by an earlier token (or cancelled) after this step was launched
            ids.append(rid)
            index.append(at)
            tokens.append(tok)
            stops.append(self._samplers[rid].params.stop_eos and eos is not None and tok == eos)
        produced = []
        if ids:
            finished = self.scheduler.resolve_rows(ids, index, tokens, stops)
            for rid, tok, stop, fin in zip(ids, tokens, stops, finished):
                self._samplers[rid].history.append(tok)
                self._outputs[rid].tokens.append(tok)
                produced.append((rid, tok))
                # a request that ended by its length did so when its last token was counted, which may be the token of
                # the step after this one: it is finished here only once that one has been read too
                if stop or (fin and not self._pending.get(rid)):
                    self._finish(rid)
        return produced

    def output(self, request_id: int) -> RequestOutput:
        return self._outputs[request_id]

    def release_output(self, request_id: int) -> RequestOutput:
        return self._outputs.pop(request_id)

    # -------------------------------------------------------------- generate
    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> list[list[int]]:
        """Generated token ids for each prompt, host tokens in and out. Prompt i
        draws from a random stream seeded by the reference engine's per-session
        mix of i and params.seed (crates/cellm-sdk/src/lib.rs:526-535)."""
        params = params or SamplingParams()
        if params.max_new_tokens == 0:
            return [[] for _ in prompts]
        ids = [self.add_request(p, params, seed=session_seed(i, params.seed)) for i, p in enumerate(prompts)]
        while self.has_unfinished():
            before = self.scheduler.stats()
            if not self.step() and self.has_unfinished():
                after = self.scheduler.stats()
                if after["running"] == 0 and after["waiting"] >= before["waiting"] > 0 and not after["preemptions"] > before["preemptions"]:
                    raise RuntimeError(f"{after['waiting']} requests wait but none can be admitted "
                                       f"(free pages {self.stats()['free_pages']}, free slots {self.cache.free_slots})")
        self.runner.check()          # a fault a kernel flagged in any step of these requests
        outs = [self.release_output(i) for i in ids]
        for o in outs:
            if o.finish_reason == "out_of_pages":
                raise RuntimeError(f"request {o.request_id} could not fit the cache pool")
        return [o.tokens for o in outs]

    def stats(self) -> dict:
        """crates/cellm-sdk/src/lib.rs:495-502: active sessions and used / free pages."""
        s = self.scheduler.stats()
        groups = range(len(self.cache.paged_keys))
        s.update({"free_pages": [self.cache.free_pages(g) for g in groups],
                  "total_pages": list(self.cache.group_pages), "free_slots": self.cache.free_slots,
                  "steps_run": self.runner.steps, "tokens_run": self.runner.tokens})
        return s
