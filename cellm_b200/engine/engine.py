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
        self.scheduler = Scheduler(self.cache, c.max_batch_tokens, c.prefill_chunk, self.plan.max_positions)
        self._samplers: dict[int, RequestSampler] = {}
        self._outputs: dict[int, RequestOutput] = {}
        self._next_id = 0
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

    def has_unfinished(self) -> bool:
        return not self.scheduler.stats()["idle"]

    # ------------------------------------------------------------------ step
    def step(self) -> list[tuple[int, int]]:
        """Runs one batch; returns (request, new token) for every request that
        produced a token in it."""
        rows, preempted, admitted, n_entries = self.scheduler.schedule_rows()
        for rid, slot in admitted:
            self.cache.zero_slot(slot)
        if n_entries == 0 or preempted:
            for rid in list(self._outputs):
                if not self._outputs[rid].finished and self.scheduler.has(rid) \
                        and self.scheduler.info(rid)["state"] == "finished":
                    self._finish(rid)     # the scheduler gave the request up (cannot fit)
        if n_entries == 0:
            return []
        logits = self.runner.run_planned(self.scheduler, self.max_layers)
        self.scheduler.step_done()
        produced = []
        if rows:
            if self.on_logits is not None:
                self.on_logits(list(rows), logits)
            samplers = [self._samplers[r] for r in rows]
            tokens = sample_rows(logits, samplers, self.runner.last_argmax)
            self.runner.check_rarely()
            eos = self.plan.eos_token_id
            stops = [s.params.stop_eos and eos is not None and tok == eos for s, tok in zip(samplers, tokens)]
            finished = self.scheduler.append_rows(tokens, stops)
            for rid, s, tok, fin in zip(rows, samplers, tokens, finished):
                s.history.append(tok)
                self._outputs[rid].tokens.append(tok)
                produced.append((rid, tok))
                if fin:
                    self._finish(rid)
        if self._check_due:
            self._check_due = False
            self.runner.check()
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
