"""The engine loop: requests in, tokens out, through scheduler, step function
and sampler.

Counterpart of the reference's ``InferenceEngine``
(crane-serve/src/engine/mod.rs:316-378: drain requests, schedule, execute the
step, send tokens, finish and clean up) without its threads and channels: the
caller adds requests and calls ``step()`` or ``run_until_done()``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..sampling import Sampler, SamplingParams
from .scheduler import Scheduler
from .step import ModelRunner, StepEntry


@dataclass
class RequestOutput:
    request_id: int
    prompt_len: int
    tokens: List[int]                 # prompt ++ generated
    finish_reason: Optional[str]
    preemptions: int = 0

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.prompt_len:]


@dataclass
class _Live:
    params: SamplingParams
    on_token: Optional[Callable[[int, int, Optional[str]], None]]
    sampled: int = 0


class LLMEngine:
    def __init__(self, runner: ModelRunner):
        self.runner = runner
        cfg = runner.cfg
        self.scheduler = Scheduler(runner.table, cfg.max_concurrent, cfg.max_batched_tokens,
                                   min(cfg.chunk_size, cfg.max_batched_tokens), runner.max_seq_len)
        self.sampler = Sampler(runner.rt, cfg.max_concurrent)
        self._live: Dict[int, _Live] = {}
        self._next_id = 1
        self.finished: Dict[int, RequestOutput] = {}
        self.timers = {"prefill_s": 0.0, "decode_s": 0.0, "prefill_tokens": 0, "decode_tokens": 0}

    # ---- requests -------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    max_new_tokens: int = 128, eos_token_ids: Optional[Sequence[int]] = None,
                    on_token: Optional[Callable[[int, int, Optional[str]], None]] = None) -> int:
        """Queues a request and returns its id.  ``on_token(id, token, finish
        reason or None)`` is called for every generated token."""
        vocab = self.runner.spec.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"prompt holds a token id outside [0, {vocab})")
        rid = self._next_id
        self._next_id += 1
        eos = list(self.runner.spec.eos_token_ids if eos_token_ids is None else eos_token_ids)
        state = self.scheduler.add(rid, prompt, max_new_tokens, eos)
        if state == "finished":
            self._finish(rid)
        else:
            self._live[rid] = _Live(params or SamplingParams(), on_token)
        return rid

    def cancel(self, rid: int) -> None:
        if rid in self._live:
            self.scheduler.cancel(rid)
            self._finish(rid)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def _finish(self, rid: int) -> None:
        st = self.scheduler.state(rid)
        self.finished[rid] = RequestOutput(rid, st.prompt_len, self.scheduler.tokens(rid),
                                           st.finish_reason, st.preemptions)
        self.scheduler.drop(rid)
        self._live.pop(rid, None)

    # ---- one step -------------------------------------------------------
    def step(self) -> List[tuple]:
        """One scheduled batch.  Returns (request id, token, finish reason) for
        every token generated in it."""
        plan = self.scheduler.schedule()
        for rid in self.scheduler.last_failed():
            self._finish(rid)
        if not plan:
            return []
        t0 = time.perf_counter()
        entries = [StepEntry(p.request_id, p.tokens, [len(p.tokens) - 1] if p.sample else [])
                   for p in plan]
        logits = self.runner.step(entries, reserved=True)
        sampled = [p for p in plan if p.sample]
        out: List[tuple] = []
        if sampled:
            params = [self._live[p.request_id].params for p in sampled]
            need_hist = any(q.repetition_penalty != 1.0 for q in params)
            hist = [self.scheduler.tokens(p.request_id) for p in sampled] if need_hist else None
            counters = [self._live[p.request_id].sampled for p in sampled]
            toks = self.sampler.sample(logits, params, hist, counters)
            reasons = self.scheduler.on_tokens([p.request_id for p in sampled], toks)
            for p, tok, reason in zip(sampled, toks, reasons):
                live = self._live[p.request_id]
                live.sampled += 1
                out.append((p.request_id, tok, reason))
                if live.on_token is not None:
                    live.on_token(p.request_id, tok, reason)
                if reason is not None:
                    self._finish(p.request_id)
        else:
            torch.cuda.current_stream(self.runner.rt.device).synchronize()
        dt = time.perf_counter() - t0
        n_tok = sum(len(p.tokens) for p in plan)
        kind = "decode" if all(len(p.tokens) == 1 for p in plan) else "prefill"
        self.timers[kind + "_s"] += dt
        self.timers[kind + "_tokens"] += n_tok
        return out

    def run_until_done(self) -> Dict[int, RequestOutput]:
        while self.scheduler.has_work():
            self.step()
        self.runner.rt.check_errors()
        done, self.finished = self.finished, {}
        return done

    def stats(self) -> dict:
        """Counters in the manner of the reference's ``EngineStats``
        (crane-serve/src/engine/stats.rs:6-84)."""
        s = self.scheduler.stats()
        t = self.timers
        s.update({
            "waiting": self.scheduler.num_waiting, "running": self.scheduler.num_running,
            "free_pages": [self.runner.table.free_pages(g) for g in range(max(1, self.runner.num_groups))],
            "avg_prefill_tokens_per_sec": t["prefill_tokens"] / t["prefill_s"] if t["prefill_s"] else 0.0,
            "avg_decode_tokens_per_sec": t["decode_tokens"] / t["decode_s"] if t["decode_s"] else 0.0,
            "kernel_launches": self.runner.rt.launches,
        })
        return s
