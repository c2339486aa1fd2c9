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
    row: int = -1                     # its row in the sampler's output of the last launched step


@dataclass
class _InFlight:
    """A launched step whose sampled tokens have not been read yet."""
    ids: List[int]
    event: torch.cuda.Event
    host: Optional[torch.Tensor]      # pinned int32 [len(ids)], valid after the event
    deferred: bool                    # the scheduler holds placeholders for these tokens


class LLMEngine:
    """With ``async_scheduling`` the engine plans and launches step N + 1 before
    it reads the tokens that step N sampled: the scheduler keeps a placeholder
    for each, and the embedding of step N + 1 takes the token ids from the
    sampler's output on the device.  The host work of a step then overlaps the
    device work of the step before it.  A request that stops on an EOS token
    in step N has been run one step too far; that step's token is dropped.
    Steps are not overlapped while a live request has a repetition penalty,
    since the penalty needs the tokens on the host."""

    def __init__(self, runner: ModelRunner):
        self.runner = runner
        cfg = runner.cfg
        self.scheduler = Scheduler(runner.table, cfg.max_concurrent, cfg.max_batched_tokens,
                                   min(cfg.chunk_size, cfg.max_batched_tokens), runner.max_seq_len)
        self.sampler = Sampler(runner.rt, cfg.max_concurrent, out=runner.deferred_tokens)
        self.async_scheduling = bool(cfg.async_scheduling)
        self._inflight: Optional[_InFlight] = None
        self._live: Dict[int, _Live] = {}
        self._next_id = 1
        self.finished: Dict[int, RequestOutput] = {}
        self.timers = {"prefill_s": 0.0, "decode_s": 0.0, "prefill_tokens": 0, "decode_tokens": 0}
        self.last_step_kind = ""          # of the batch the last step() launched: "decode" (single tokens
                                          # only), "prefill" (prompt portions only), "mixed", or "" (none)

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
        return self.scheduler.has_work() or self._inflight is not None

    def _finish(self, rid: int) -> None:
        st = self.scheduler.state(rid)
        self.finished[rid] = RequestOutput(rid, st.prompt_len, self.scheduler.tokens(rid),
                                           st.finish_reason, st.preemptions)
        self.scheduler.drop(rid)
        self._live.pop(rid, None)

    # ---- one step -------------------------------------------------------
    def step(self) -> List[tuple]:
        """Plans and launches one batch.  Returns (request id, token, finish
        reason) for every token that has become known: this batch's, or, when
        steps overlap, the batch's before it."""
        t0 = time.perf_counter()
        out: List[tuple] = []
        overlap = self.async_scheduling and all(
            l.params.repetition_penalty == 1.0 for l in self._live.values())
        if self._inflight is not None and not overlap:
            out += self.flush()
        plan = self.scheduler.schedule()
        for rid in self.scheduler.last_failed():
            self._finish(rid)
        cur = self._launch(plan, overlap) if plan else None
        self.last_step_kind = ""
        if self._inflight is not None:
            out += self.flush()
        if cur is not None:
            self._inflight = cur
            if not cur.deferred:
                out += self.flush()
            n_tok = sum(len(p.tokens) for p in plan)
            kind = "decode" if all(len(p.tokens) == 1 for p in plan) else "prefill"
            self.last_step_kind = kind if kind == "decode" or all(len(p.tokens) > 1 for p in plan) else "mixed"
            self.timers[kind + "_s"] += time.perf_counter() - t0
            self.timers[kind + "_tokens"] += n_tok
        return out

    def _launch(self, plan, overlap: bool) -> _InFlight:
        entries = []
        for p in plan:
            toks = p.tokens
            if toks[-1] < 0:
                # the request's last token is still on the device, in the row it was sampled to
                toks = toks.copy()
                toks[-1] = -(self._live[p.request_id].row + 2)
            entries.append(StepEntry(p.request_id, toks, [len(toks) - 1] if p.sample else []))
        logits = self.runner.step(entries, reserved=True)
        sampled = [p.request_id for p in plan if p.sample]
        if not sampled:
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(self.runner.rt.device))
            return _InFlight([], event, None, overlap)
        lives = [self._live[rid] for rid in sampled]
        params = [l.params for l in lives]
        need_hist = any(q.repetition_penalty != 1.0 for q in params)
        hist = [self.scheduler.tokens(rid) for rid in sampled] if need_hist else None
        event, host = self.sampler.sample_async(logits, params, hist, [l.sampled for l in lives])
        for row, l in enumerate(lives):
            l.sampled += 1
            l.row = row
        if overlap:
            self.scheduler.expect_tokens(sampled)
        return _InFlight(sampled, event, host, overlap)

    def flush(self) -> List[tuple]:
        """Waits for the launched step, if one is open, and takes its tokens in."""
        f, self._inflight = self._inflight, None
        if f is None:
            return []
        f.event.synchronize()
        if not f.ids:
            return []
        toks = f.host.tolist()
        if f.deferred:
            reasons = self.scheduler.resolve_tokens(f.ids, toks)
        else:
            reasons = self.scheduler.on_tokens(f.ids, toks)
        out: List[tuple] = []
        for rid, tok, reason in zip(f.ids, toks, reasons):
            live = self._live.get(rid)
            if live is None:
                continue                      # finished a step earlier; this token was one too many
            out.append((rid, tok, reason))
            if live.on_token is not None:
                live.on_token(rid, tok, reason)
            if reason is not None:
                self._finish(rid)
        return out

    def run_until_done(self) -> Dict[int, RequestOutput]:
        while self.has_work():
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
