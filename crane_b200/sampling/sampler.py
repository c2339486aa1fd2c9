"""Choosing the next token from float logits on the device, every row with its
own options.

What the reference samples with (crane-serve/src/engine/sampling.rs:117-327,
crane-core/src/models/hunyuan_dense/model.rs:304-339): greedy when no
temperature is given or it is <= 0; a repetition penalty over the last
``repeat_last_n`` tokens; temperature via the Gumbel-max trick; top-k (at most
64 on the device) and top-p inside the top-k set.  All of it runs in the
kernels of ``csrc/sampling.cu``; only the chosen token ids come back to the host.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch


@dataclass
class SamplingParams:
    temperature: Optional[float] = None     # None or <= 0: greedy
    top_p: Optional[float] = None           # None, <= 0 or >= 1: off
    top_k: Optional[int] = None             # None or 0: off; clamped to 64 on the device
    repetition_penalty: float = 1.0
    repeat_last_n: int = 64
    seed: Optional[int] = None              # None: from the clock, as the reference's server does

    @property
    def greedy(self) -> bool:
        return self.temperature is None or self.temperature <= 0.0

    def resolved_seed(self) -> int:
        if self.seed is None:
            self.seed = time.time_ns() & ((1 << 63) - 1)
        return self.seed


class _Stage:
    """One pinned host block of everything the host stages for a step's sampling
    kernels, and the event recorded behind the transfers that read it."""

    def __init__(self, opt_bytes: int, max_rows: int):
        self.opts = torch.zeros(opt_bytes, dtype=torch.uint8).pin_memory()
        self.pen = torch.ones(max_rows, dtype=torch.float32).pin_memory()
        self.ctx_len = torch.zeros(max_rows, dtype=torch.int32).pin_memory()
        self.ctx: Optional[torch.Tensor] = None          # [max_rows, max_context] int32, pinned
        self.copied = torch.cuda.Event()
        self.copied.record()


class Sampler:
    def __init__(self, rt, max_rows: int, max_context: int = 64, out: Optional[torch.Tensor] = None):
        """``out``: the int32 device buffer [max_rows] that the chosen ids are
        written to (one of the sampler's own if not given)."""
        self.rt = rt
        self.max_rows = max_rows
        self.max_context = max_context
        dev = rt.device
        self.out = out if out is not None else torch.zeros(max_rows, dtype=torch.int32, device=dev)
        # two host buffers in turn: a read-back may be in flight while the last one is read
        self._hosts = [torch.zeros(max_rows, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._turn = 0
        # What the host stages for a step's kernels (per-row options, penalty contexts) is copied to
        # the device by a transfer queued BEHIND the step's forward pass, so the device reads the
        # pinned block long after the host has gone on, possibly to stage the next step.  Hence two
        # blocks in turn, each with an event recorded behind its transfer; a block is rewritten
        # only after the transfer that last read it has happened.
        r8 = (max_rows + 1) // 2 * 2
        self._r8 = r8
        self._opt_bytes = r8 * 4 * 3 + max_rows * 8 * 2
        self._stages = [_Stage(self._opt_bytes, max_rows) for _ in range(2)]
        self._stage_turn = 0
        self.d_opts = torch.zeros(self._opt_bytes, dtype=torch.uint8, device=dev)
        self.d_pen = torch.ones(max_rows, dtype=torch.float32, device=dev)
        self._alloc_context(max_context)

    def _opt_views(self, buf: torch.Tensor):
        r8, n = self._r8, self.max_rows
        a = r8 * 4
        return (buf[0:a].view(torch.float32), buf[a:2 * a].view(torch.int32),
                buf[2 * a:3 * a].view(torch.float32), buf[3 * a:3 * a + n * 8].view(torch.int64),
                buf[3 * a + n * 8:3 * a + n * 16].view(torch.int64))

    def _alloc_context(self, n: int) -> None:
        self.max_context = n
        for st in self._stages:
            st.copied.synchronize()
            st.ctx = torch.zeros((self.max_rows, n), dtype=torch.int32).pin_memory()
        self.d_ctx = torch.zeros((self.max_rows, n), dtype=torch.int32, device=self.rt.device)
        self.d_ctx_len = torch.zeros(self.max_rows, dtype=torch.int32, device=self.rt.device)

    def _next_stage(self) -> "_Stage":
        st = self._stages[self._stage_turn]
        self._stage_turn ^= 1
        st.copied.synchronize()          # the transfer that last read this block has happened
        return st

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                      histories: Optional[Sequence[Sequence[int]]] = None,
                      counters: Optional[Sequence[int]] = None) -> torch.Tensor:
        """logits [R, V] float (changed in place by a repetition penalty).
        ``histories``: per row the request's tokens so far; ``counters``: per row
        how many tokens the request has sampled before (keys the random
        stream).  Returns int32 [R] on the device."""
        rows = logits.shape[0]
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows to sample, the sampler holds {self.max_rows}")
        k = self.rt.kernels
        out = self.out[:rows]
        penal = [p.repetition_penalty != 1.0 for p in params]
        greedy = all(p.greedy for p in params)
        if not any(penal) and greedy:
            k.sample(logits, out)
            self.rt.launches += 1
            return out
        if any(penal):
            need = max(p.repeat_last_n for p, on in zip(params, penal) if on)
            if need > self.max_context:
                self._alloc_context(need)
        st = self._next_stage()
        if any(penal):
            pen, ctx, ctx_len = st.pen.numpy(), st.ctx.numpy(), st.ctx_len.numpy()
            for r, (p, on) in enumerate(zip(params, penal)):
                ctx_len[r] = 0
                pen[r] = 1.0
                if on and histories is not None and p.repeat_last_n > 0:
                    h = list(histories[r])[-p.repeat_last_n:]
                    ctx[r, :len(h)] = h
                    ctx_len[r] = len(h)
                    pen[r] = p.repetition_penalty
            self.d_ctx[:rows].copy_(st.ctx[:rows], non_blocking=True)
            self.d_ctx_len[:rows].copy_(st.ctx_len[:rows], non_blocking=True)
            self.d_pen[:rows].copy_(st.pen[:rows], non_blocking=True)
            k.repetition_penalty(logits, self.d_ctx[:rows], self.d_ctx_len[:rows], self.d_pen[:rows])
            self.rt.launches += 1
        if greedy:
            st.copied.record()
            k.sample(logits, out)
            self.rt.launches += 1
            return out
        temp, topk, topp, seed, counter = (v.numpy() for v in self._opt_views(st.opts))
        for r, p in enumerate(params):
            temp[r] = 0.0 if p.greedy else p.temperature
            topk[r] = p.top_k or 0
            topp[r] = 1.0 if p.top_p is None else p.top_p
            seed[r] = p.resolved_seed()
            counter[r] = counters[r] if counters is not None else 0
        self.d_opts.copy_(st.opts, non_blocking=True)
        st.copied.record()
        d_temp, d_topk, d_topp, d_seed, d_counter = self._opt_views(self.d_opts)
        k.sample(logits, out, temperature=d_temp, top_k=d_topk, top_p=d_topp, seed=d_seed,
                 counter=d_counter)
        self.rt.launches += 1
        return out

    def sample_async(self, logits, params, histories=None, counters=None):
        """Samples and starts the copy to the host.  Returns (event, pinned
        int32 view): the ids are there once the event has happened.  At most
        two such read-backs may be open at a time."""
        out = self.sample_device(logits, params, histories, counters)
        n = out.shape[0]
        host = self._hosts[self._turn][:n]
        self._turn ^= 1
        host.copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(self.rt.device))
        return event, host

    def sample(self, logits, params, histories=None, counters=None) -> List[int]:
        event, host = self.sample_async(logits, params, histories, counters)
        event.synchronize()
        return host.tolist()
