"""Python face of the native scheduler (``csrc/host/scheduler.cpp``)."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int32, c_int64, c_void_p
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..cache.manager import PageTable
from ..csrc import build

FINISH_REASONS = {0: None, 1: "stop", 2: "length", 3: "cancelled", 4: "cache_too_small"}

_lib = None


def _host():
    global _lib
    if _lib is None:
        lib = build.load_host()
        I, L, P = c_int, c_int64, c_void_p
        sig = {
            "crane_sched_create": ([P, I, I, I, I], P),
            "crane_sched_destroy": ([P], None),
            "crane_sched_add": ([P, L, P, I, I, P, I], I),
            "crane_sched_schedule": ([P, P, P, P, P, I, P, I, P], I),
            "crane_sched_on_token": ([P, L, c_int32], I),
            "crane_sched_on_tokens": ([P, I, P, P, P], None),
            "crane_sched_expect_tokens": ([P, I, P], None),
            "crane_sched_resolve_tokens": ([P, I, P, P, P], None),
            "crane_sched_cancel": ([P, L], I),
            "crane_sched_drop": ([P, L], I),
            "crane_sched_has_work": ([P], I),
            "crane_sched_num_waiting": ([P], I),
            "crane_sched_num_running": ([P], I),
            "crane_sched_state": ([P, L, P], I),
            "crane_sched_tokens": ([P, L, P, I], I),
            "crane_sched_stats": ([P, P], None),
            "crane_sched_last_preempted": ([P, P, I], I),
            "crane_sched_last_failed": ([P, P, I], I),
        }
        for name, (args, res) in sig.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, res
        _lib = lib
    return _lib


@dataclass
class PlannedEntry:
    request_id: int
    start: int
    tokens: np.ndarray      # int32 view, valid until the next schedule() call
    sample: bool


@dataclass
class RequestState:
    finish_reason: Optional[str]
    prompt_len: int
    num_tokens: int
    computed: int
    running: bool
    preemptions: int


class Scheduler:
    """Admits, cuts prompts into portions under the token budget, decodes,
    finishes and frees; preempts the most recently admitted request when pages
    run out."""

    def __init__(self, table: PageTable, max_running: int, max_batched_tokens: int, chunk_size: int,
                 max_seq_len: int):
        self._lib = _host()
        self._table = table                      # keeps the native cache alive
        self._h = self._lib.crane_sched_create(table.handle, max_running, max_batched_tokens,
                                               chunk_size, max_seq_len)
        if not self._h:
            raise ValueError("invalid scheduler settings")
        self.max_running, self.max_batched_tokens = max_running, max_batched_tokens
        self.chunk_size, self.max_seq_len = chunk_size, max_seq_len
        cap = max_running + 1
        self._ids = np.zeros(cap, dtype=np.int64)
        self._start = np.zeros(cap, dtype=np.int32)
        self._count = np.zeros(cap, dtype=np.int32)
        self._sample = np.zeros(cap, dtype=np.int32)
        self._tokens = np.zeros(max_batched_tokens, dtype=np.int32)
        self._ntok = c_int32(0)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.crane_sched_destroy(h)

    def add(self, rid: int, prompt: Sequence[int], max_new_tokens: int, eos: Sequence[int]) -> str:
        """"queued", "finished" (nothing may be generated) or raises for a
        prompt that is empty or longer than the sequence limit."""
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        e = np.ascontiguousarray(list(eos), dtype=np.int32)
        r = self._lib.crane_sched_add(self._h, rid, p.ctypes.data, len(p), int(max_new_tokens),
                                      e.ctypes.data, len(e))
        if r == -2:
            raise ValueError(f"request id {rid} is in use")
        if r == -1:
            raise ValueError(f"prompt of {len(p)} tokens refused: it must hold 1 to "
                             f"{self.max_seq_len} tokens (the sequence limit)")
        return "finished" if r == 1 else "queued"

    def schedule(self) -> List[PlannedEntry]:
        n = self._lib.crane_sched_schedule(
            self._h, self._ids.ctypes.data, self._start.ctypes.data, self._count.ctypes.data,
            self._sample.ctypes.data, len(self._ids), self._tokens.ctypes.data, len(self._tokens),
            ctypes.byref(self._ntok))
        if n < 0:
            raise RuntimeError("the scheduler planned more than its caller's arrays hold")
        out, off = [], 0
        for i in range(n):
            c = int(self._count[i])
            out.append(PlannedEntry(int(self._ids[i]), int(self._start[i]),
                                    self._tokens[off:off + c], bool(self._sample[i])))
            off += c
        return out

    def on_token(self, rid: int, token: int) -> Optional[str]:
        return FINISH_REASONS[self._lib.crane_sched_on_token(self._h, rid, int(token))]

    def on_tokens(self, ids: Sequence[int], tokens: Sequence[int]) -> List[Optional[str]]:
        """``on_token`` for several requests in one native call."""
        a = np.asarray(ids, dtype=np.int64)
        t = np.asarray(tokens, dtype=np.int32)
        r = np.zeros(len(a), dtype=np.int32)
        self._lib.crane_sched_on_tokens(self._h, len(a), a.ctypes.data, t.ctypes.data, r.ctypes.data)
        return [FINISH_REASONS[int(v)] for v in r]

    def expect_tokens(self, ids: Sequence[int]) -> None:
        """The tokens sampled for these requests are still on the device: a
        placeholder takes each one's place so that the next step can be planned."""
        a = np.asarray(ids, dtype=np.int64)
        self._lib.crane_sched_expect_tokens(self._h, len(a), a.ctypes.data)

    def resolve_tokens(self, ids: Sequence[int], tokens: Sequence[int]) -> List[Optional[str]]:
        """Fills the oldest placeholder of each request in; returns the finish reasons."""
        a = np.asarray(ids, dtype=np.int64)
        t = np.asarray(tokens, dtype=np.int32)
        r = np.zeros(len(a), dtype=np.int32)
        self._lib.crane_sched_resolve_tokens(self._h, len(a), a.ctypes.data, t.ctypes.data, r.ctypes.data)
        return [FINISH_REASONS[int(v)] for v in r]

    def cancel(self, rid: int) -> None:
        self._lib.crane_sched_cancel(self._h, rid)

    def drop(self, rid: int) -> None:
        self._lib.crane_sched_drop(self._h, rid)

    def has_work(self) -> bool:
        return bool(self._lib.crane_sched_has_work(self._h))

    @property
    def num_waiting(self) -> int:
        return self._lib.crane_sched_num_waiting(self._h)

    @property
    def num_running(self) -> int:
        return self._lib.crane_sched_num_running(self._h)

    def state(self, rid: int) -> RequestState:
        out = np.zeros(6, dtype=np.int32)
        if self._lib.crane_sched_state(self._h, rid, out.ctypes.data) != 0:
            raise KeyError(f"unknown request {rid}")
        return RequestState(FINISH_REASONS[int(out[0])], int(out[1]), int(out[2]), int(out[3]),
                            bool(out[4]), int(out[5]))

    def tokens(self, rid: int) -> List[int]:
        n = self._lib.crane_sched_tokens(self._h, rid, None, 0)
        if n < 0:
            raise KeyError(f"unknown request {rid}")
        out = np.zeros(max(n, 1), dtype=np.int32)
        self._lib.crane_sched_tokens(self._h, rid, out.ctypes.data, n)
        return out[:n].tolist()

    def stats(self) -> dict:
        out = np.zeros(8, dtype=np.int64)
        self._lib.crane_sched_stats(self._h, out.ctypes.data)
        keys = ("steps", "requests", "finished", "prompt_tokens", "generated_tokens",
                "scheduled_tokens", "preemptions", "rejected")
        return {k: int(v) for k, v in zip(keys, out)}

    def last_preempted(self) -> List[int]:
        out = np.zeros(self.max_running + 1, dtype=np.int64)
        n = self._lib.crane_sched_last_preempted(self._h, out.ctypes.data, len(out))
        return out[:n].tolist()

    def last_failed(self) -> List[int]:
        out = np.zeros(self.max_running + 1, dtype=np.int64)
        n = self._lib.crane_sched_last_failed(self._h, out.ctypes.data, len(out))
        return out[:n].tolist()
