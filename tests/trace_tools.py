"""Builds replay traces, runs bin/trace_run on them and compares what it wrote
with the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# the largest error of a row, relative to the largest |logit| of the compared rows
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
# and the root-mean-square error of a row relative to the root-mean-square of its logits: rounding
# spreads evenly over a row and stays far below the largest error's bound, while a fault of logic
# (a key tile left out, a slice dropped) moves the whole row
TOL_RMS = {"float32": 1e-5, "bfloat16": 2.5e-2}
worst_rms = {"float32": 0.0, "bfloat16": 0.0}        # the largest seen so far in this process, for reports


def run_trace(model_dir: str, dtype: str, steps: List[dict], max_tokens: int, page_size: int,
              out_dir: str, timeout: int = 600, extra_args: Sequence[str] = ()) -> Dict[int, np.ndarray]:
    os.makedirs(out_dir, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), "--page-size", str(page_size), *extra_args]
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], proc.stdout[-2000:]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n:
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n, -1)
        else:
            assert not os.path.exists(path)
    return out


def make_requests(rng: np.random.Generator, vocab: int, lengths: Sequence[int]) -> Dict[str, List[int]]:
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(lengths)}


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class TraceBuilder:
    """Collects steps and remembers, for every wanted row, which request and
    position it is."""

    def __init__(self, page_size: int, first_step: int = 0):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}
        self.progress: Dict[str, int] = {}
        self.live: Dict[str, int] = {}
        self.page_size = page_size
        self.peak_tokens = 0
        self.pages_taken = 0
        self.next_step = first_step

    def step(self, entries: List[Tuple[str, List[int], List[int]]], end: Sequence[str] = ()) -> int:
        """entries: (request id, tokens, wanted places among them)."""
        sid = self.next_step
        self.next_step += 1
        rows = []
        for rid, toks, want in entries:
            start = self.progress.get(rid, 0)
            before = round_up(self.live.get(rid, 0), self.page_size)
            self.progress[rid] = start + len(toks)
            self.live[rid] = start + len(toks)
            self.pages_taken += (round_up(self.live[rid], self.page_size) - before) // self.page_size
            rows.extend((rid, start + w) for w in want)
        held = sum(round_up(n, self.page_size) for n in self.live.values())
        self.peak_tokens = max(self.peak_tokens, held)
        self.steps.append({"step": sid, "entries": [{"id": r, "tokens": list(t), "want": list(w)}
                                                     for r, t, w in entries], "end": list(end)})
        if rows:
            self.rows[sid] = rows
        for rid in end:
            self.live.pop(rid, None)
        return sid

    def live_count(self) -> int:
        return len(self.live)


def trace_whole(tb: TraceBuilder, reqs: Dict[str, List[int]]) -> None:
    """Each request alone, in one step, every position wanted."""
    for rid, toks in reqs.items():
        tb.step([(rid, toks, list(range(len(toks))))], end=[rid])


def trace_tail_decode(tb: TraceBuilder, reqs: Dict[str, List[int]], tail: int = 32, suffix="t") -> None:
    """Most of a request in one step, its last `tail` tokens one by one."""
    for rid, toks in reqs.items():
        name = rid + suffix
        head = max(1, len(toks) - tail)
        cuts = [(0, head)] + [(i, i + 1) for i in range(head, len(toks))]
        for a, b in cuts:
            tb.step([(name, toks[a:b], [b - a - 1])], end=[name] if b == len(toks) else [])


def trace_portions(tb: TraceBuilder, reqs: Dict[str, List[int]], rng: np.random.Generator,
                   suffix="p") -> None:
    """Portions of changing size, down to two tokens; the last place of every
    portion and a random one are wanted."""
    sizes = [7, 2, 13, 2, 5, 31, 3, 2, 64, 9, 2, 17]
    for rid, toks in reqs.items():
        name = rid + suffix
        pos, k = 0, int(rng.integers(0, len(sizes)))
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            if len(toks) - pos - n == 1:          # never leave a single token as a "portion"
                n += 1
            k += 1
            want = sorted({n - 1, int(rng.integers(0, n))})
            end = [name] if pos + n == len(toks) else []
            tb.step([(name, toks[pos:pos + n], want)], end=end)
            pos += n


def trace_mixed(tb: TraceBuilder, reqs: Dict[str, List[int]], rng: np.random.Generator,
                max_live: int = 4, tail: int = 32, suffix="m") -> None:
    """Up to `max_live` requests at a time: portions of some beside single
    decoded tokens of others; a request may sit a step out."""
    waiting = [(rid + suffix, toks) for rid, toks in reqs.items()]
    live: Dict[str, List[int]] = {}
    done: Dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            name, toks = waiting.pop(0)
            live[name] = toks
            done[name] = 0
        entries, ended = [], []
        for name in list(live):
            toks, pos = live[name], done[name]
            if len(live) > 1 and rng.random() < 0.2:
                continue                           # left out of this step, goes on later
            left = len(toks) - pos
            if left <= tail:
                n, want = 1, [0]
            else:
                n = int(min(left - tail, rng.integers(2, 40)))
                if n < 2:
                    n = min(2, left)
                want = sorted({n - 1, int(rng.integers(0, n))})
            entries.append((name, toks[pos:pos + n], want))
            done[name] = pos + n
            if done[name] == len(toks):
                ended.append(name)
        if not entries:
            continue
        tb.step(entries, end=ended)
        for name in ended:
            del live[name]


def expected_rows(rows: List[Tuple[str, int]], plain: Dict[str, np.ndarray]) -> np.ndarray:
    return np.stack([plain[_base(r)][p] for r, p in rows])


# The same position computed under different cuttings and batchings (whole, decoded one by one, in
# portions, mixed with other requests) goes through the same weights and the same rounding places;
# only the kernels that the cutting selects differ (prefill or decode attention, tile shapes of the
# products).  So the engine agrees with ITSELF across cuttings far more closely than with the plain
# float64 logits in true 32-bit (measured: 4e-6 at most), where this is the sharpest check of the
# cache and the batch.  In bfloat16 the roundings of the activations differ between kernels as much
# as they differ from float64 (measured: up to 1.5e-2 in the worst row), so there the bound is the
# one of TOL_RMS; single wrong keys and tiles are caught by the kernels' own tests with planted keys.
# Root-mean-square difference of two rows relative to the root-mean-square of the logits.
TOL_CUTS = {"float32": 1e-5, "bfloat16": 2.5e-2}


def _base(name: str) -> str:
    return name.rstrip("tpm") if name[-1] in "tpm" else name


def compare_cuts(runs: Sequence[Tuple[Dict[int, np.ndarray], "TraceBuilder"]], dtype: str, label: str = "") -> float:
    """runs: (logits by step, the trace that asked for them) of one model.  Every
    (request, position) that was wanted more than once is compared with its
    first occurrence.  Returns the worst relative root-mean-square difference."""
    first: Dict[Tuple[str, int], Tuple[np.ndarray, str]] = {}
    worst, pairs = 0.0, 0
    for got, tb in runs:
        for sid in sorted(tb.rows):
            for i, (r, p) in enumerate(tb.rows[sid]):
                key, row = (_base(r), p), got[sid][i].astype(np.float64)
                if key not in first:
                    first[key] = (row, f"step {sid} as {r}")
                    continue
                ref, where = first[key]
                d = float(np.sqrt(((row - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean()))
                pairs += 1
                worst = max(worst, d)
                assert d <= TOL_CUTS[dtype], (
                    f"{label} {dtype}: request {key[0]} position {p} differs between {where} and step {sid} "
                    f"as {r}: relative rms difference {d:.3e} > {TOL_CUTS[dtype]:.1e}")
    print(f"{label} {dtype}: {pairs} positions computed more than once, worst difference between cuttings {worst:.3e}")
    return worst


def compare(got: Dict[int, np.ndarray], tb: TraceBuilder, plain: Dict[str, np.ndarray], dtype: str,
            label: str = "") -> float:
    """Asserts every wanted row against the plain logits; returns the worst
    relative error.  On failure names the first wrong (step, request, position)."""
    worst = 0.0
    call_rms = 0.0
    tol = TOL[dtype]
    for sid in sorted(tb.rows):
        rows = tb.rows[sid]
        want = expected_rows(rows, plain)
        have = got[sid]
        assert have.shape == want.shape, f"{label} step {sid}: shape {have.shape} vs {want.shape}"
        assert np.isfinite(have).all(), f"{label} step {sid}: non-finite logits"
        scale = np.abs(want).max()
        err = np.abs(have - want).max(axis=1) / scale
        bad = np.nonzero(err > tol)[0]
        if bad.size:
            r, p = rows[int(bad[0])]
            raise AssertionError(
                f"{label} {dtype}: first wrong logits at step {sid}, request {r}, position {p}: "
                f"relative error {err[bad[0]]:.3e} > {tol:.1e} "
                f"(page offset {p % tb.page_size}, page {p // tb.page_size})")
        worst = max(worst, float(err.max()))
        rms = np.sqrt(((have - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1))
        worst_rms[dtype] = max(worst_rms[dtype], float(rms.max()))
        call_rms = max(call_rms, float(rms.max()))
        bad = np.nonzero(rms > TOL_RMS[dtype])[0]
        if bad.size:
            r, p = rows[int(bad[0])]
            raise AssertionError(
                f"{label} {dtype}: root-mean-square error of the logits at step {sid}, request {r}, "
                f"position {p}: {rms[bad[0]]:.3e} > {TOL_RMS[dtype]:.1e}")
    print(f"{label} {dtype}: worst max error {worst:.3e}, worst rms error {call_rms:.3e}")
    return worst
