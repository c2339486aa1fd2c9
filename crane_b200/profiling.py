"""Runs one kernel of the engine alone, at a given size, and reports its time
against the roofline: the command that profiles are taken with.

    python -m crane_b200.profiling gemm --m 2048 --n 12288 --k 2048 [--silu-mul]
    python -m crane_b200.profiling gemm --m 8 --n 12288 --k 2048          (few tokens: swap-AB, slices)
    python -m crane_b200.profiling decode-attention --batch 8 --context 8192
    python -m crane_b200.profiling prefill-attention --tokens 2048
    python -m crane_b200.profiling rmsnorm --rows 2048 --hidden 2048

Times are CUDA-event times over --reps launches after --warmup; operands are
re-used between launches, so keep them larger than the 126 MB L2 where the
figure is to mean DRAM traffic (--sets N rotates through N copies of the
weights).  Peaks come from MEASURED_PEAKS.json beside the package's parent
folder if present, else 6650 GB/s and 1590 TFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from .kernels import Partials, get_kernels

DEV = "cuda:0"
BF = torch.bfloat16


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        out.update({k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops") if d.get(k)})
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


GRAPH = True


def _time(fn, warmup, reps):
    """Seconds per launch.  The launches are captured in a CUDA graph and
    replayed (as the engine's decode steps are), so short kernels are not timed
    at the host's launch rate; --no-graph launches them one by one."""
    for _ in range(max(1, warmup)):
        fn()
    torch.cuda.synchronize()
    run = lambda: [fn() for _ in range(reps)]
    if GRAPH:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        run = g.replay
        run()
        torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    run()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e-3 / reps


def _report(name, seconds, nbytes, flops, extra=None):
    pk = _peaks()
    rec = {"kernel": name, "us": round(seconds * 1e6, 2),
           "GB/s": round(nbytes / seconds / 1e9, 1), "frac_hbm": round(nbytes / seconds / 1e9 / pk["hbm_gbs"], 4),
           "TFLOP/s": round(flops / seconds / 1e12, 1),
           "frac_bf16": round(flops / seconds / 1e12 / pk["bf16_tflops"], 4), "peaks": pk["source"]}
    rec.update(extra or {})
    print(json.dumps(rec))


def gemm(a):
    K = get_kernels()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.randn(a.m, a.k, device=DEV).to(BF)
    ws = [(torch.randn(a.n, a.k, device=DEV) / a.k ** 0.5).to(BF) for _ in range(a.sets)]
    state = {"i": 0}
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if a.m <= 64 or a.swap:
        bn = a.bn or (16 if a.m <= 16 else 32 if a.m <= 32 else 64 if a.m <= 64 else 128 if a.m <= 128 else 256)
        slices = a.slices or K.slices_for((a.n + 127) // 128, a.k, sms)
        out = torch.empty(slices, a.m, a.n, device=DEV) if slices > 1 else torch.empty(a.m, a.n, device=DEV, dtype=BF)

        def fn():
            w = ws[state["i"] % a.sets]; state["i"] += 1
            K.gemm_tcgen05(x, w, None, out, err, split_k=slices, swap=True, bn=bn)
        extra = {"mode": "swap-AB", "bn": bn, "slices": slices}
    elif a.slices > 1:
        bn = a.bn or 128
        out = torch.empty(a.slices, a.m, a.n, device=DEV)

        def fn():
            w = ws[state["i"] % a.sets]; state["i"] += 1
            K.gemm_tcgen05(x, w, None, out, err, split_k=a.slices, bn=bn)
        extra = {"mode": "tiles in slices", "bn": bn, "slices": a.slices}
    else:
        bn = a.bn or (256 if a.n >= 2048 else 128)
        cols = a.n // 2 if a.silu_mul else a.n
        out = torch.empty(a.m, cols, device=DEV, dtype=BF)

        def fn():
            w = ws[state["i"] % a.sets]; state["i"] += 1
            if a.pair:
                K.gemm_pair(x, w, None, out, err, bn=bn, silu_mul=a.silu_mul, tile_rows=512 if a.tall else 256)
            else:
                K.gemm_tcgen05(x, w, None, out, err, bn=bn, silu_mul=a.silu_mul, tile_rows=256 if a.tall else 128)
        extra = {"mode": "pairs of SMs" if a.pair else "persistent", "bn": bn, "silu_mul": a.silu_mul,
                 "tile_rows": (256 if a.tall else 128) * (2 if a.pair else 1)}
    t = _time(fn, a.warmup, a.reps)
    assert int(err.item()) == 0
    nbytes = 2 * (a.m * a.k + a.n * a.k) + out.numel() * out.element_size()
    _report(f"gemm {a.m}x{a.n}x{a.k}", t, nbytes, 2.0 * a.m * a.n * a.k, extra)


def decode_attention(a):
    K = get_kernels()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    nq, nkv, d, ps, B, T = a.q_heads, a.kv_heads, a.head_dim, a.page_size, a.batch, a.context
    mb = T // ps + 1
    pages = B * mb
    kp = torch.randn(pages, nkv, ps, d, device=DEV).to(BF)
    vp = torch.randn(pages, nkv, ps, d, device=DEV).to(BF)
    table = torch.randperm(pages, device=DEV).to(torch.int32).view(B, mb)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    kvl = torch.full((B,), T, dtype=torch.int32, device=DEV)
    cols = (nq + 2 * nkv) * d
    qkv = torch.randn(B, cols, device=DEV).to(BF)
    cos = torch.randn(T + 8, d // 2, device=DEV); sin = torch.randn(T + 8, d // 2, device=DEV)
    w = torch.ones(d, device=DEV)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    splits = a.splits or K.decode_splits(B, nkv, sms)       # what the attention part chooses
    o = torch.empty(B, nq * d, device=DEV, dtype=BF)
    po = torch.empty(B * nq * splits * d, device=DEV); pml = torch.empty(B * nq * splits * 2, device=DEV)

    def fn():
        K.paged_decode_attention_fused(qkv, cols, True, cos, sin, w, w, 1e-5, o, kp, vp, cu, kvl, table, ps,
                                       nq, nkv, d, 0, d ** -0.5, splits, po, pml, err)
    t = _time(fn, a.warmup, a.reps)
    assert int(err.item()) == 0
    nbytes = B * T * nkv * d * 2 * 2
    _report(f"decode attention B{B} T{T}", t, nbytes, 4.0 * B * T * nq * d, {"splits": splits})


def prefill_attention(a):
    K = get_kernels()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    nq, nkv, d, ps, T = a.q_heads, a.kv_heads, a.head_dim, a.page_size, a.tokens
    mb = T // ps + 1
    kp = torch.randn(mb, nkv, ps, d, device=DEV).to(BF); vp = torch.randn(mb, nkv, ps, d, device=DEV).to(BF)
    table = torch.arange(mb, dtype=torch.int32, device=DEV).view(1, mb)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    kvl = torch.tensor([T], dtype=torch.int32, device=DEV)
    q = torch.randn(T, nq * d, device=DEV).to(BF); o = torch.empty_like(q)

    tc = a.kernel != "mma" and K.prefill_attention_tc_supports(d, nq, nkv, ps)

    def fn():
        if tc:
            K.prefill_attention_tc(q, o, kp, vp, cu, kvl, table, ps, (T + 127) // 128, nq, nkv, d, 0, d ** -0.5, err)
        else:
            K.paged_prefill_attention(q, o, kp, vp, cu, kvl, table, ps, (T + 63) // 64, nq, nkv, d, 0,
                                      d ** -0.5, err)
    t = _time(fn, a.warmup, a.reps)
    assert int(err.item()) == 0
    _report(f"prefill attention T{T}", t, 2 * (2 * T * nq * d + 2 * T * nkv * d), 4.0 * nq * d * T * T / 2,
            {"kernel_kind": "tcgen05" if tc else "mma.sync"})


def rmsnorm(a):
    K = get_kernels()
    # --sets copies in turn, so that a launch finds none of its rows in L2 (48 MB per copy at 2048 x 2048)
    xs = [torch.randn(a.rows, a.hidden, device=DEV) for _ in range(a.sets)]
    deltas = [torch.randn(a.rows, a.hidden, device=DEV).to(BF) for _ in range(a.sets)]
    outs = [torch.empty(a.rows, a.hidden, device=DEV, dtype=BF) for _ in range(a.sets)]
    w = torch.ones(a.hidden, device=DEV)
    state = {"i": 0}

    def fn():
        i = state["i"] % a.sets; state["i"] += 1
        K.add_rmsnorm(xs[i], deltas[i], w, 1e-5, outs[i])
    t = _time(fn, a.warmup, a.reps)
    _report(f"add_rmsnorm {a.rows}x{a.hidden}", t, a.rows * a.hidden * (4 + 2 + 4 + 2), 0.0, {"sets": a.sets})


def hardware(a):
    """What one thread can issue and what a barrier across the SMs costs."""
    from ctypes import c_int, c_void_p
    from .csrc import build
    lib = build.load_microbench()
    lib.crane_microbench_mma_issue.argtypes = [c_int, c_int, c_void_p, c_void_p]
    lib.crane_microbench_mma_issue.restype = c_int
    lib.crane_microbench_grid_barrier.argtypes = [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.crane_microbench_grid_barrier.restype = c_int
    st = torch.cuda.current_stream(DEV).cuda_stream
    out = torch.zeros(3, dtype=torch.int64, device=DEV)
    reps = 500
    for n in (64, 128, 256):
        for _ in range(2):                                   # the second run is reported
            rc = lib.crane_microbench_mma_issue(n, reps, out.data_ptr(), st)
            assert rc == 0, rc
            torch.cuda.synchronize()
        issue, done, ok = out.tolist()
        print(json.dumps({"measurement": f"tcgen05.mma 128x{n}x16 issued back to back by one thread",
                          "products": 4 * reps, "cycles_per_product_issue_loop": round(issue / (4 * reps), 1),
                          "cycles_per_product_until_complete": round(done / (4 * reps), 1),
                          "tensor_core_cycles_per_product": n // 2, "completed": bool(ok)}))
    sms = torch.cuda.get_device_properties(DEV).multi_processor_count
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    cycles = torch.zeros(1, dtype=torch.int64, device=DEV)
    rounds = 1000
    for ctas in (sms, sms // 2, 32):
        for _ in range(2):
            counter.zero_(); err.zero_()
            rc = lib.crane_microbench_grid_barrier(ctas, rounds, counter.data_ptr(), cycles.data_ptr(), err.data_ptr(), st)
            assert rc == 0, rc
            torch.cuda.synchronize()
        print(json.dumps({"measurement": "barrier across the SMs (release-add, acquire-loads)", "ctas": ctas,
                          "rounds": rounds, "cycles_per_barrier": round(int(cycles.item()) / rounds),
                          "wait_ran_out": bool(int(err.item()))}))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--no-graph", action="store_true", help="launch one by one instead of replaying a graph")
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, required=True); g.add_argument("--n", type=int, required=True)
    g.add_argument("--k", type=int, required=True); g.add_argument("--bn", type=int, default=0)
    g.add_argument("--slices", type=int, default=0); g.add_argument("--sets", type=int, default=1)
    g.add_argument("--silu-mul", action="store_true")
    g.add_argument("--swap", action="store_true", help="weights on the 128-row side also for more than 64 tokens")
    g.add_argument("--pair", action="store_true", help="many tokens: the kernel in which two SMs share a tile")
    g.add_argument("--tall", action="store_true", help="many tokens: tiles of 256 rows on one SM (bn 128, 192, 256), of 512 rows with --pair (bn 192, 224, 256)")
    for name in ("decode-attention", "prefill-attention"):
        p = sub.add_parser(name)
        p.add_argument("--q-heads", type=int, default=16); p.add_argument("--kv-heads", type=int, default=4)
        p.add_argument("--head-dim", type=int, default=128); p.add_argument("--page-size", type=int, default=64)
        p.add_argument("--batch", type=int, default=8); p.add_argument("--context", type=int, default=8192)
        p.add_argument("--tokens", type=int, default=2048); p.add_argument("--splits", type=int, default=0)
        p.add_argument("--kernel", default="auto", choices=["auto", "mma"])
    sub.add_parser("hardware", help="issue rate of tcgen05.mma from one thread; cost of a barrier across the SMs")
    r = sub.add_parser("rmsnorm")
    r.add_argument("--rows", type=int, default=2048); r.add_argument("--hidden", type=int, default=2048)
    r.add_argument("--sets", type=int, default=1)
    a = ap.parse_args(argv)
    global GRAPH
    GRAPH = not a.no_graph
    {"gemm": gemm, "decode-attention": decode_attention, "prefill-attention": prefill_attention,
     "rmsnorm": rmsnorm, "hardware": hardware}[a.what](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
