#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Hunyuan-1.8B layer
sizes with random weights (bfloat16), printed as ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192]
                    [--layers L] [--impl reference]

A step is one decode step of the whole batch.  ``value`` is decoded tokens per
second with the K steps timed on the device (CUDA events); ``e2e`` is the same
through the Python entry point (``LLMEngine.step``: host token ids in, sampled
token ids out, every step).  The cache of every request is first filled to the
context length with random keys and values, so the step reads what a real
request of that length would read; inputs (weights and cache, far more than the
126 MB of L2) are larger than L2, so nothing is flushed between steps.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = {
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
    "vocab_size": 120818, "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 32,
    "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 128, "hidden_act": "silu",
    "max_position_embeddings": 32768, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": {"alpha": 1000.0, "type": "dynamic"}, "use_qk_norm": True,
    "tie_word_embeddings": True, "attention_bias": False,
}
# the other layer sizes of the baseline's configurations, for --sizes (the default run keeps 1.8B)
OTHER_SIZES = {
    "4b": {"hidden_size": 3072, "intermediate_size": 8192, "num_attention_heads": 32, "num_key_value_heads": 8},
    "7b": {"hidden_size": 4096, "intermediate_size": 14336, "num_attention_heads": 32, "num_key_value_heads": 8,
           "vocab_size": 128167, "tie_word_embeddings": False},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in d.items() if k in out and v})
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(float(r[0]))); mx = max(mx, int(float(r[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def param_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * i + 2 * h + 2 * cfg["head_dim"]
    head = v * h if cfg["tie_word_embeddings"] else 2 * v * h     # tied: the table is read once as the head
    return 2 * (layers * per_layer + head), 2 * layers * per_layer


def decode_bytes(cfg, layers, batch, context):
    weights, _ = param_bytes(cfg, layers)
    kv_per_token = 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    return weights + batch * context * kv_per_token


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * i
    gemm = 2 * tokens * layers * per_layer + 2 * v * h            # the head runs on the last row only
    attn = layers * 4 * q * tokens * tokens / 2                    # causal: half of QK^T and PV
    return gemm + attn


def build_model(cfg, engine_opts, seed=0, dtype="bf16"):
    """Random weights drawn and rounded to bfloat16; ``dtype`` "fp32" loads the
    same rounded values into the true 32-bit path."""
    import torch
    from crane_b200.generation import ModelForCausalLM
    from crane_b200.weights.random_init import model_manifest_for, random_tensors
    tensors = random_tensors(model_manifest_for(cfg), seed, torch.bfloat16, "cuda:0")
    return ModelForCausalLM.from_tensors(cfg, tensors, dtype, **engine_opts)


def fill_cache(model, batch, context, seed=1):
    """Admits `batch` requests and gives each `context` cached positions of
    random keys and values, without running a prefill."""
    import torch
    g = torch.Generator(device="cuda:0"); g.manual_seed(seed)
    for lc in model.runner.pools.layers:
        if lc.k is not None:
            lc.k.normal_(0.0, 1.0, generator=g)
            lc.v.normal_(0.0, 1.0, generator=g)
    ids = list(range(1000, 1000 + batch))
    for rid in ids:
        model.runner.table.admit(rid)
        model.runner.table.extend(rid, context)
    return ids


def check_decode_logits(model, cfg, ids, context, vocab, page):
    """One decode step of the live requests `ids` (cache filled to `context`) on
    the serving path against the same step on the engine's true 32-bit path (no
    tensor cores, plain kernels): same weights, same cached keys and values, same
    tokens.  Outside every timed region.  Returns the largest difference relative
    to the largest logit, and how many rows pick the same token."""
    import numpy as np
    import torch
    from crane_b200.engine import StepEntry
    batch = len(ids)
    ref = build_model(cfg, dict(page_size=page, num_pages=batch * (context // page + 2) + 8,
                                max_concurrent=max(batch, 1), max_seq_len=context + 1024,
                                max_batched_tokens=max(batch, 64), use_cuda_graphs=False), dtype="fp32")
    r16, r32 = model.runner, ref.runner
    blocks = (context + page - 1) // page
    for rid in ids:
        r32.table.admit(rid)
        r32.table.extend(rid, context)
    pages = {}                                    # per layer group: (pages here, pages there) of all requests
    for lc16, lc32 in zip(r16.pools.layers, r32.pools.layers):
        if lc16.k is None:
            continue
        if lc16.group not in pages:
            src = np.concatenate([r16.table.block_table(rid, lc16.group, blocks) for rid in ids])
            dst = np.concatenate([r32.table.block_table(rid, lc32.group, blocks) for rid in ids])
            pages[lc16.group] = (torch.from_numpy(src).to("cuda:0", torch.long),
                                 torch.from_numpy(dst).to("cuda:0", torch.long))
        src, dst = pages[lc16.group]
        lc32.k[dst] = lc16.k[src].float()
        lc32.v[dst] = lc16.v[src].float()
    toks = [(5 * i + 2) % vocab for i in range(batch)]
    entries = [StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]
    got = r16.step(entries).float().clone()
    want = r32.step(entries).float()
    r16.rt.check_errors()
    r32.rt.check_errors()
    err = float((got - want).abs().max() / want.abs().max())
    same = int((got.argmax(dim=1) == want.argmax(dim=1)).sum())
    del ref, r32, want
    torch.cuda.empty_cache()
    return err, same


def time_decode(model, ids, steps, warmup, vocab, mark=False):
    """K decode steps of the whole batch, timed on the device.  `mark`: the
    timed steps lie between cudaProfilerStart and cudaProfilerStop."""
    import torch
    from crane_b200.engine import StepEntry
    from crane_b200.sampling import SamplingParams
    runner, sampler = model.runner, model.engine.sampler
    greedy = [SamplingParams() for _ in ids]
    toks = [(7 * i + 3) % vocab for i in range(len(ids))]

    def one():
        logits = runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)])
        return sampler.sample_device(logits, greedy)
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    launches0 = runner.rt.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if mark:
        torch.cuda.profiler.start()
    start.record()
    for _ in range(steps):
        one()
    stop.record()
    torch.cuda.synchronize()
    if mark:
        torch.cuda.profiler.stop()
    runner.rt.check_errors()
    return start.elapsed_time(stop) / steps, (runner.rt.launches - launches0) // steps


def time_decode_e2e(model, batch, context, steps, warmup, vocab):
    """The same through the entry point: requests added with host token ids,
    every step plans on the host, copies its inputs from pinned memory and
    reads the sampled ids back."""
    import torch
    eng = model.engine
    runner = model.runner
    ids = []
    for b in range(batch):
        rid = eng.add_request([(11 * b + 5) % vocab], None, max_new_tokens=steps + warmup + 8,
                              eos_token_ids=[])
        ids.append(rid)
    eng.step()                                    # the one-token prompts
    for rid in ids:                               # then stretch every request to the context length
        runner.table.extend(rid, context - runner.table.length(rid))
    for _ in range(warmup):
        eng.step()
    eng.flush()                                   # nothing in flight when the clock starts
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 0
    for _ in range(steps):
        n += len(eng.step())
    n += len(eng.flush())                         # the last step's tokens are read inside the clock
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for rid in ids:
        eng.cancel(rid)
    eng.finished.clear()
    m = runner.meta
    return n / dt, m.total * 4, batch * 4


def time_prefill(model, tokens, vocab, reps=3, mark=False):
    """`mark`: the last repetition lies between cudaProfilerStart and cudaProfilerStop."""
    import torch
    from crane_b200.engine import StepEntry
    runner = model.runner
    prompt = [(13 * i + 1) % vocab for i in range(tokens)]
    times = []
    for r in range(reps + 1):
        rid = 5000 + r
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if mark and r == reps:
            torch.cuda.profiler.start()
        start.record()
        runner.step([StepEntry(rid, prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        if mark and r == reps:
            torch.cuda.profiler.stop()
        runner.end(rid)
        if r > 0:                                 # the first run warms up
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]                 # the median


def time_prefill_chunked(model, tokens, chunk, vocab, reps=2):
    """One prompt of `tokens` tokens in portions of `chunk`, one step each, as the
    scheduler cuts a long prompt under its token budget; the whole prompt timed."""
    import torch
    from crane_b200.engine import StepEntry
    runner = model.runner
    prompt = [(13 * i + 1) % vocab for i in range(tokens)]
    times = []
    for r in range(reps + 1):
        rid = 7000 + r
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for a in range(0, tokens, chunk):
            b = min(tokens, a + chunk)
            runner.step([StepEntry(rid, prompt[a:b], [b - a - 1] if b == tokens else [])])
        stop.record()
        torch.cuda.synchronize()
        runner.end(rid)
        if r > 0:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def serve_workload(model, cfg, args, pk):
    """The serving mix: `--requests` requests with seeded prompt lengths between
    `--prompt-min` and `--prompt-max` and `--new-tokens` generated tokens each, all
    added at once, through the engine's scheduler (continuous batching, prompt
    portions beside decoded tokens under the token budget).  Reports the running
    averages the reference's engine keeps (crane-serve/src/engine/stats.rs:41-54:
    prompt tokens over the time of steps that held prompt tokens, decoded tokens
    over the time of pure decode steps), the whole job's tokens per second, the
    steps' wall-time percentiles and the share of mixed steps."""
    import numpy as np
    import torch
    from crane_b200.sampling import SamplingParams
    eng = model.engine
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(args.seed)
    lengths = rng.integers(args.prompt_min, args.prompt_max + 1, args.requests)
    prompts = [rng.integers(0, vocab, int(n)).tolist() for n in lengths]
    # warm-up: a short mix that touches the step shapes' kernels
    for p in prompts[:4]:
        eng.add_request(p[:300], SamplingParams(temperature=0.7, seed=1), 8, [])
    eng.run_until_done()
    for k in eng.timers:
        eng.timers[k] = 0 if isinstance(eng.timers[k], int) else 0.0
    launches0 = model.runner.rt.launches
    for i, p in enumerate(prompts):
        eng.add_request(p, SamplingParams(temperature=0.7, seed=100 + i), args.new_tokens, [])
    kinds, times = [], []
    torch.cuda.synchronize()
    t_all = time.perf_counter()
    with ClockSampler() as clocks:
        while eng.has_work():
            t0 = time.perf_counter()
            eng.step()
            times.append(time.perf_counter() - t0)
            kinds.append(eng.last_step_kind)
        torch.cuda.synchronize()
    wall = time.perf_counter() - t_all
    model.runner.rt.check_errors()
    done = eng.finished
    generated = sum(len(o.generated) for o in done.values())
    prompt_tokens = int(lengths.sum())
    st = eng.stats()
    ms = np.asarray(times) * 1e3
    by_kind = {k: ms[[i for i, x in enumerate(kinds) if x == k]] for k in ("decode", "prefill", "mixed")}
    pct = lambda a: {"n": int(a.size), "p50": round(float(np.percentile(a, 50)), 3),
                     "p90": round(float(np.percentile(a, 90)), 3),
                     "p99": round(float(np.percentile(a, 99)), 3)} if a.size else {"n": 0}
    return {
        "workload": "serve", "requests": args.requests, "prompt_tokens": prompt_tokens,
        "prompt_len_min": int(lengths.min()), "prompt_len_max": int(lengths.max()),
        "generated_tokens": generated, "wall_s": round(wall, 3),
        "total_tokens_per_s": round((prompt_tokens + generated) / wall, 1),
        "generated_tokens_per_s": round(generated / wall, 1),
        "avg_prefill_tokens_per_sec": round(st["avg_prefill_tokens_per_sec"], 1),
        "avg_decode_tokens_per_sec": round(st["avg_decode_tokens_per_sec"], 1),
        "steps": len(times), "mixed_step_share": round(kinds.count("mixed") / max(1, len(kinds)), 3),
        "step_ms": {k: pct(v) for k, v in by_kind.items()},
        "preemptions": st.get("preemptions", 0), "gpu_launches": model.runner.rt.launches - launches0,
        "graph_replays": model.runner.graph_replays, "clocks": clocks.summary(),
    }


def mixed_step_workload(model, cfg, args):
    """What a step of `--batch` decoded tokens at `--context` beside one prompt
    portion of `--portion` tokens costs, against a pure decode step plus the
    portion alone, with the single tokens on the split-KV decode kernel (the
    engine's choice at such contexts) and with everything on the prefill kernel."""
    import torch
    from crane_b200.engine import StepEntry
    runner = model.runner
    vocab = cfg["vocab_size"]
    ids = fill_cache(model, args.batch, args.context)
    toks = [(7 * i + 3) % vocab for i in range(len(ids))]
    portion = [(13 * i + 1) % vocab for i in range(args.portion)]
    nxt = [9000]

    def timed(make_entries, reps, after=None):
        out = []
        for r in range(reps + 2):
            entries = make_entries()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.step(entries)
            b.record()
            torch.cuda.synchronize()
            if after:
                after(entries)
            if r >= 2:
                out.append(a.elapsed_time(b))
        out.sort()
        return out[len(out) // 2]

    def decode_entries():
        return [StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]

    def portion_entry():
        nxt[0] += 1
        return StepEntry(nxt[0], portion, [len(portion) - 1])

    def end_portion(entries):
        runner.end(entries[-1].request_id)
    reps = max(3, args.steps // 8)
    res = {"workload": "mixed-step", "batch": args.batch, "context": args.context, "portion": args.portion}
    res["decode_ms"] = round(timed(decode_entries, reps), 4)
    res["portion_ms"] = round(timed(lambda: [portion_entry()], reps, end_portion), 4)
    res["mixed_ms"] = round(timed(lambda: decode_entries() + [portion_entry()], reps, end_portion), 4)
    keep = runner.cfg.mixed_decode_min_keys
    runner.cfg.mixed_decode_min_keys = 1 << 60
    res["mixed_prefill_kernel_only_ms"] = round(timed(lambda: decode_entries() + [portion_entry()], reps, end_portion), 4)
    runner.cfg.mixed_decode_min_keys = keep
    res["mixed_over_sum"] = round(res["mixed_ms"] / (res["decode_ms"] + res["portion_ms"]), 3)
    runner.rt.check_errors()
    return res


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "cryptomilk/Crane is a Rust workspace on Candle; there is no cargo or rustc "
                      "in this image and no vendored crates, so it cannot be built or installed offline"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--impl", default="crane_b200")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    ap.add_argument("--only-prefill", action="store_true",
                    help="measure the 2,048-token prefill alone (for profiling); prints its record only")
    ap.add_argument("--prefill-tokens", type=int, default=2048,
                    help="with --only-prefill: another prompt length than the contract's 2,048 (one step)")
    ap.add_argument("--sizes", default="1.8b", choices=["1.8b", "4b", "7b"],
                    help="layer sizes: Hunyuan 1.8B (the default, the headline configuration), 4B or 7B")
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="with --only-prefill: also time the prompt in portions of this many tokens, a step each")
    ap.add_argument("--workload", default="", choices=["", "serve", "mixed-step"],
                    help="serve: a mix of requests through the scheduler; mixed-step: decoded tokens beside "
                         "one prompt portion in one step; each prints its own record only")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--portion", type=int, default=512)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-check", action="store_true",
                    help="skip the comparison of one decode step's logits with the 32-bit path")
    ap.add_argument("--only-decode", action="store_true",
                    help="measure the decode step alone (for profiling: the timed steps lie between "
                         "cudaProfilerStart and cudaProfilerStop); prints its record only")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    cfg = dict(MODEL)
    cfg.update(OTHER_SIZES.get(args.sizes, {}))
    full_layers = cfg["num_hidden_layers"]
    # a context beyond the configuration's limit: the same layer sizes with a longer position table
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], args.context + 2048,
                                         args.prefill_tokens + 2048)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers, vocab = cfg["num_hidden_layers"], cfg["vocab_size"]
    pk = peaks()
    page = 64
    need_tokens = 64 * (args.context + args.steps + args.warmup + 64) if not args.no_points else \
        args.batch * (args.context + args.steps + args.warmup + 64)
    need_tokens = max(need_tokens, args.batch * (args.context + args.steps + args.warmup + 64))
    opts = dict(page_size=page, num_pages=need_tokens // page + 64, max_concurrent=max(64, args.batch),
                max_seq_len=args.context + 1024, max_batched_tokens=2048, chunk_size=2048)
    if args.only_prefill:
        pt = args.prefill_tokens
        opts.update(num_pages=pt // page + 8, max_concurrent=4, max_seq_len=pt + 1024,
                    max_batched_tokens=max(2048, pt), chunk_size=max(2048, pt))
    if args.only_decode:
        opts.update(num_pages=args.batch * (args.context + args.steps + args.warmup + 64) // page + 64)
    if args.workload == "serve":
        per = args.prompt_max + args.new_tokens + page
        cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], per + 64)
        opts.update(num_pages=args.requests * per // page + 64, max_concurrent=args.requests,
                    max_seq_len=per, max_batched_tokens=2048, chunk_size=2048)
    if args.workload == "mixed-step":
        opts.update(num_pages=(args.batch * (args.context + 256) + 4 * args.portion) // page + 64,
                    max_concurrent=args.batch + 2, max_batched_tokens=max(2048, args.batch + args.portion))
    model = build_model(cfg, opts)
    runner = model.runner
    if args.workload == "serve":
        print(json.dumps(dict(serve_workload(model, cfg, args, pk), sizes=args.sizes, layers=layers)))
        return 0
    if args.workload == "mixed-step":
        print(json.dumps(dict(mixed_step_workload(model, cfg, args), sizes=args.sizes, layers=layers)))
        return 0
    if args.only_prefill:
        pms = time_prefill(model, pt, vocab, reps=max(1, args.steps), mark=True)
        flops = prefill_flops(cfg, layers, pt)
        rec = {"value": round(pt * 1000.0 / pms, 1), "tokens": pt, "ms": round(pms, 3), "layers": layers,
               "sizes": args.sizes, "tflops": round(flops / (pms * 1e-3) / 1e12, 1),
               "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        if args.prefill_chunk:
            cms = time_prefill_chunked(model, pt, args.prefill_chunk, vocab)
            rec["chunked"] = {"chunk": args.prefill_chunk, "value": round(pt * 1000.0 / cms, 1),
                              "ms": round(cms, 3),
                              "frac": round(flops / (cms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        print(json.dumps({"prefill": rec}))
        return 0

    def decode_point(batch):
        ids = fill_cache(model, batch, args.context)
        ms, launches = time_decode(model, ids, args.steps, args.warmup, vocab, mark=args.only_decode)
        for rid in ids:
            runner.end(rid)
        return ms, launches

    if args.only_decode:
        ms, launches = decode_point(args.batch)
        gbs = decode_bytes(cfg, layers, args.batch, args.context + args.warmup + args.steps // 2) / (ms * 1e-3) / 1e9
        print(json.dumps({"decode": {"value": round(args.batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
                                     "layers": layers, "sizes": args.sizes, "batch": args.batch,
                                     "context": args.context, "launches_per_step": launches,
                                     "gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}}))
        return 0

    check = None
    if not args.no_check:
        # the serving path's logits at the headline shape against the 32-bit path, before anything is timed
        ids = fill_cache(model, args.batch, args.context)
        err, same = check_decode_logits(model, cfg, ids, args.context, vocab, page)
        for rid in ids:
            runner.end(rid)
        check = {"against": "float32 path of the same engine, one decode step", "max_rel_err": round(err, 5),
                 "same_argmax": same, "rows": args.batch}
        # Rounding of the bfloat16 activations adds up over the layers: measured at this shape with 1,
        # 2, 4, 8, 16 and 32 layers, 0.0057, 0.0079, 0.0105, 0.0138, 0.0181 and 0.0316 of the largest
        # logit, that is 0.0057 * sqrt(layers).  Twice that is the bound; a key slice left out in one
        # layer moves the logits by several times as much.
        check["bound"] = round(1.2e-2 * layers ** 0.5, 5)
        if not err < check["bound"]:
            print(json.dumps({"error": "the serving path's logits differ from the 32-bit path's", "check": check}))
            return 1

    with ClockSampler() as clocks:
        ms, launches = decode_point(args.batch)
    clock = clocks.summary()
    value = args.batch * 1000.0 / ms
    bytes_step = decode_bytes(cfg, layers, args.batch, args.context + args.warmup + args.steps // 2)
    achieved = bytes_step / (ms * 1e-3) / 1e9
    e2e_value, h2d, d2h = time_decode_e2e(model, args.batch, args.context, args.steps, args.warmup, vocab)

    out = {
        "metric": "decode tokens/s (Hunyuan-%s sizes, batch %d, context %d)" % (args.sizes.upper(), args.batch, args.context),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": "Hunyuan-%s-sized, random weights" % args.sizes.upper(), "layers": layers,
                   "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
                   "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": vocab, "global_batch": args.batch, "seq_len": args.context,
                   "page_size": page, "parallelism": "none", "l2": "inputs larger than L2",
                   "cuda_graphs": bool(runner.graph_replays)},
        "clocks": clock,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "peaks": pk["source"]},
    }
    if check is not None:
        out["check"] = check
    if not args.no_points:
        # the prefill first: right after the batch-64 point the power cap holds the SM clock down
        # for a moment, which says nothing about the prefill
        tokens = 2048
        pms = time_prefill(model, tokens, vocab, reps=5)
        flops = prefill_flops(cfg, layers, tokens)
        out["prefill"] = {"value": round(tokens * 1000.0 / pms, 1), "tokens": tokens,
                          "ms": round(pms, 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        points = {}
        for b in (1, 64):
            pms, _ = decode_point(b)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
