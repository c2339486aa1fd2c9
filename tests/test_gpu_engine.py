"""The engine above the step function: greedy generation through the Python
entry point against the plain implementation, batches through the scheduler,
preemption, long decoding, the first tokens of a sequence, streamers, sampling
with a seed, and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_hunyuan as ph
import tiny_configs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load(folder, dtype, **opts):
    from crane_b200.generation import ModelForCausalLM
    return ModelForCausalLM.from_pretrained(folder, dtype, **opts)


def greedy_cfg(n, **kw):
    from crane_b200.generation import GenerationConfig
    return GenerationConfig(max_new_tokens=n, temperature=None, **kw)


def assert_greedy_consistent(pc, pw, tokens, prompt_len, rel_tol):
    """Every generated token is the plain argmax of its prefix, up to `rel_tol`
    of the logit scale (bfloat16 may pick another of two near-equal logits)."""
    logits = ph.logits_all(pc, pw, tokens[:-1])
    for i in range(prompt_len, len(tokens)):
        row = logits[i - 1]
        assert row[tokens[i]] >= row.max() - rel_tol * np.abs(row).max(), (i, tokens[i], int(row.argmax()))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_float32_equals_plain(name, model_folders):
    folder = model_folders(name, "float32")
    pc, pw = ph.load_folder(folder)
    m = load(folder, "fp32", page_size=tiny_configs.TINY[name]["page_size"], num_pages=32,
             max_concurrent=4, max_batched_tokens=64)
    rng = np.random.default_rng(3)
    for n in (1, 5, 17):
        prompt = rng.integers(0, pc.vocab_size, n).tolist()
        got = m.generate(prompt, greedy_cfg(8, eos_token_id=-1))
        assert got == ph.greedy_generate(pc, pw, prompt, 8)
    m.runner.table.check()
    assert m.runner.table.live() == 0


@pytest.mark.parametrize("name", ["A", "B", "D80", "D192", "D144"])
def test_greedy_generation_bfloat16(name, model_folders):
    folder = model_folders(name, "bfloat16")
    pc, pw = ph.load_folder(folder)
    m = load(folder, "bf16", page_size=tiny_configs.TINY[name]["page_size"] if name.startswith("D") else 16,
             num_pages=32, max_concurrent=4, max_batched_tokens=64)
    prompt = np.random.default_rng(4).integers(0, pc.vocab_size, 12).tolist()
    got = m.generate(prompt, greedy_cfg(12, eos_token_id=-1))
    assert len(got) == 24 and got[:12] == prompt
    assert_greedy_consistent(pc, pw, got, 12, 3e-2)


def test_eos_streamer_and_return_value(model_folders):
    """EOS ends generation, stays in the returned list, is not streamed; the
    streamer is finalized exactly once (hunyuan_dense/model.rs:341-370)."""
    from crane_b200.generation import ListStreamer
    folder = model_folders("B", "float32")
    pc, pw = ph.load_folder(folder)
    m = load(folder, "fp32", page_size=16, num_pages=32, max_concurrent=2, max_batched_tokens=64)
    prompt = [3, 1, 4, 1, 5]
    free_run = ph.greedy_generate(pc, pw, prompt, 10)
    eos = free_run[7]
    first = free_run.index(eos, 5)
    s = ListStreamer()
    got = m.generate(prompt, greedy_cfg(10, eos_token_id=eos), s)
    assert got == free_run[:first + 1] and s.tokens == free_run[5:first] and s.finalized
    s2 = ListStreamer()
    assert m.generate(prompt, greedy_cfg(3, eos_token_id=-1), s2) == free_run[:8]
    assert s2.tokens == free_run[5:8] and s2.finalized


def test_batch_through_the_scheduler_equals_one_by_one(model_folders):
    folder = model_folders("B", "float32")
    pc, pw = ph.load_folder(folder)
    m = load(folder, "fp32", page_size=16, num_pages=64, max_concurrent=4, max_batched_tokens=48,
             chunk_size=32)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, pc.vocab_size, n).tolist() for n in (5, 40, 97, 2, 61, 33)]
    outs = m.generate_batch(prompts, greedy_cfg(9, eos_token_id=-1))
    for p, o in zip(prompts, outs):
        assert o == ph.greedy_generate(pc, pw, p, 9)
    st = m.stats()
    assert st["finished"] == 6 and st["preemptions"] == 0 and st["kernel_launches"] > 0
    m.runner.table.check()
    assert m.runner.table.free_pages() == 64


def test_preemption_recomputes_and_output_is_unchanged(model_folders):
    folder = model_folders("B", "float32")
    pc, pw = ph.load_folder(folder)
    # 10 pages of 16 tokens: three requests of ~40 tokens + 30 new cannot all stay
    m = load(folder, "fp32", page_size=16, num_pages=10, max_concurrent=3, max_batched_tokens=64,
             chunk_size=32)
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, pc.vocab_size, n).tolist() for n in (40, 38, 35)]
    outs = m.generate_batch(prompts, greedy_cfg(30, eos_token_id=-1))
    assert m.stats()["preemptions"] > 0
    for p, o in zip(prompts, outs):
        assert len(o) == len(p) + 30
        assert_greedy_consistent(pc, pw, o, len(p), 1e-4)
    m.runner.table.check()
    assert m.runner.table.free_pages() == 10


@pytest.mark.parametrize("dtype,tol", [("fp32", 1e-4), ("bf16", 3e-2)])
def test_long_decoding(dtype, tol, model_folders):
    folder = model_folders("B", "float32" if dtype == "fp32" else "bfloat16")
    pc, pw = ph.load_folder(folder)
    m = load(folder, dtype, page_size=16, num_pages=40, max_concurrent=2, max_batched_tokens=64)
    got = m.generate([7, 8, 9], greedy_cfg(400, eos_token_id=-1))
    assert len(got) == 403
    assert_greedy_consistent(pc, pw, got, 3, tol)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_first_tokens_of_a_sequence(dtype, tol, model_folders):
    """Positions 0, 1, 2 one token at a time: a sequence's first token has
    nothing before it."""
    from crane_b200.config import EngineConfig
    from crane_b200.engine import ModelRunner, StepEntry
    folder = model_folders("A", dtype)
    pc, pw = ph.load_folder(folder)
    r = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, num_pages=4, max_concurrent=2,
                                         max_batched_tokens=16))
    toks = [200, 3, 77]
    want = ph.logits_all(pc, pw, toks)
    for i, t in enumerate(toks):
        got = r.step([StepEntry(1, [t], [0])]).cpu().numpy()[0]
        assert np.abs(got - want[i]).max() / np.abs(want[i]).max() < tol
    r.end(1)
    r.rt.check_errors()


def test_sampling_with_a_seed_is_reproducible(model_folders):
    from crane_b200.generation import GenerationConfig
    folder = model_folders("B", "float32")
    m = load(folder, "fp32", page_size=16, num_pages=32, max_concurrent=3, max_batched_tokens=128)
    prompts = [[1, 2, 3, 4, 5], list(range(40)), list(range(97))]      # the workload of tiny config B
    cfg = GenerationConfig(max_new_tokens=12, temperature=0.8, eos_token_id=-1, seed=1)
    a = m.generate_batch(prompts, cfg)
    b = m.generate_batch(prompts, cfg)
    assert a == b
    c = m.generate_batch(prompts, GenerationConfig(max_new_tokens=12, temperature=0.8, eos_token_id=-1, seed=2))
    assert a != c
    rep = m.generate(prompts[0], GenerationConfig(max_new_tokens=12, temperature=0.8, top_p=0.9, top_k=20,
                                                  repetition_penalty=1.3, repeat_last_n=8,
                                                  eos_token_id=-1, seed=1))
    assert len(rep) == 17


@pytest.mark.parametrize("opts", [dict(temperature=0.8, top_k=12), dict(temperature=1.2, top_p=0.85),
                                  dict(temperature=0.9, top_k=20, top_p=0.9, repetition_penalty=1.3, repeat_last_n=8),
                                  dict(temperature=None, repetition_penalty=1.7, repeat_last_n=5)])
def test_sampling_options_through_the_engine_follow_the_plain_rules(opts, model_folders):
    """Every token that ``generate`` returns is the one the plain rules pick from
    the plain logits of its prefix: the repetition penalty over the last
    ``repeat_last_n`` tokens of prompt ++ generated, the top-k / top-p set, and
    the request's own random stream keyed by seed and the count of tokens it has
    sampled before."""
    from crane_b200.generation import GenerationConfig
    folder = model_folders("B", "float32")
    pc, pw = ph.load_folder(folder)
    m = load(folder, "fp32", page_size=16, num_pages=32, max_concurrent=3, max_batched_tokens=128)
    prompt = [7, 7, 7, 300, 12, 5, 7, 19, 300, 2, 44]
    n_new, seed = 14, 77
    got = m.generate(prompt, GenerationConfig(max_new_tokens=n_new, eos_token_id=-1, seed=seed, **opts))
    assert got[:len(prompt)] == prompt and len(got) == len(prompt) + n_new
    logits = ph.logits_all(pc, pw, got[:-1])
    temp = opts.get("temperature")
    for i in range(len(prompt), len(got)):
        row = logits[i - 1]
        pen = opts.get("repetition_penalty", 1.0)
        if pen != 1.0:
            row = ph.apply_repetition_penalty(row, pen, got[max(0, i - opts["repeat_last_n"]):i])
        if temp is None:
            assert row[got[i]] >= row.max() - 1e-4 * np.abs(row).max(), (i, got[i], int(row.argmax()))
            continue
        top_p = opts.get("top_p", 1.0)
        top_k = opts.get("top_k", 0) or (64 if top_p < 1.0 else 0)       # top-p works inside the best 64
        keep = ph.top_k_top_p_keep(row, temp, top_k, top_p)
        assert got[i] in set(int(j) for j in keep), (i, got[i], keep[:8])
        score = ph.gumbel_scores(row, temp, ph.uniform_noise(seed, i - len(prompt), pc.vocab_size))
        assert score[got[i]] >= score[keep].max() - 1e-3, (i, got[i], int(keep[np.argmax(score[keep])]))


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_overlapped_steps_change_no_token(dtype, model_folders):
    """The engine that launches a step before it has read the last one's tokens
    gives the tokens of the engine that waits: with EOS tokens that stop
    requests early, temperature sampling, and a pool so small that requests
    are preempted and recomputed."""
    from crane_b200.generation import GenerationConfig
    folder = model_folders("B", "float32" if dtype == "fp32" else "bfloat16")
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, 300, n).tolist() for n in (40, 38, 35, 3, 17)]
    runs = {}
    for overlap in (False, True):
        m = load(folder, dtype, page_size=16, num_pages=12, max_concurrent=3, max_batched_tokens=64,
                 chunk_size=32, async_scheduling=overlap)
        free = m.generate_batch(prompts, greedy_cfg(30, eos_token_id=-1))
        eos = free[0][len(prompts[0]) + 11]              # stops the first request after 12 tokens
        runs[overlap] = (free,
                         m.generate_batch(prompts, greedy_cfg(30, eos_token_id=eos)),
                         m.generate_batch(prompts, GenerationConfig(max_new_tokens=20, temperature=0.9,
                                                                    top_k=30, eos_token_id=eos, seed=5)),
                         m.generate(prompts[3], greedy_cfg(1, eos_token_id=-1)))
        assert m.stats()["preemptions"] > 0
        assert len(runs[overlap][1][0]) <= len(prompts[0]) + 12
        m.runner.table.check()
        assert m.runner.table.free_pages() == 12
        assert not m.engine.has_work()
    assert runs[False] == runs[True]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_overlapped_steps_on_a_lagging_device_change_no_token(dtype, model_folders):
    """The same comparison while the device is far behind the host, as it is at
    real model sizes: every forward pass of the model is preceded on the stream
    by tens of milliseconds of ordinary finite work (large products), so that a
    step's sampler runs long after the host has planned and launched the step
    after it.  Rows carry their own temperature, top-k, top-p and seed; requests end
    at different times and one is added late, so the rows of the batch shift.
    Whatever the host stages for a step's sampler must still be that step's
    when the device gets to it."""
    from crane_b200.engine import LLMEngine, ModelRunner
    from crane_b200.config import EngineConfig
    from crane_b200.sampling import SamplingParams
    folder = model_folders("B", "float32" if dtype == "fp32" else "bfloat16")
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, 300, n).tolist() for n in (9, 14, 3, 11, 6)]
    options = [(dict(temperature=0.7, seed=11), 5), (dict(temperature=None), 14),
               (dict(temperature=1.3, top_k=20, seed=12), 9), (dict(temperature=0.9, top_p=0.8, seed=13), 14),
               (dict(temperature=1.1, seed=14), 8)]
    a = torch.randn(4096, 4096, device="cuda:0")
    w = torch.randn(4096, 4096, device="cuda:0")
    c = torch.empty(4096, 4096, device="cuda:0")
    runs = {}
    for overlap in (False, True):
        runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, num_pages=32, max_concurrent=4,
                                                  max_batched_tokens=64, chunk_size=32,
                                                  async_scheduling=overlap))
        eng = LLMEngine(runner)
        forward = runner.model.forward

        def slow_forward(ctx, layers, forward=forward, runner=runner):
            for _ in range(3):                               # behind the step's metadata, before its sampler
                runner.rt.kernels.gemm_simt(a, w, None, c)
            return forward(ctx, layers)
        runner.model.forward = slow_forward
        ids = [eng.add_request(p, SamplingParams(**o), n, [-1]) for p, (o, n) in zip(prompts[:4], options[:4])]
        steps = behind = 0
        while eng.has_work():
            if steps == 6:
                ids.append(eng.add_request(prompts[4], SamplingParams(**options[4][0]), options[4][1], [-1]))
            eng.step()
            steps += 1
            if eng._inflight is not None and not eng._inflight.event.query():
                behind += 1
        runner.rt.check_errors()
        runs[overlap] = [eng.finished[i].tokens for i in ids]
        if overlap:
            assert behind >= steps // 2, (behind, steps)      # the device did lag behind the host
        runner.table.check()
    assert runs[False] == runs[True]
    for toks, p, (o, n) in zip(runs[True], prompts, options):
        assert len(toks) == len(p) + n


@pytest.mark.parametrize("name", ["B", "C", "S18", "D144"])
def test_small_steps_replay_graphs_with_the_same_logits(name, model_folders):
    """Steps with prompt portions of up to graph_max_tokens tokens are padded to
    a multiple of 64 rows and, from the second step of a shape on, replay a
    captured graph: prompts of different lengths under one shape, then a
    portion beside decoded tokens, then decoding, give the logits of an engine
    that launches every step kernel by kernel; the padding rows write nothing
    into the cache (the decoded tokens that follow read it).  Every step here
    finds the device idle (its results are read each time): only then does a
    step take a graph."""
    from crane_b200.engine import StepEntry
    folder = model_folders(name, "bfloat16")
    rng = np.random.default_rng(3)
    vocab = tiny_configs.TINY[name]["config"]["vocab_size"]
    prompts = [rng.integers(0, vocab, n).tolist() for n in (70, 100, 128, 65, 90, 101)]
    runs = {}
    for graphs in (0, 1024):
        m = load(folder, "bf16", page_size=tiny_configs.TINY[name]["page_size"], num_pages=64,
                 max_concurrent=16, max_batched_tokens=256, chunk_size=256, graph_max_tokens=graphs)
        r = m.runner
        out = []
        for i, p in enumerate(prompts):                         # one shape: 128 rows, 1 entry, 2 wanted
            out.append(r.step([StepEntry(i, p, [0, len(p) - 1])]).float().cpu())
        for i in (20, 21, 22):                                  # portions of which nothing is wanted
            p = rng.integers(0, vocab, 150).tolist()
            assert r.step([StepEntry(i, p[:100], [])]).shape[0] == 0
            torch.cuda.synchronize()                            # a graph is taken only while the device idles
            out.append(r.step([StepEntry(i, p[100:], [49])]).float().cpu())
            r.end(i)
        for t, n_single in enumerate((4, 3, 2, 4)):             # single tokens beside a portion of 30:
            fresh = rng.integers(0, vocab, 30).tolist()         # 5, 4, 3, 5 entries fill shapes of 8, 4, 4, 8
            entries = [StepEntry(i, [int(rng.integers(0, vocab))], [0]) for i in range(n_single)]
            entries.append(StepEntry(10 + t, fresh, [29]))
            out.append(r.step(entries).float().cpu())
            assert out[-1].shape[0] == n_single + 1
        for t in range(3):                                      # all ten decode (the decode graphs)
            ids = list(range(4)) + [4, 5] + [10, 11, 12, 13]
            out.append(r.step([StepEntry(i, [int(rng.integers(0, vocab))], [0]) for i in ids]).float().cpu())
        r.rt.check_errors()
        runs[graphs] = (out, r.graph_replays + r.graph_captures)     # steps that took the graph path
        for i in list(range(6)) + [10, 11, 12, 13]:
            r.end(i)
        r.table.check()
        rng = np.random.default_rng(3)
        prompts = [rng.integers(0, vocab, n).tolist() for n in (70, 100, 128, 65, 90, 101)]
    assert runs[0][1] == 3                                      # only the decode steps
    assert runs[1024][1] == 3 + 5 + 2 + 4                       # prompts 2..6, mixed steps 3 and 4, 4 portions
    for a, b in zip(runs[0][0], runs[1024][0]):
        assert a.shape == b.shape
        assert (a - b).abs().max() <= 2e-3 * a.abs().max()


def test_decode_steps_under_a_limit_that_is_no_power_of_two(model_folders):
    """Six requests at most: decode steps of five or six entries are padded to six
    (not to eight, which the step's buffers could not hold, and not left to the
    path of mixed steps, which once took them: rotary kernel, decode kernel and
    prefill kernel over padding rows instead of the one fused kernel)."""
    from crane_b200.engine import StepEntry
    folder = model_folders("S18", "bfloat16")
    vocab = tiny_configs.TINY["S18"]["config"]["vocab_size"]
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, vocab, n).tolist() for n in (40, 70, 33, 90, 65, 50)]
    outs = {}
    for limit in (6, 8):
        m = load(folder, "bf16", page_size=64, num_pages=32, max_concurrent=limit, max_batched_tokens=512)
        r = m.runner
        assert [r._bucket(n) for n in (1, 2, 3, 4, 5, 6)] == [1, 2, 4, 4, min(8, limit), min(8, limit)]
        for i, p in enumerate(prompts):
            r.step([StepEntry(i, p, [])])
        got, per_step = [], []
        for t in range(3):
            toks = [int(rng.integers(0, vocab)) for _ in range(5)]
            before = r.rt.launches
            got.append(r.step([StepEntry(i, [toks[i]], [0]) for i in range(5)]).float().cpu())
            per_step.append(r.rt.launches - before)
        r.rt.check_errors()
        outs[limit] = (got, per_step[-1])
        rng = np.random.default_rng(8)
        prompts = [rng.integers(0, vocab, n).tolist() for n in (40, 70, 33, 90, 65, 50)]
    # the decode step's kernels under either limit: per layer norm, q/k/v, fused attention (8 key slices
    # at these short contexts, which merge in their cluster), output, norm, gate/up, silu, down;
    # embedding, final norm, head in slices and their sum
    layers = tiny_configs.TINY["S18"]["config"]["num_hidden_layers"]
    assert outs[6][1] == outs[8][1] == 8 * layers + 4, (outs[6][1], outs[8][1])
    for a, b in zip(outs[6][0], outs[8][0]):
        assert (a - b).abs().max() <= 2e-3 * a.abs().max()


def test_refusals(model_folders):
    folder = model_folders("A", "float32")
    m = load(folder, "fp32", page_size=16, num_pages=16, max_concurrent=2, max_batched_tokens=64)
    with pytest.raises(ValueError, match="refused"):
        m.generate(list(range(129)), greedy_cfg(1))            # longer than max_position_embeddings
    with pytest.raises(ValueError, match="token id"):
        m.generate([1, 999], greedy_cfg(1))
    assert m.generate([1, 2], greedy_cfg(200, eos_token_id=-1))[:2] == [1, 2]   # clamped to the limit
    assert m.runner.table.live() == 0


def test_command_line(model_folders):
    folder = model_folders("A", "float32")
    pc, pw = ph.load_folder(folder)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "crane"), "-m", folder, "--dtype", "fp32",
           "--prompt-ids", "5,6,7", "--max-new-tokens", "6", "--eos-token-id", "-1", "--page-size", "16",
           "--num-pages", "8", "-c", "2", "--max-batched-tokens", "32"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    want = ph.greedy_generate(pc, pw, [5, 6, 7], 6)[3:]
    assert p.stdout.strip().splitlines()[-1] == ",".join(map(str, want))
    # random weights from the folder's config.json alone
    p = subprocess.run(cmd + ["--random-weights", "--seed", "3"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    assert len(p.stdout.strip().splitlines()[-1].split(",")) == 6
