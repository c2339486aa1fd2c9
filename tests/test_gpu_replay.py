"""Replay through bin/trace_run against the plain implementation: requests
whole, with the last 32 tokens decoded one by one, in portions of changing
size, and mixed with other requests in a pool so small that pages are used
again; in true 32-bit and in bfloat16."""
import numpy as np
import pytest

import plain_hunyuan as ph
import tiny_configs
import trace_tools as tt

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 17, 100, 65, 128, 33], "B": [5, 40, 97, 300, 129, 64, 210],
           "C": [3, 70, 255, 96, 31]}


def _plain(folder, reqs):
    cfg, w = ph.load_folder(folder)
    return {rid: ph.logits_all(cfg, w, toks) for rid, toks in reqs.items()}


@pytest.fixture(scope="module")
def cases(model_folders):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            folder = model_folders(name, dtype)
            rng = np.random.default_rng(100 + ord(name))
            vocab = tiny_configs.TINY[name]["config"]["vocab_size"]
            reqs = tt.make_requests(rng, vocab, LENGTHS[name])
            made[(name, dtype)] = (folder, reqs, _plain(folder, reqs))
        return made[(name, dtype)]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_alone_whole_tail_portions(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tiny_configs.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs)
    tt.trace_portions(tb, reqs, np.random.default_rng(7))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    worst = tt.compare(got, tb, plain, dtype, f"config {name}")
    tt.compare_cuts([(got, tb)], dtype, f"config {name}")
    print(f"config {name} {dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_with_page_reuse(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tiny_configs.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_mixed(tb, reqs, np.random.default_rng(11))
    pool_pages = tb.peak_tokens // ps
    assert tb.pages_taken > pool_pages, "the trace must make the pool hand pages out again"
    assert max(len(s["entries"]) for s in tb.steps) >= 3
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    worst = tt.compare(got, tb, plain, dtype, f"config {name} mixed")
    print(f"config {name} {dtype} mixed: worst relative error {worst:.3e}")


@pytest.mark.parametrize("name", ["B", "C"])
def test_mixed_with_the_decode_kernel_for_single_tokens(name, cases, tmp_path):
    """The same mixed traces with every single token of a mixed step sent to the
    split-KV decode kernel and the portions to the prefill kernel (the engine
    does this by itself once the single tokens read thousands of cached keys;
    here from the first key on)."""
    folder, reqs, plain = cases(name, "bfloat16")
    ps = tiny_configs.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_mixed(tb, reqs, np.random.default_rng(12))
    assert any(len(s["entries"]) >= 3 and min(len(e["tokens"]) for e in s["entries"]) == 1
               and max(len(e["tokens"]) for e in s["entries"]) > 1 for s in tb.steps)
    got = tt.run_trace(folder, "bfloat16", tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"),
                       extra_args=["--mixed-decode-min-keys", "0"])
    tt.compare(got, tb, plain, "bfloat16", f"config {name} mixed, decode kernel")
