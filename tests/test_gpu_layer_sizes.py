"""Replay at the layer sizes of Hunyuan 1.8B / 4B / 7B (one or two layers, small
vocabulary): the sizes at which the tcgen05 products, the tcgen05 prefill
attention and the split-KV decode attention are the kernels that run.  Whole
prompts, the last 32 tokens one by one, portions of changing size and mixed
batches in a pool with page reuse, in bfloat16 against the plain implementation;
the 1.8B sizes also in true 32-bit."""
import numpy as np
import pytest

import plain_hunyuan as ph
import tiny_configs
import trace_tools as tt

pytestmark = pytest.mark.gpu

LENGTHS = {"S18": [300, 33, 513, 129], "S4": [257, 40, 130], "S7": [200, 131, 66]}


@pytest.mark.parametrize("name,dtype", [("S18", "bfloat16"), ("S18", "float32"), ("S4", "bfloat16"),
                                        ("S7", "bfloat16")])
def test_replay_at_model_layer_sizes(name, dtype, model_folders, tmp_path):
    folder = model_folders(name, dtype)
    ps = tiny_configs.TINY[name]["page_size"]
    cfg, w = ph.load_folder(folder)
    rng = np.random.default_rng(40 + len(name))
    reqs = tt.make_requests(rng, cfg.vocab_size, LENGTHS[name])
    plain = {rid: ph.logits_all(cfg, w, toks) for rid, toks in reqs.items()}
    # alone: whole, tail decoded, portions
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs)
    tt.trace_portions(tb, reqs, np.random.default_rng(7))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "alone"))
    worst = tt.compare(got, tb, plain, dtype, f"{name} alone")
    runs = [(got, tb)]
    # mixed, pool so small that pages are used again
    tm = tt.TraceBuilder(ps)
    tt.trace_mixed(tm, reqs, np.random.default_rng(11))
    assert tm.pages_taken > tm.peak_tokens // ps
    got = tt.run_trace(folder, dtype, tm.steps, tm.peak_tokens, ps, str(tmp_path / "mixed"))
    worst = max(worst, tt.compare(got, tm, plain, dtype, f"{name} mixed"))
    runs.append((got, tm))
    if dtype == "bfloat16":
        # once more with every single token of a mixed step on the split-KV decode kernel
        got = tt.run_trace(folder, dtype, tm.steps, tm.peak_tokens, ps, str(tmp_path / "mixed_split"),
                           extra_args=["--mixed-decode-min-keys", "0"])
        worst = max(worst, tt.compare(got, tm, plain, dtype, f"{name} mixed, decode kernel"))
        runs.append((got, tm))
    tt.compare_cuts(runs, dtype, name)
    print(f"{name} {dtype}: worst relative error {worst:.3e}")
