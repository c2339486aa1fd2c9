"""Replay at configurations drawn at random: head sizes that are no multiple of
16, odd numbers of heads and groups, widths and vocabularies that are no power
of two, with and without QK-norm, biases, a tied head, NTK-alpha and cross-layer
cache sharing; whole, tail decoded, in portions and mixed with page reuse, in
32-bit and in bfloat16, against the plain implementation.  NARROW is such a
draw that found a fault: 35 heads of 256 into a width of 320, where the output
projection of 798 tokens overran its buffer of partial sums."""
import numpy as np
import pytest

import plain_hunyuan as ph
import trace_tools as tt

pytestmark = pytest.mark.gpu


def draw(rng, big):
    """(config, page size, prompt lengths, weight scale).  The weights' scale falls with the width,
    as a trained model's does: a product then neither grows nor shrinks its input much, and the
    bounds measure rounding, not a draw's amplification of it (at a scale of 0.08 and a width of
    2,056 four layers amplify float32 rounding to 2e-5 and bfloat16 rounding to 5e-2)."""
    if big:      # sizes at which the tensor-core kernels run
        d = int(rng.choice([64, 128, 128, 256, 96]))
        hidden = int(rng.choice([256, 512, 1024, 1536, 320, 2048]))
        inter = int(rng.choice([512, 1024, 1536, 2816, 352]))
        layers, longest, std = int(rng.choice([1, 2])), 900, min(0.08, 0.9 / hidden ** 0.5)
    else:
        d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 160, 192, 208, 256, 6, 20, 40]))
        hidden = int(rng.choice([64, 72, 100, 136, 200, 264, 520, 1000, 50, 36]))
        inter = int(rng.choice([96, 100, 250, 352, 1000, 1336, 80, 24]))
        layers, longest, std = int(rng.choice([1, 2, 3, 4])), 330, min(0.08, 0.9 / hidden ** 0.5)
    nkv = int(rng.choice([1, 2, 3, 5]))
    cfg = {
        "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
        "vocab_size": int(rng.choice([257, 1001, 300, 64, 2049, 131])), "hidden_size": hidden,
        "intermediate_size": inter, "num_hidden_layers": layers,
        "num_attention_heads": nkv * int(rng.choice([1, 2, 3, 4, 7, 8])), "num_key_value_heads": nkv,
        "head_dim": d, "hidden_act": "silu", "max_position_embeddings": 2048,
        "rms_norm_eps": float(rng.choice([1e-5, 1e-6, 3e-4])), "rope_theta": float(rng.choice([10000.0, 1e6, 500.0])),
        "use_qk_norm": bool(rng.random() < 0.6), "tie_word_embeddings": bool(rng.random() < 0.5),
        "attention_bias": bool(rng.random() < 0.3),
    }
    if rng.random() < 0.5:
        cfg["rope_scaling"] = {"alpha": float(rng.choice([2.0, 1000.0, 7.5])), "type": "dynamic"}
    if rng.random() < 0.25 and layers >= 2:
        cfg["use_cla"], cfg["cla_share_factor"] = True, 2
    page_size = int(rng.choice([16, 32, 64, 128]))
    lengths = [int(x) for x in rng.integers(34, longest, size=int(rng.integers(2, 5)))]
    return cfg, page_size, lengths, std


NARROW = ({
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense", "vocab_size": 131,
    "hidden_size": 320, "intermediate_size": 1536, "num_hidden_layers": 1, "num_attention_heads": 35,
    "num_key_value_heads": 5, "head_dim": 256, "hidden_act": "silu", "max_position_embeddings": 2048,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "use_qk_norm": False, "tie_word_embeddings": False,
    "attention_bias": True}, 128, [798, 815, 71, 647], 0.03)


# (seed, sizes of the tensor-core kernels), or a configuration itself
@pytest.mark.parametrize("seed,big", [(1001, False), (1005, False), (2008, True), (3004, True), (7, NARROW)])
def test_replay_at_a_random_configuration(seed, big, tmp_path):
    from crane_b200.weights.random_init import write_model_folder
    cfg, ps, lengths, std = big if isinstance(big, tuple) else draw(np.random.default_rng(seed), big)
    for dtype in ("float32", "bfloat16"):
        folder = write_model_folder(str(tmp_path / dtype), cfg, seed, dtype, std=std, norm_std=0.05)
        c, w = ph.load_folder(folder)
        reqs = tt.make_requests(np.random.default_rng(seed + 1), c.vocab_size, lengths)
        plain = {rid: ph.logits_all(c, w, toks) for rid, toks in reqs.items()}
        tb = tt.TraceBuilder(ps)
        tt.trace_whole(tb, reqs)
        tt.trace_tail_decode(tb, reqs)
        tt.trace_portions(tb, reqs, np.random.default_rng(7))
        got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / (dtype + "_alone")))
        tt.compare(got, tb, plain, dtype, f"seed {seed} alone")
        tm = tt.TraceBuilder(ps)
        tt.trace_mixed(tm, reqs, np.random.default_rng(11))
        got2 = tt.run_trace(folder, dtype, tm.steps, tm.peak_tokens, ps, str(tmp_path / (dtype + "_mixed")))
        tt.compare(got2, tm, plain, dtype, f"seed {seed} mixed")
        tt.compare_cuts([(got, tb), (got2, tm)], dtype, f"seed {seed}")
