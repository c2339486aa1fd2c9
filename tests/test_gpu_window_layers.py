"""A toy architecture defined here: layers of the package's attention that
alternate between all earlier positions and a sliding window.  The two kinds
form two layer groups with pages and block tables of their own, the windowed
group gives pages back as the window passes them, and the logits still match a
plain whole-sequence computation however the tokens are cut."""
import numpy as np
import pytest
import torch

import plain_hunyuan as ph
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu

CFG = {"architectures": ["ToyWindowForCausalLM"], "hidden": 64, "inter": 96, "vocab": 120, "layers": 4,
       "heads": 4, "kv_heads": 2, "head_dim": 16, "window": 24, "max_pos": 512, "eps": 1e-5, "theta": 1e4}


def register():
    from crane_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleStep, register_architecture

    def build_spec(c):
        h = c["hidden"]
        norm = lambda p: PartSpec("norm", "rms_norm", {"size": h, "eps": c["eps"]}, p)
        pos = PartSpec("position", "rope", {"head_dim": c["head_dim"], "theta": c["theta"], "alpha": 0.0,
                                            "max_positions": c["max_pos"]})
        layers = []
        for i in range(c["layers"]):
            p = f"model.layers.{i}."
            attn = PartSpec("mixer", "gqa_attention", {
                "hidden_size": h, "num_heads": c["heads"], "num_kv_heads": c["kv_heads"],
                "head_dim": c["head_dim"], "bias": False, "qk_norm": False, "own_kv": True,
                "window": c["window"] if i % 2 else 0, "position": pos}, p + "self_attn.")
            layers.append(LayerSpec("prenorm_residual", {
                "norm1": norm(p + "input_layernorm."), "mixer": attn,
                "norm2": norm(p + "post_attention_layernorm."),
                "ffn": PartSpec("ffn", "swiglu", {"hidden_size": h, "intermediate_size": c["inter"]}, p + "mlp.")}))
        return ModelSpec("ToyWindowForCausalLM", h, c["vocab"], c["max_pos"],
                         PartSpec("embed", "token_embedding", {"vocab_size": c["vocab"], "hidden_size": h},
                                  "model.embed_tokens."),
                         layers, [ScheduleStep(i) for i in range(c["layers"])], norm("model.norm."),
                         PartSpec("head", "lm_head", {"vocab_size": c["vocab"], "hidden_size": h,
                                                      "tied_to": "model.embed_tokens.weight"}, "lm_head."))
    register_architecture("ToyWindowForCausalLM", lambda d: d, build_spec)


def plain_logits(w, tokens):
    """Whole sequence, no cache, windows on the odd layers, from the plain parts."""
    c = CFG
    cfg = ph.PlainConfig(vocab_size=c["vocab"], hidden_size=c["hidden"], intermediate_size=c["inter"],
                         num_hidden_layers=c["layers"], num_attention_heads=c["heads"],
                         num_key_value_heads=c["kv_heads"], head_dim=c["head_dim"],
                         max_position_embeddings=c["max_pos"], rms_norm_eps=c["eps"], rope_theta=c["theta"],
                         rope_alpha=0.0, attention_bias=False, use_qk_norm=False, tie_word_embeddings=True,
                         use_cla=False, cla_share_factor=1)
    pos = np.arange(len(tokens))
    x = ph.embed(tokens, w["model.embed_tokens.weight"])
    for i in range(c["layers"]):
        p = f"model.layers.{i}."
        h = ph.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        a, _ = ph.attention_layer(h, cfg, w, p + "self_attn.", pos, window=c["window"] if i % 2 else 0)
        x = x + a
        h = ph.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        x = x + ph.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                          w[p + "mlp.down_proj.weight"])
    return ph.linear(ph.rms_norm(x, w["model.norm.weight"], c["eps"]), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_full_and_windowed_layers_in_groups_of_their_own(dtype, tol):
    from crane_b200.config import EngineConfig, resolve
    from crane_b200.engine import ModelRunner, StepEntry
    from crane_b200.parts import model_manifest
    from crane_b200.weights.random_init import random_tensors
    register()
    spec = resolve(CFG).build_spec(CFG)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = random_tensors(model_manifest(spec), 9, store, std=0.08, norm_std=0.05)
    w = {k: v.double().numpy() for k, v in tensors.items()}
    r = ModelRunner(None, EngineConfig(dtype=dtype, page_size=8, num_pages=40, max_concurrent=3,
                                       max_batched_tokens=128), config=CFG, tensors=tensors)
    assert r.num_groups == 2 and [g.window for g in r.pools.groups] == [0, 24]
    rng = np.random.default_rng(2)
    a, b = rng.integers(0, 120, 150).tolist(), rng.integers(0, 120, 90).tolist()
    want_a, want_b = plain_logits(w, a), plain_logits(w, b)

    def check(got, want, rows):
        got = got.cpu().numpy()
        assert np.abs(got - want[rows]).max() / np.abs(want).max() < tol

    # request a in portions that straddle the window, with request b mixed in, then decoding
    check(r.step([StepEntry(1, a[:50], [0, 23, 24, 25, 49])]), want_a, [0, 23, 24, 25, 49])
    out = r.step([StepEntry(1, a[50:53], [2]), StepEntry(2, b[:40], [39])])
    check(out[:1], want_a, [52]); check(out[1:], want_b, [39])
    out = r.step([StepEntry(2, b[40:], [49]), StepEntry(1, a[53:120], [0, 66])])
    check(out[:1], want_b, [89]); check(out[1:], want_a, [53, 119])
    r.end(2)
    for i in range(120, 150):
        check(r.step([StepEntry(1, [a[i]], [0])]), want_a, [i])
    # the windowed group holds only the pages its window needs, the other group every page
    full_blocks = (150 + 7) // 8
    assert r.table.total_pages(0) - r.table.free_pages(0) == full_blocks
    assert r.table.total_pages(1) - r.table.free_pages(1) <= (24 + 8) // 8 + 1
    bt = r.table.block_table(1, 1, 64)
    assert bt[0] == -1 and bt[full_blocks - 1] >= 0
    r.end(1)
    r.table.check()
    r.rt.check_errors()
    assert r.table.free_pages(0) == 40 and r.table.free_pages(1) == 40
