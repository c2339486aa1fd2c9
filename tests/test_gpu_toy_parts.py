"""Toy parts defined here, outside the package: a feed-forward that routes
every token to one of several small experts, and a position encoding with a
frequency law of its own.  One layer uses both, the next layer the package's
own parts; the model is registered, built from random tensors and stepped in
portions without a change to the package's files."""
import numpy as np
import pytest
import torch

from gpu_helpers import DEV, rel_err

pytestmark = pytest.mark.gpu


def register_toys():
    from crane_b200.config import (LayerSpec, ModelSpec, PartSpec, ScheduleStep,
                                   register_architecture)
    from crane_b200.parts import Part, register_part
    from crane_b200.weights import TensorSpec

    @register_part("ffn", "toy_routed")
    class Routed(Part):
        """y = scale * gelu(h W1[e]^T) W2[e]^T with e = argmax of the float router logits."""
        kind = "ffn"
        capturable = False          # it reads its routing on the host: no CUDA graph can hold that

        @classmethod
        def manifest(cls, spec):
            h, i, e = (spec.params[k] for k in ("hidden_size", "expert_size", "experts"))
            p = spec.prefix
            return {p + "router": TensorSpec((e, h), "float32"), p + "w1": TensorSpec((e, i, h)),
                    p + "w2": TensorSpec((e, h, i))}

        def load(self, weights, rt):
            p = self.prefix
            self.router, self.w1, self.w2 = weights[p + "router"], weights[p + "w1"], weights[p + "w2"]
            self.scale = float(self.params["scale"])

        def forward(self, h, ctx, rt):
            logits = h.float() @ self.router.t()                  # router logits in 32-bit
            pick = logits.argmax(dim=-1)
            top = logits.topk(2, dim=-1).values
            Routed.last_margin = float(((top[:, 0] - top[:, 1]) / logits.abs().max(dim=-1).values).min())
            out = torch.zeros_like(h)
            for e in range(self.router.shape[0]):
                rows = (pick == e).nonzero().flatten()
                if rows.numel():
                    a = torch.nn.functional.gelu(h[rows].float() @ self.w1[e].float().t())
                    out[rows] = (self.scale * (a @ self.w2[e].float().t())).to(h.dtype)
            return out

    @register_part("position", "toy_harmonic")
    class Harmonic(Part):
        """Rotation angle of pair j at position p: p * base / (j + 1)."""
        kind = "position"

        def load(self, weights, rt):
            self._tables = None

        def tables(self, rt, n):
            if self._tables is None or self._tables[0].shape[0] < n:
                half = self.params["head_dim"] // 2
                freq = self.params["base"] / torch.arange(1, half + 1, dtype=torch.float64)
                ang = torch.arange(n, dtype=torch.float64)[:, None] * freq[None, :]
                self._tables = (ang.cos().float().to(rt.device), ang.sin().float().to(rt.device))
            return self._tables

    def build_spec(cfg):
        h, d = cfg["hidden_size"], cfg["head_dim"]
        norm = lambda p: PartSpec("norm", "rms_norm", {"size": h, "eps": cfg["eps"]}, p)
        def attn(prefix, position):
            return PartSpec("mixer", "gqa_attention", {
                "hidden_size": h, "num_heads": 3, "num_kv_heads": 1, "head_dim": d, "bias": False,
                "qk_norm": True, "qk_norm_eps": cfg["eps"], "window": 0, "own_kv": True,
                "position": position}, prefix)
        harmonic = PartSpec("position", "toy_harmonic", {"head_dim": d, "base": cfg["base"]}, "")
        rope = PartSpec("position", "rope", {"head_dim": d, "theta": 1e4, "alpha": 0.0,
                                             "max_positions": cfg["max_pos"]}, "")
        routed = PartSpec("ffn", "toy_routed", {"hidden_size": h, "expert_size": cfg["expert_size"],
                                                "experts": cfg["experts"], "scale": cfg["scale"]}, "l0.moe.")
        dense = PartSpec("ffn", "swiglu", {"hidden_size": h, "intermediate_size": cfg["inter"]}, "l1.ffn.")
        layers = [LayerSpec("prenorm_residual", {"norm1": norm("l0.n1."), "mixer": attn("l0.attn.", harmonic),
                                                 "norm2": norm("l0.n2."), "ffn": routed}),
                  LayerSpec("prenorm_residual", {"norm1": norm("l1.n1."), "mixer": attn("l1.attn.", rope),
                                                 "norm2": norm("l1.n2."), "ffn": dense})]
        return ModelSpec("ToyRoutedForCausalLM", h, cfg["vocab"], cfg["max_pos"],
                         PartSpec("embed", "token_embedding", {"vocab_size": cfg["vocab"], "hidden_size": h}, "emb."),
                         layers, [ScheduleStep(0), ScheduleStep(1)], norm("final."),
                         PartSpec("head", "lm_head", {"vocab_size": cfg["vocab"], "hidden_size": h,
                                                      "tied_to": None}, "head."))

    register_architecture("ToyRoutedForCausalLM", lambda d: d, build_spec)
    return Routed, Harmonic


CFG = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 40, "head_dim": 16, "inter": 56,
       "expert_size": 24, "experts": 3, "scale": 0.5, "vocab": 75, "max_pos": 96, "eps": 1e-5, "base": 0.37}


def build(dtype, tensors=None):
    from crane_b200.config import EngineConfig, resolve
    from crane_b200.engine import ModelRunner
    from crane_b200.parts import model_manifest
    from crane_b200.weights.random_init import random_tensors
    spec = resolve(CFG).build_spec(CFG)
    if tensors is None:
        tensors = random_tensors(model_manifest(spec), 7, torch.float32, std=0.2)
    return tensors, ModelRunner(None, EngineConfig(dtype=dtype, page_size=16, num_pages=8, max_concurrent=2,
                                                   max_batched_tokens=64), config=CFG, tensors=tensors)


def test_toy_feed_forward_and_position_are_built_and_stepped():
    register_toys()
    tensors, r = build("float32")
    assert {"l0.moe.router", "l0.moe.w1", "l0.moe.w2", "l1.ffn.down_proj.weight", "head.weight"} <= set(tensors)
    assert tensors["l0.moe.router"].dtype == torch.float32
    rng = np.random.default_rng(1)
    a, b = rng.integers(0, 75, 37).tolist(), rng.integers(0, 75, 19).tolist()
    whole_a = r.step([StepEntry(1, a, list(range(37)))]).cpu()
    whole_b = r.step([StepEntry(2, b, list(range(19)))]).cpu()
    r.end(1); r.end(2)
    got_a, got_b = [], []
    got_a.append(r.step([StepEntry(11, a[:5], list(range(5)))]).cpu())
    out = r.step([StepEntry(11, a[5:20], list(range(15))), StepEntry(12, b[:2], [0, 1])]).cpu()
    got_a.append(out[:15]); got_b.append(out[15:])
    out = r.step([StepEntry(12, b[2:], list(range(17))), StepEntry(11, a[20:21], [0])]).cpu()
    got_b.append(out[:17]); got_a.append(out[17:])
    got_a.append(r.step([StepEntry(11, a[21:], list(range(16)))]).cpu())
    assert rel_err(torch.cat(got_a), whole_a) < 2e-5
    assert rel_err(torch.cat(got_b), whole_b) < 2e-5
    r.end(11); r.end(12)
    r.table.check()
    # the position encoding is the toy's, not the package's: another base, other logits
    other = dict(CFG, base=0.11)
    from crane_b200.config import EngineConfig
    from crane_b200.engine import ModelRunner
    r2 = ModelRunner(None, EngineConfig(dtype="float32", page_size=16, num_pages=8, max_concurrent=2,
                                        max_batched_tokens=64), config=other, tensors=tensors)
    moved = r2.step([StepEntry(1, a, list(range(37)))]).cpu()
    assert rel_err(moved[0], whole_a[0]) < 2e-5                   # position 0 is not rotated
    assert rel_err(moved[20:], whole_a[20:]) > 1e-3


def test_toy_model_in_bfloat16_follows_the_float_one():
    Routed, _ = register_toys()
    tensors, r32 = build("float32")
    _, r16 = build("bfloat16", tensors)
    # a prompt in which no routing decision hangs on bfloat16 rounding: every token's best two
    # router logits are at least a tenth of the largest apart
    for seed in range(40):
        tokens = np.random.default_rng(seed).integers(0, 75, 30).tolist()
        want = r32.step([StepEntry(seed + 1, tokens, list(range(30)))]).cpu()
        r32.end(seed + 1)
        if Routed.last_margin > 0.1:
            break
    else:
        pytest.fail("no prompt with wide routing margins among 40")
    got = r16.step([StepEntry(1, tokens, list(range(30)))]).cpu()
    assert rel_err(got, want) < 3e-2
    # The toy feed-forward reads its routing on the host and says so (capturable = False): steps of
    # the same shape, which the engine would otherwise capture and replay, are launched kernel by
    # kernel every time and give the same bits.
    r16.end(1)
    again = r16.step([StepEntry(2, tokens, list(range(30)))]).cpu()
    assert torch.equal(again, got)
    r16.end(2)
    third = r16.step([StepEntry(3, tokens, list(range(30)))]).cpu()
    assert torch.equal(third, got) and r16.graph_replays == 0
    r16.rt.check_errors()


def test_toy_routed_feed_forward_alone():
    """The part alone against its formula, every expert taken by some token."""
    from crane_b200.config import PartSpec
    from crane_b200.parts import Runtime, build_part
    Routed, _ = register_toys()
    torch.manual_seed(0)
    h, i, e = 40, 24, 3
    w = {"f.router": torch.randn(e, h, device=DEV), "f.w1": torch.randn(e, i, h, device=DEV) * 0.2,
         "f.w2": torch.randn(e, h, i, device=DEV) * 0.2}
    part = build_part(PartSpec("ffn", "toy_routed", {"hidden_size": h, "expert_size": i, "experts": e,
                                                     "scale": 2.0}, "f."))
    rt = Runtime(DEV, torch.float32, 64)
    part.load(w, rt)
    x = torch.randn(50, h, device=DEV)
    got = part.forward(x, None, rt)
    pick = (x @ w["f.router"].t()).argmax(-1)
    assert set(pick.tolist()) == {0, 1, 2}
    want = torch.stack([2.0 * torch.nn.functional.gelu(x[t] @ w["f.w1"][pick[t]].t()) @ w["f.w2"][pick[t]].t()
                        for t in range(50)])
    assert rel_err(got, want) < 1e-5


from crane_b200.engine import StepEntry  # noqa: E402  (after the marks, as the other GPU tests do)
