"""A toy architecture defined here, outside the package: one layer mixes with
a running sum kept in the request's state slot, the next with the package's
attention.  It is registered, built from tensors and stepped in portions
without touching the package's files."""
import numpy as np
import pytest
import torch

from gpu_helpers import DEV, rel_err

pytestmark = pytest.mark.gpu


def register_toy():
    from crane_b200.config import (LayerSpec, ModelSpec, PartSpec, ScheduleStep,
                                   register_architecture)
    from crane_b200.parts import CacheNeed, Part, register_part
    from crane_b200.weights import TensorSpec

    @register_part("mixer", "toy_running_sum")
    class RunningSum(Part):
        """out_t = W (decay * s_{t-1} + h_t), s kept per request between steps."""
        kind = "mixer"

        @classmethod
        def manifest(cls, spec):
            h = spec.params["hidden_size"]
            return {spec.prefix + "w": TensorSpec((h, h))}

        def load(self, weights, rt):
            self.w = weights[self.prefix + "w"]
            self.h = self.params["hidden_size"]
            self.decay = self.params["decay"]

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.h,), state_dtype=torch.float32)

        def forward(self, h, ctx, cache, rt):
            out = torch.empty_like(h)
            cu, kv = ctx.h_cu_q, ctx.h_kv_len
            for e in range(ctx.n_entries):
                a, b, slot = int(cu[e]), int(cu[e + 1]), int(ctx.h_slots[e])
                if int(kv[e]) - (b - a) == 0:
                    cache.state[slot].zero_()             # a fresh request in a used slot
                s = cache.state[slot]
                for t in range(a, b):
                    s = self.decay * s + h[t].float()
                    out[t] = (self.w.float() @ s).to(h.dtype)
                cache.state[slot].copy_(s)
            return out

    def build_spec(cfg):
        h = cfg["hidden_size"]
        norm = lambda p: PartSpec("norm", "rms_norm", {"size": h, "eps": cfg["eps"]}, p)
        ffn = lambda p: PartSpec("ffn", "swiglu", {"hidden_size": h, "intermediate_size": cfg["inter"]}, p)
        attn = PartSpec("mixer", "gqa_attention", {
            "hidden_size": h, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "bias": False,
            "qk_norm": False, "window": 0, "own_kv": True,
            "position": PartSpec("position", "rope", {"head_dim": 16, "theta": 1e4, "alpha": 0.0,
                                                      "max_positions": cfg["max_pos"]})}, "l1.attn.")
        toy = PartSpec("mixer", "toy_running_sum", {"hidden_size": h, "decay": cfg["decay"]}, "l0.mix.")
        layers = [LayerSpec("prenorm_residual", {"norm1": norm("l0.n1."), "mixer": toy,
                                                 "norm2": norm("l0.n2."), "ffn": ffn("l0.ffn.")}),
                  LayerSpec("prenorm_residual", {"norm1": norm("l1.n1."), "mixer": attn,
                                                 "norm2": norm("l1.n2."), "ffn": ffn("l1.ffn.")})]
        # the toy layer runs twice (same weights, a state of its own each time): the schedule is data
        return ModelSpec("ToyStateForCausalLM", h, cfg["vocab"], cfg["max_pos"],
                         PartSpec("embed", "token_embedding", {"vocab_size": cfg["vocab"], "hidden_size": h}, "emb."),
                         layers, [ScheduleStep(0), ScheduleStep(1), ScheduleStep(0)],
                         norm("final."), PartSpec("head", "lm_head", {"vocab_size": cfg["vocab"],
                                                                      "hidden_size": h, "tied_to": "emb.weight"}, "head."))

    register_architecture("ToyStateForCausalLM", lambda d: d, build_spec)


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from crane_b200.config import EngineConfig, resolve
    from crane_b200.engine import ModelRunner, StepEntry
    from crane_b200.parts import model_manifest
    from crane_b200.weights.random_init import random_tensors
    register_toy()
    cfg = {"architectures": ["ToyStateForCausalLM"], "hidden_size": 48, "inter": 64, "vocab": 90,
           "max_pos": 128, "eps": 1e-5, "decay": 0.7}
    spec = resolve(cfg).build_spec(cfg)
    tensors = random_tensors(model_manifest(spec), 3, torch.float32, std=0.1)
    assert "l0.mix.w" in tensors and "l1.attn.q_proj.weight" in tensors

    def runner():
        return ModelRunner(None, EngineConfig(dtype="float32", page_size=16, num_pages=8,
                                              max_concurrent=2, max_batched_tokens=64),
                           config=cfg, tensors=tensors)
    rng = np.random.default_rng(0)
    a, b = rng.integers(0, 90, 40).tolist(), rng.integers(0, 90, 23).tolist()
    r = runner()
    kinds = [n.kind for n in r.model.cache_needs()]
    assert kinds == ["state", "kv", "state"] and r.pools.layers[0].state.shape == (2, 48)
    assert r.pools.layers[2].state.data_ptr() != r.pools.layers[0].state.data_ptr()
    whole_a = r.step([StepEntry(1, a, list(range(40)))]).cpu()
    whole_b = r.step([StepEntry(2, b, list(range(23)))]).cpu()
    r.end(1); r.end(2)
    # the same two requests in portions, interleaved, in a fresh engine and in the used one
    for eng in (runner(), r):
        got_a, got_b = [], []
        got_a.append(eng.step([StepEntry(11, a[:7], list(range(7)))]).cpu())
        out = eng.step([StepEntry(11, a[7:30], list(range(23))), StepEntry(12, b[:2], [0, 1])]).cpu()
        got_a.append(out[:23]); got_b.append(out[23:])
        out = eng.step([StepEntry(12, b[2:], list(range(21))), StepEntry(11, a[30:31], [0])]).cpu()
        got_b.append(out[:21]); got_a.append(out[21:])
        got_a.append(eng.step([StepEntry(11, a[31:], list(range(9)))]).cpu())
        assert rel_err(torch.cat(got_a), whole_a) < 2e-5
        assert rel_err(torch.cat(got_b), whole_b) < 2e-5
        eng.end(11); eng.end(12)
        eng.table.check()
    # and the state really matters: without the decay the logits differ
    assert float((whole_a[5] - whole_a[4]).abs().max()) > 0
