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


def register_device_toy():
    """The same running sum written so that a recorded graph can replay it: it
    reads the step's metadata on the device only, leaves padding rows (entry -1)
    alone and touches no slot for an entry without rows."""
    from crane_b200.config import (LayerSpec, ModelSpec, PartSpec, ScheduleStep, register_architecture)
    from crane_b200.parts import CacheNeed, Part, register_part
    from crane_b200.weights import TensorSpec

    @register_part("mixer", "toy_running_sum_on_device")
    class RunningSumOnDevice(Part):
        kind = "mixer"
        state_graph_safe = True

        @classmethod
        def manifest(cls, spec):
            h = spec.params["hidden_size"]
            return {spec.prefix + "w": TensorSpec((h, h))}

        def load(self, weights, rt):
            self.w = weights[self.prefix + "w"]
            self.h = self.params["hidden_size"]
            self.decay = float(self.params["decay"])

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.h,), state_dtype=torch.float32)

        def forward(self, h, ctx, cache, rt):
            n, dev = h.shape[0], h.device
            ent = ctx.tok_entry.long()                         # -1: a row that pads the step
            live = ent >= 0
            e_safe = ent.clamp_min(0)
            cu = ctx.cu_q.long()
            q_len = cu[1:] - cu[:-1]
            valid = q_len > 0                                  # False: an entry that pads the step
            slots = ctx.slots.long()
            fresh = (ctx.kv_len.long() - q_len) == 0           # the request's first tokens: state starts at 0
            prev = cache.state[slots] * (valid & ~fresh)[:, None]
            idx = torch.arange(n, device=dev)
            gap = idx[:, None] - idx[None, :]
            same = (ent[:, None] == ent[None, :]) & live[:, None] & live[None, :] & (gap >= 0)
            weights = torch.where(same, torch.pow(self.decay, gap.clamp_min(0).float()), 0.0)
            first = idx - cu[e_safe]
            # (rows that pad the step hold whatever the buffers held: they must not reach a sum, not even times 0)
            hf = torch.where(live[:, None], h.float(), 0.0)
            s = weights @ hf + (torch.pow(self.decay, (first + 1).float()) * live)[:, None] * prev[e_safe]
            out = (s @ self.w.float().T).to(h.dtype)
            s_last = s[(cu[1:] - 1).clamp_min(0)]              # the state behind each entry's last row
            n_slots = cache.state.shape[0]
            onehot = ((slots[:, None] == torch.arange(n_slots, device=dev)[None, :]) & valid[:, None]).float()
            hit = onehot.sum(0) > 0
            cache.state.copy_(torch.where(hit[:, None], onehot.T @ s_last, cache.state))
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
        toy = PartSpec("mixer", "toy_running_sum_on_device", {"hidden_size": h, "decay": cfg["decay"]}, "l0.mix.")
        layers = [LayerSpec("prenorm_residual", {"norm1": norm("l0.n1."), "mixer": toy,
                                                 "norm2": norm("l0.n2."), "ffn": ffn("l0.ffn.")}),
                  LayerSpec("prenorm_residual", {"norm1": norm("l1.n1."), "mixer": attn,
                                                 "norm2": norm("l1.n2."), "ffn": ffn("l1.ffn.")})]
        return ModelSpec("ToyDeviceStateForCausalLM", h, cfg["vocab"], cfg["max_pos"],
                         PartSpec("embed", "token_embedding", {"vocab_size": cfg["vocab"], "hidden_size": h}, "emb."),
                         layers, [ScheduleStep(0), ScheduleStep(1), ScheduleStep(0)],
                         norm("final."), PartSpec("head", "lm_head", {"vocab_size": cfg["vocab"],
                                                                      "hidden_size": h, "tied_to": "emb.weight"}, "head."))

    register_architecture("ToyDeviceStateForCausalLM", lambda d: d, build_spec)


def test_a_mixer_with_state_replays_graphs_when_it_bears_padding():
    """A model with a stateful mixer that says ``state_graph_safe`` replays graphs
    on the bfloat16 path: its steps of single tokens are padded with rows of no
    entry and entries without rows (never with copies of an entry), and give
    what the engine without graphs gives; states of requests that sit a step out
    or share a step with padding entries stay as they were."""
    from crane_b200.config import EngineConfig, resolve
    from crane_b200.engine import ModelRunner, StepEntry
    from crane_b200.parts import model_manifest
    from crane_b200.weights.random_init import random_tensors
    register_device_toy()
    cfg = {"architectures": ["ToyDeviceStateForCausalLM"], "hidden_size": 48, "inter": 64, "vocab": 90,
           "max_pos": 256, "eps": 1e-5, "decay": 0.7}
    spec = resolve(cfg).build_spec(cfg)
    tensors = random_tensors(model_manifest(spec), 3, torch.bfloat16, std=0.1)
    rng = np.random.default_rng(1)
    reqs = {i: rng.integers(0, 90, n).tolist() for i, n in ((1, 40), (2, 23), (3, 31))}
    runs = {}
    for graphs in (False, True):
        r = ModelRunner(None, EngineConfig(dtype="bfloat16", page_size=16, num_pages=16, max_concurrent=4,
                                           max_batched_tokens=64, use_cuda_graphs=graphs),
                        config=cfg, tensors=tensors)
        assert r._graphs_ok == graphs
        out = []
        # prompts in portions, then single tokens: three requests, then two (one sits steps out), then three
        out.append(r.step([StepEntry(1, reqs[1][:20], [19]), StepEntry(2, reqs[2][:9], [8])]).float().cpu())
        out.append(r.step([StepEntry(3, reqs[3][:12], [11]), StepEntry(1, reqs[1][20:30], [9])]).float().cpu())
        pos = {1: 30, 2: 9, 3: 12}
        for live in ([1, 2, 3], [1, 2, 3], [1, 2, 3], [1, 3], [1, 3], [1, 3], [2], [1, 2, 3], [1, 2, 3]):
            torch.cuda.synchronize()                      # an idle device: a step of a seen shape replays its graph
            out.append(r.step([StepEntry(i, [reqs[i][pos[i]]], [0]) for i in live]).float().cpu())
            for i in live:
                pos[i] += 1
        torch.cuda.synchronize()
        r.rt.check_errors()
        runs[graphs] = (out, r.graph_replays)
        # whole sequences in a fresh pass give the same last logits
        for i in (1, 2, 3):
            r.end(i)
        whole = r.step([StepEntry(7, reqs[1][:pos[1]], [pos[1] - 1])]).float().cpu()
        assert rel_err(whole[0], runs[graphs][0][-1][0]) < 3e-2, (graphs, r.graph_replays, r.graph_captures)
        r.end(7)
    assert runs[False][1] == 0 and runs[True][1] >= 3
    for a, b in zip(runs[False][0], runs[True][0]):
        assert a.shape == b.shape
        # (padded steps send single tokens through the prefill attention, unpadded ones through the
        # fused decode attention: the same values up to bfloat16 rounding)
        assert (a - b).abs().max() <= 2e-2 * a.abs().max()


def test_a_mixer_whose_values_are_wider_than_its_keys_gets_pools_of_its_own_shapes():
    """A toy single-head attention with 8-wide keys and 24-wide values, defined
    here: the cache manager gives it a K pool and a V pool of those widths, and
    it steps in portions over reused pages like any other mixer."""
    from crane_b200.config import (EngineConfig, LayerSpec, ModelSpec, PartSpec, ScheduleStep,
                                   register_architecture, resolve)
    from crane_b200.engine import ModelRunner, StepEntry
    from crane_b200.parts import CacheNeed, Part, model_manifest, register_part
    from crane_b200.weights import TensorSpec
    from crane_b200.weights.random_init import random_tensors

    @register_part("mixer", "toy_wide_values")
    class WideValues(Part):
        kind = "mixer"
        capturable = False          # it plans on the host

        @classmethod
        def manifest(cls, spec):
            h, dk, dv = (spec.params[k] for k in ("hidden_size", "key_dim", "value_dim"))
            p = spec.prefix
            return {p + "wq": TensorSpec((dk, h)), p + "wk": TensorSpec((dk, h)), p + "wv": TensorSpec((dv, h)),
                    p + "wo": TensorSpec((h, dv))}

        def load(self, weights, rt):
            p = self.prefix
            self.wq, self.wk, self.wv, self.wo = (weights[p + n] for n in ("wq", "wk", "wv", "wo"))

        def cache_need(self):
            return CacheNeed("kv", kv_heads=1, head_dim=self.params["key_dim"], v_head_dim=self.params["value_dim"])

        def forward(self, h, ctx, cache, rt):
            x = h.float()
            q, k, v = x @ self.wq.float().t(), x @ self.wk.float().t(), x @ self.wv.float().t()
            table = ctx.block_tables[cache.group].cpu().numpy()
            ps = cache.page_size
            out = torch.empty(h.shape[0], self.wv.shape[0], device=h.device)
            for e in range(ctx.n_entries):
                a, b, n = int(ctx.h_cu_q[e]), int(ctx.h_cu_q[e + 1]), int(ctx.h_kv_len[e])
                for t in range(a, b):                          # write, then attend to everything so far
                    p = n - (b - a) + (t - a)
                    cache.k[int(table[e, p // ps]), 0, p % ps] = k[t].to(cache.k.dtype)
                    cache.v[int(table[e, p // ps]), 0, p % ps] = v[t].to(cache.v.dtype)
                pages = torch.from_numpy(table[e, :(n + ps - 1) // ps].astype(np.int64)).to(h.device)
                keys = cache.k[pages, 0].reshape(-1, cache.k.shape[-1])[:n].float()
                vals = cache.v[pages, 0].reshape(-1, cache.v.shape[-1])[:n].float()
                for t in range(a, b):
                    p = n - (b - a) + (t - a)
                    w = torch.softmax(keys[:p + 1] @ q[t] / keys.shape[1] ** 0.5, dim=0)
                    out[t] = w @ vals[:p + 1]
            return (out @ self.wo.float().t()).to(h.dtype)

    def build_spec(cfg):
        h = cfg["hidden_size"]
        norm = lambda p: PartSpec("norm", "rms_norm", {"size": h, "eps": 1e-5}, p)
        ffn = PartSpec("ffn", "swiglu", {"hidden_size": h, "intermediate_size": 64}, "l0.ffn.")
        mix = PartSpec("mixer", "toy_wide_values", {"hidden_size": h, "key_dim": 8, "value_dim": 24}, "l0.mix.")
        layers = [LayerSpec("prenorm_residual", {"norm1": norm("l0.n1."), "mixer": mix, "norm2": norm("l0.n2."),
                                                 "ffn": ffn})]
        return ModelSpec("ToyWideValuesForCausalLM", h, cfg["vocab"], 128,
                         PartSpec("embed", "token_embedding", {"vocab_size": cfg["vocab"], "hidden_size": h}, "emb."),
                         layers, [ScheduleStep(0)], norm("final."),
                         PartSpec("head", "lm_head", {"vocab_size": cfg["vocab"], "hidden_size": h,
                                                      "tied_to": "emb.weight"}, "head."))

    register_architecture("ToyWideValuesForCausalLM", lambda d: d, build_spec)
    cfg = {"architectures": ["ToyWideValuesForCausalLM"], "hidden_size": 48, "vocab": 70}
    spec = resolve(cfg).build_spec(cfg)
    tensors = random_tensors(model_manifest(spec), 5, torch.float32, std=0.2)
    r = ModelRunner(None, EngineConfig(dtype="float32", page_size=8, num_pages=9, max_concurrent=2,
                                       max_batched_tokens=64), config=cfg, tensors=tensors)
    lc = r.pools.layers[0]
    assert tuple(lc.k.shape) == (9, 1, 8, 8) and tuple(lc.v.shape) == (9, 1, 8, 24)
    rng = np.random.default_rng(2)
    a, b = rng.integers(0, 70, 37).tolist(), rng.integers(0, 70, 30).tolist()
    whole_a = r.step([StepEntry(1, a, list(range(37)))]).cpu()
    r.end(1)
    whole_b = r.step([StepEntry(2, b, list(range(30)))]).cpu()
    r.end(2)
    got_a = [r.step([StepEntry(3, a[:5], list(range(5)))]).cpu()]
    out = r.step([StepEntry(3, a[5:20], list(range(15))), StepEntry(4, b[:9], list(range(9)))]).cpu()
    got_a.append(out[:15]); got_b = [out[15:]]
    out = r.step([StepEntry(4, b[9:], list(range(21))), StepEntry(3, a[20:], list(range(17)))]).cpu()
    got_b.append(out[:21]); got_a.append(out[21:])
    assert rel_err(torch.cat(got_a), whole_a) < 2e-5 and rel_err(torch.cat(got_b), whole_b) < 2e-5
    r.end(3); r.end(4)
    r.table.check()
