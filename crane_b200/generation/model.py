"""The Python entry point in the reference's manner: load a model folder,
``generate(input_ids, config, streamer)``.

``generate`` follows the reference's loop
(crane-core/src/models/hunyuan_dense/model.rs:295-371): returns prompt ++
generated; an EOS token ends generation, stays in the returned list and is not
streamed; the streamer is finalized exactly once; ``report_speed`` prints
tokens per second over the whole loop.  Unlike the reference it runs through
the scheduler, so ``generate_batch`` serves many prompts at once with
continuous batching.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

from ..config import EngineConfig
from ..engine.llm_engine import LLMEngine
from ..engine.step import ModelRunner
from ..sampling import SamplingParams
from .config import GenerationConfig
from .streamer import TokenStreamer


def _sampling(config: GenerationConfig) -> SamplingParams:
    return SamplingParams(temperature=config.temperature, top_p=config.top_p, top_k=config.top_k,
                          repetition_penalty=config.repetition_penalty,
                          repeat_last_n=config.repeat_last_n, seed=config.seed)


class ModelForCausalLM:
    def __init__(self, runner: ModelRunner):
        self.runner = runner
        self.engine = LLMEngine(runner)
        self.config = runner.model_config

    @classmethod
    def from_pretrained(cls, model_dir: str, dtype: str = "bf16", model_type: Optional[str] = None,
                        random_weights: bool = False, seed: int = 0, **engine_options) -> "ModelForCausalLM":
        """``model_dir`` holds config.json and safetensors; the model class is
        chosen by config.json.  ``random_weights``: only config.json is read and
        the weights are drawn from ``seed``.  ``engine_options`` are
        ``EngineConfig`` fields."""
        if random_weights:
            import torch
            from ..config import read_config_json
            from ..weights.random_init import model_manifest_for, random_tensors
            cfg = read_config_json(model_dir)
            store = torch.float32 if dtype in ("fp32", "float32", "f32") else torch.bfloat16
            device = engine_options.get("device", "cuda:0")
            tensors = random_tensors(model_manifest_for(cfg, model_type), seed, store, device)
            return cls(ModelRunner(None, EngineConfig(dtype=dtype, **engine_options), config=cfg,
                                   tensors=tensors, model_type=model_type))
        return cls(ModelRunner(model_dir, EngineConfig(dtype=dtype, **engine_options),
                               model_type=model_type))

    @classmethod
    def from_tensors(cls, config: dict, tensors, dtype: str = "bf16", **engine_options):
        """A model from a config.json dict and tensors by name already in memory."""
        return cls(ModelRunner(None, EngineConfig(dtype=dtype, **engine_options), config=config,
                               tensors=tensors))

    @property
    def device(self):
        return self.runner.rt.device

    def _eos(self, config: GenerationConfig) -> List[int]:
        return [config.eos_token_id] if config.eos_token_id is not None else list(
            self.runner.spec.eos_token_ids)

    def generate(self, input_ids: Sequence[int], config: Optional[GenerationConfig] = None,
                 streamer: Optional[TokenStreamer] = None) -> List[int]:
        config = config or GenerationConfig()
        eos = self._eos(config)
        t0 = time.perf_counter()

        def on_token(rid: int, token: int, reason: Optional[str]) -> None:
            if streamer is not None and not (reason == "stop" and token in eos):
                streamer.append(token)
        try:
            rid = self.engine.add_request(list(input_ids), _sampling(config), config.max_new_tokens,
                                          eos, on_token)
            out = self.engine.run_until_done()[rid]
        finally:
            if streamer is not None:
                streamer.finalize()
        if out.finish_reason == "cache_too_small":
            raise RuntimeError("the cache pool is too small for this request")
        if config.report_speed:
            n = len(out.generated)
            print(f"\n{n} tokens generated ({n / (time.perf_counter() - t0):.2f} token/s)\n")
        return out.tokens

    def generate_batch(self, prompts: Sequence[Sequence[int]],
                       config: Optional[GenerationConfig] = None) -> List[List[int]]:
        """Every prompt through the scheduler at once; results in the order given."""
        config = config or GenerationConfig()
        eos = self._eos(config)
        ids = []
        for i, p in enumerate(prompts):
            sp = _sampling(config)
            if sp.seed is not None:
                sp.seed += i                     # one random stream per prompt
            ids.append(self.engine.add_request(list(p), sp, config.max_new_tokens, eos))
        done = self.engine.run_until_done()
        return [done[i].tokens for i in ids]

    def warmup(self) -> None:
        """A short generation that compiles and loads everything
        (hunyuan_dense/model.rs:278-287: 3-token prompt, 5 new tokens)."""
        v = self.runner.spec.vocab_size
        self.generate([1 % v, 2 % v, 3 % v], GenerationConfig(max_new_tokens=5, temperature=None,
                                                              eos_token_id=-1))

    def clear_kv_cache(self) -> None:
        """Nothing to clear between calls: a finished request has already given
        its pages back.  Kept for callers of the reference's API."""

    def stats(self) -> dict:
        return self.engine.stats()
