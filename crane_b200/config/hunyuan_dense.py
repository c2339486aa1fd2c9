"""Typed configuration of Hunyuan Dense, read from the keys of its config.json.

Keys, defaults and which keys are read but unused follow the reference's
serde struct (crane-core/src/models/hunyuan_dense/modeling.rs:108-160).
Validation beyond the reference: head grouping, even head size, sizes > 0.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model of this architecture."""


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` object; only `alpha` changes the model (modeling.rs:202-219)."""
    alpha: Optional[float] = None
    beta_fast: Optional[float] = None
    beta_slow: Optional[float] = None
    factor: Optional[float] = None
    mscale: Optional[float] = None
    mscale_all_dim: Optional[float] = None
    type: Optional[str] = None

    @staticmethod
    def from_dict(d: Optional[Dict[str, Any]]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise ConfigError(f"rope_scaling must be an object, got {type(d).__name__}")
        known = {f.name for f in fields(RopeScaling)}
        return RopeScaling(**{k: v for k, v in d.items() if k in known})


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
             "rms_norm_eps")


@dataclass(frozen=True)
class HunyuanDenseConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    max_position_embeddings: int
    rms_norm_eps: float
    head_dim: int = 0                      # 0: hidden_size // num_attention_heads
    hidden_act: str = "silu"               # read, never consulted (modeling.rs:129, 730)
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    attention_bias: bool = False
    use_qk_norm: bool = True
    tie_word_embeddings: bool = True
    use_cla: bool = False
    cla_share_factor: int = 1
    eos_token_id: Optional[Tuple[int, ...]] = None   # not in the reference's struct; honoured if present
    architectures: Tuple[str, ...] = ("HunYuanDenseV1ForCausalLM",)
    model_type: str = "hunyuan_v1_dense"

    # ---- derived ----
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rope_alpha(self) -> float:
        a = self.rope_scaling.alpha if self.rope_scaling is not None else None
        return float(a) if a is not None and a > 0 else 0.0

    @property
    def cla_active(self) -> bool:
        return self.use_cla and self.cla_share_factor > 1

    # ---- construction ----
    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "HunyuanDenseConfig":
        missing = [k for k in _REQUIRED if d.get(k) is None]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        eos = d.get("eos_token_id")
        if isinstance(eos, int):
            eos = (eos,)
        elif isinstance(eos, (list, tuple)):
            eos = tuple(int(e) for e in eos)
        else:
            eos = None
        head_dim = d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"]
        cfg = HunyuanDenseConfig(
            vocab_size=int(d["vocab_size"]),
            hidden_size=int(d["hidden_size"]),
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=int(d["num_attention_heads"]),
            num_key_value_heads=int(d["num_key_value_heads"]),
            max_position_embeddings=int(d["max_position_embeddings"]),
            rms_norm_eps=float(d["rms_norm_eps"]),
            head_dim=int(head_dim),
            hidden_act=str(d.get("hidden_act", "silu")),
            rope_theta=float(d["rope_theta"]) if d.get("rope_theta") is not None else 10000.0,
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            attention_bias=bool(d.get("attention_bias") or False),
            use_qk_norm=bool(d.get("use_qk_norm", True)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
            use_cla=bool(d.get("use_cla") or False),
            cla_share_factor=int(d.get("cla_share_factor") or 1),
            eos_token_id=eos,
            architectures=tuple(d.get("architectures") or ("HunYuanDenseV1ForCausalLM",)),
            model_type=str(d.get("model_type", "hunyuan_v1_dense")),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be > 0, got {self.rope_theta}")
        if self.cla_share_factor < 1:
            raise ConfigError(f"cla_share_factor must be >= 1, got {self.cla_share_factor}")

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "attention_bias": self.attention_bias,
            "use_qk_norm": self.use_qk_norm,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_cla": self.use_cla,
            "cla_share_factor": self.cla_share_factor,
        }
        if self.rope_scaling is not None:
            d["rope_scaling"] = {k: v for k, v in vars(self.rope_scaling).items() if v is not None}
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id)
        return d


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d


# --------------------------------------------------------------------------
# layout of the model as parts
# --------------------------------------------------------------------------
ARCHITECTURE = "HunYuanDenseV1ForCausalLM"
ALIASES = ("hunyuan", "hunyuan_dense", "hunyuandense", "hunyuan_v1_dense")
# the reference's stop token when none is given
# (crane-core/src/models/hunyuan_dense/model.rs:311)
DEFAULT_EOS_TOKEN_ID = 120020


def build_spec(cfg: HunyuanDenseConfig):
    """Hunyuan Dense as data: pre-norm residual blocks of grouped-query
    attention (rotary encoding, then per-head RMSNorm of q and k) and a
    SiLU-gated feed-forward; final RMSNorm; head tied to the embedding or not
    (modeling.rs:743-867).  With cross-layer sharing, layer i with
    i % factor != 0 has no keys or values of its own and reads the cache of
    the last layer with i % factor == 0 (modeling.rs:1035-1058)."""
    from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

    position = PartSpec("position", "rope", {
        "head_dim": cfg.head_dim, "theta": cfg.rope_theta, "alpha": cfg.rope_alpha,
        "max_positions": cfg.max_position_embeddings})
    layers, schedule, ignored = [], [], {}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        shared = cfg.cla_active and i % cfg.cla_share_factor != 0
        anchor = i - i % cfg.cla_share_factor if shared else None
        mixer = PartSpec("mixer", "gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "bias": cfg.attention_bias, "qk_norm": cfg.use_qk_norm, "qk_norm_eps": cfg.rms_norm_eps,
            "window": 0, "own_kv": not shared, "position": position}, prefix=p + "self_attn.")
        if shared:
            for n in ("k_proj", "v_proj"):
                ignored[p + f"self_attn.{n}.weight"] = "layer reads another layer's cache"
                if cfg.attention_bias:
                    ignored[p + f"self_attn.{n}.bias"] = "layer reads another layer's cache"
            if cfg.use_qk_norm:
                ignored[p + "self_attn.key_layernorm.weight"] = "layer reads another layer's cache"
        layers.append(LayerSpec("prenorm_residual", {
            "norm1": PartSpec("norm", "rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                              prefix=p + "input_layernorm."),
            "mixer": mixer,
            "norm2": PartSpec("norm", "rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                              prefix=p + "post_attention_layernorm."),
            "ffn": PartSpec("ffn", "swiglu", {"hidden_size": cfg.hidden_size,
                                              "intermediate_size": cfg.intermediate_size},
                            prefix=p + "mlp."),
        }))
        schedule.append(ScheduleStep(i, anchor))
    if cfg.tie_word_embeddings:
        ignored["lm_head.weight"] = "head is tied to the embedding"
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embed=PartSpec("embed", "token_embedding",
                       {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                       prefix="model.embed_tokens."),
        layers=layers,
        schedule=schedule,
        final_norm=PartSpec("norm", "rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                            prefix="model.norm."),
        head=PartSpec("head", "lm_head", {
            "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None},
            prefix="lm_head."),
        eos_token_ids=list(cfg.eos_token_id) if cfg.eos_token_id else [DEFAULT_EOS_TOKEN_ID],
        ignored_tensors=ignored,
    )
