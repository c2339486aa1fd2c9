"""Plain, slow Hunyuan Dense: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the
``crane_b200`` package: it reads the model folder with the ``safetensors``
library, keeps everything in float64 NumPy arrays and recomputes the whole
sequence for every answer.

It rests on the formulas of the reference alone (cryptomilk/Crane cannot be
compiled here: it is Rust on Candle and no Rust toolchain is installed), each
function citing the reference file and line it restates.  Two behaviours of
the reference are deliberately not restated, because they are artefacts of
its reduced-precision tensors and not of the architecture:

* cos/sin are *not* rounded to the model dtype before use
  (crane-core/src/models/hunyuan_dense/modeling.rs:1004-1009 rounds them);
* masked scores are excluded instead of getting the finite constant -1e9
  added (modeling.rs:1012-1033); for any realistic score the softmax is the
  same to the last bit.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

F = np.float64


# --------------------------------------------------------------------------
# configuration (crane-core/src/models/hunyuan_dense/modeling.rs:108-160)
# --------------------------------------------------------------------------
@dataclass
class PlainConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_alpha: float          # <= 0: plain RoPE
    attention_bias: bool
    use_qk_norm: bool
    tie_word_embeddings: bool
    use_cla: bool
    cla_share_factor: int

    @staticmethod
    def from_dict(d: dict) -> "PlainConfig":
        # defaults as in modeling.rs:135-159 (use_qk_norm and
        # tie_word_embeddings default to true, rope_theta to 10000,
        # head_dim to hidden_size / num_attention_heads)
        scaling = d.get("rope_scaling") or {}
        alpha = scaling.get("alpha")
        return PlainConfig(
            vocab_size=d["vocab_size"],
            hidden_size=d["hidden_size"],
            intermediate_size=d["intermediate_size"],
            num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d["num_key_value_heads"],
            head_dim=d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"],
            max_position_embeddings=d["max_position_embeddings"],
            rms_norm_eps=d["rms_norm_eps"],
            rope_theta=d.get("rope_theta") or 10000.0,
            rope_alpha=float(alpha) if alpha is not None else 0.0,
            attention_bias=bool(d.get("attention_bias") or False),
            use_qk_norm=d.get("use_qk_norm", True),
            tie_word_embeddings=d.get("tie_word_embeddings", True),
            use_cla=bool(d.get("use_cla") or False),
            cla_share_factor=int(d.get("cla_share_factor") or 1),
        )


def load_folder(folder: str):
    """Read config.json and model.safetensors into (PlainConfig, {name: float64 array})."""
    import torch
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = PlainConfig.from_dict(json.load(f))
    weights: Dict[str, np.ndarray] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(torch.float64).numpy()
    return cfg, weights


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed(tokens: Sequence[int], table: np.ndarray) -> np.ndarray:
    """x0 = E[token], no scaling (modeling.rs:831-835, 998)."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(F)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """y = x * rsqrt(mean(x^2) + eps) * w, weight applied after normalising
    (crane-core/kernels/fused_ops.cu:45-51, 91-98; modeling.rs:334-343)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * w


def rope_inv_freq(head_dim: int, theta: float, alpha: float) -> np.ndarray:
    """inv_freq[j] = 1 / base^(2j/d); base = theta * alpha^(d/(d-2)) when alpha > 0.
    The power is taken in float64, rounded to float32, and the reciprocal is a
    float32 division (modeling.rs:197-239)."""
    base = float(theta)
    if alpha > 0.0:
        # (head_dim 2: the reference's f64 division by zero gives +inf; powf(0) of the result is 1)
        base = base * float(alpha) ** (head_dim / (head_dim - 2.0) if head_dim != 2 else float("inf"))
    out = np.empty(head_dim // 2, dtype=np.float32)
    for n, i in enumerate(range(0, head_dim, 2)):
        out[n] = np.float32(1.0) / np.float32(base ** (i / head_dim))
    return out


def rope_angles(positions: np.ndarray, inv_freq: np.ndarray) -> np.ndarray:
    """angle[p, j] = float32(p) * inv_freq[j], a float32 product
    (modeling.rs:221-228: an F32 matmul of positions and inv_freq)."""
    p = positions.astype(np.float32)[:, None]
    return (p * inv_freq[None, :]).astype(np.float32)


def apply_rope(x: np.ndarray, angles: np.ndarray) -> np.ndarray:
    """Half-split rotation of x [T, heads, d] (modeling.rs:541-543 calls the
    contiguous-halves `rope`, not the interleaved one): for j < d/2
    out[j] = x[j] cos - x[j+d/2] sin ; out[j+d/2] = x[j+d/2] cos + x[j] sin."""
    half = x.shape[-1] // 2
    cos = np.cos(angles.astype(F))[:, None, :]
    sin = np.sin(angles.astype(F))[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], axis=-1)


def linear(x: np.ndarray, w: np.ndarray, b: Optional[np.ndarray] = None) -> np.ndarray:
    """y = x W^T (+ b), weights stored [out, in] (modeling.rs:273-330)."""
    y = x @ w.T
    return y if b is None else y + b


def softmax_rows(s: np.ndarray) -> np.ndarray:
    m = np.max(s, axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray,
                     window: int = 0) -> np.ndarray:
    """q [T, nq, d], k/v [T, nkv, d] of one whole sequence -> [T, nq*d].
    scores = q k^T / sqrt(d); position i sees j <= i (modeling.rs:629-636,
    1012-1033); query head h reads kv head h // (nq/nkv) (modeling.rs:611-626).
    `window` > 0 additionally hides j <= i - window (no Hunyuan layer uses it;
    it is here for the parts tests)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    n_rep = nq // nkv
    out = np.zeros((T, nq, d), dtype=F)
    idx = np.arange(T)
    # (the rows in blocks of 2048 only so that a long sequence's [T, T] scores need not exist at once)
    for r0 in range(0, T, 2048):
        r1 = min(T, r0 + 2048)
        allowed = idx[None, :r1] <= idx[r0:r1, None]
        if window > 0:
            allowed &= idx[None, :r1] > idx[r0:r1, None] - window
        for h in range(nq):
            g = h // n_rep
            s = (q[r0:r1, h, :] @ k[:r1, g, :].T) * (1.0 / math.sqrt(d))
            s = np.where(allowed, s, -np.inf)
            out[r0:r1, h, :] = softmax_rows(s) @ v[:r1, g, :]
    return out.reshape(T, nq * d)


def silu(x: np.ndarray) -> np.ndarray:
    """silu(x) = x / (1 + exp(-x)) (crane-core/kernels/fused_ops.cu:39-42)."""
    return x / (1.0 + np.exp(-x))


def swiglu(h: np.ndarray, w_gate, w_up, w_down) -> np.ndarray:
    """down( silu(gate(h)) * up(h) ), no biases (modeling.rs:667-694, 711-732)."""
    return linear(silu(linear(h, w_gate)) * linear(h, w_up), w_down)


def attention_layer(h: np.ndarray, cfg: PlainConfig, w: Dict[str, np.ndarray], prefix: str,
                    positions: np.ndarray, shared_kv=None, window: int = 0):
    """Projection, RoPE, then per-head RMSNorm of q and k, cache of the
    post-RoPE post-norm k, attention, output projection
    (modeling.rs:491-646).  With `shared_kv` only q is computed and the given
    (k, v) of the anchor layer are attended (modeling.rs:501-514)."""
    T = h.shape[0]
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    bias = (lambda n: w[prefix + n + ".bias"]) if cfg.attention_bias else (lambda n: None)
    angles = rope_angles(positions, rope_inv_freq(d, cfg.rope_theta, cfg.rope_alpha))
    q = linear(h, w[prefix + "q_proj.weight"], bias("q_proj")).reshape(T, nq, d)
    q = apply_rope(q, angles)
    if cfg.use_qk_norm:
        q = rms_norm(q, w[prefix + "query_layernorm.weight"], cfg.rms_norm_eps)
    if shared_kv is None:
        k = linear(h, w[prefix + "k_proj.weight"], bias("k_proj")).reshape(T, nkv, d)
        v = linear(h, w[prefix + "v_proj.weight"], bias("v_proj")).reshape(T, nkv, d)
        k = apply_rope(k, angles)
        if cfg.use_qk_norm:
            k = rms_norm(k, w[prefix + "key_layernorm.weight"], cfg.rms_norm_eps)
    else:
        k, v = shared_kv
    o = causal_attention(q, k, v, window)
    return linear(o, w[prefix + "o_proj.weight"], bias("o_proj")), (k, v)


def decoder_layer(x: np.ndarray, cfg: PlainConfig, w, i: int, positions, shared_kv=None):
    """Pre-norm residual block (modeling.rs:792-810)."""
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
    a, kv = attention_layer(h, cfg, w, p + "self_attn.", positions, shared_kv)
    x = x + a
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
    m = swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
               w[p + "mlp.down_proj.weight"])
    return x + m, kv


def hidden_states(cfg: PlainConfig, w, tokens: Sequence[int]) -> np.ndarray:
    """Final-norm output for every position of one whole sequence
    (modeling.rs:990-1061).  Cross-layer sharing: layer i with
    i % factor != 0 attends the k, v of the last layer with i % factor == 0
    (modeling.rs:1035-1058)."""
    positions = np.arange(len(tokens))
    x = embed(tokens, w["model.embed_tokens.weight"])
    anchor = None
    for i in range(cfg.num_hidden_layers):
        shared = None
        if cfg.use_cla and cfg.cla_share_factor > 1 and i % cfg.cla_share_factor != 0:
            shared = anchor
        x, kv = decoder_layer(x, cfg, w, i, positions, shared)
        if cfg.use_cla and cfg.cla_share_factor > 1 and i % cfg.cla_share_factor == 0:
            anchor = kv
    return rms_norm(x, w["model.norm.weight"], cfg.rms_norm_eps)


def logits_all(cfg: PlainConfig, w, tokens: Sequence[int]) -> np.ndarray:
    """Logits [T, V] at every position (the reference computes only the last
    row, modeling.rs:1062-1065; the head is the embedding when tied,
    modeling.rs:846-854)."""
    h = hidden_states(cfg, w, tokens)
    head = w["model.embed_tokens.weight"] if cfg.tie_word_embeddings else w["lm_head.weight"]
    return linear(h, head)


def greedy_generate(cfg: PlainConfig, w, prompt: Sequence[int], steps: int,
                    eos: Optional[int] = None) -> List[int]:
    """prompt ++ generated, ties to the lowest index; stops after an EOS,
    which stays in the list (crane-core/src/models/hunyuan_dense/model.rs:315-350)."""
    toks = list(prompt)
    for _ in range(steps):
        nxt = int(np.argmax(logits_all(cfg, w, toks)[-1]))
        toks.append(nxt)
        if eos is not None and nxt == eos:
            break
    return toks


# --------------------------------------------------------------------------
# sampling (crane-serve/src/engine/sampling.rs:117-327)
# --------------------------------------------------------------------------
_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_noise(seed: int, counter: int, vocab: int) -> np.ndarray:
    """The engine's counter-based uniforms, restated: u in [1e-7, 0.999)
    (range of sampling.rs:288-290) from a 24-bit fraction of
    splitmix64(splitmix64(seed + counter * GOLDEN) ^ index * ODD)."""
    key = _splitmix64((seed + counter * 0x9E3779B97F4A7C15) & _M64)
    out = np.empty(vocab, dtype=np.float64)
    for i in range(vocab):
        x = _splitmix64(key ^ ((i * 0xD6E8FEB86659FD93) & _M64))
        r = np.float32(x >> 40) * np.float32(1.0 / 16777216.0)
        out[i] = np.float32(1e-7) + np.float32(0.999 - 1e-7) * r
    return out


def apply_repetition_penalty(logits: np.ndarray, penalty: float, context: Sequence[int]) -> np.ndarray:
    """Seen tokens: logit / penalty if >= 0 else logit * penalty, once per
    distinct token (crane-core/src/models/utils.rs:25-44; sampling.rs:301-327)."""
    out = logits.copy()
    for t in set(int(c) for c in context):
        if 0 <= t < out.shape[0]:
            out[t] = out[t] / penalty if out[t] >= 0 else out[t] * penalty
    return out


def gumbel_scores(logits: np.ndarray, temperature: float, u: np.ndarray) -> np.ndarray:
    """argmax of logits/T - log(-log u) samples the softmax (sampling.rs:288-298)."""
    return logits / temperature - np.log(-np.log(u))


def top_k_top_p_keep(logits: np.ndarray, temperature: float, top_k: int, top_p: float) -> np.ndarray:
    """Indices that survive top-k then top-p, best first.  top-p keeps the
    candidates whose cumulative probability is <= top_p plus the one after
    them, and always the first (sampling.rs:237-258: mask_le OR its shift by
    one); the probabilities are a softmax over the top-k set only."""
    order = np.argsort(-logits, kind="stable")
    if top_k > 0:
        order = order[: min(top_k, logits.shape[0])]
    if 0.0 < top_p < 1.0:
        p = softmax_rows((logits[order] / temperature)[None, :])[0]
        le = np.cumsum(p) <= top_p
        keep = le.copy()
        keep[1:] |= le[:-1]
        keep[0] = True
        order = order[keep]
    return order
