"""Grouped-query attention over the paged cache.

One product for q, k and v (the three matrices merged, as in the reference,
crane-core/src/models/hunyuan_dense/modeling.rs:349-365, 516-528); rotary
encoding of q and k, THEN per-head RMSNorm of q and k with one [d] weight each
(modeling.rs:541-555); the post-rotary, post-norm k and the raw v go to the
cache (modeling.rs:557); scores q k^T / sqrt(d), causal, softmax, times v;
query head h reads kv head h // (nq / nkv) (modeling.rs:572-636); output
projection (modeling.rs:638-645).  A layer without keys and values of its own
computes q only and reads the cache it is given (modeling.rs:501-514).
"""
from __future__ import annotations

import math
import os

import torch

from ..weights.loader import TensorSpec
from .base import CacheNeed, Part, build_part, query_tiles, register_part


@register_part("mixer", "gqa_attention")
class GqaAttention(Part):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``bias`` (q/k/v/o biases), ``qk_norm`` + ``qk_norm_eps``, ``window`` (0: all
    earlier positions), ``own_kv`` (False: reads another layer's cache),
    ``position`` (a PartSpec of kind position, or None), ``scale`` (default
    1/sqrt(head_dim)); and how heads are rotated and normalised, whose defaults
    are the reference's: ``rotary_dim`` (the leading elements of a head that
    are rotated; default all), ``rope_pairing`` ("half": element i with
    i + rotary_dim/2, or "interleaved": 2i with 2i + 1), ``qk_norm_order``
    ("after_rope" or "before_rope"), ``qk_norm_offset`` (the norms multiply by
    offset + w: 0, or 1 for weights stored as w - 1).
    Tensors: ``<prefix>{q,k,v,o}_proj.weight`` (+ ``.bias``),
    ``<prefix>query_layernorm.weight`` / ``key_layernorm.weight`` [head_dim]."""
    kind = "mixer"

    @classmethod
    def manifest(cls, spec):
        a = spec.params
        h, nq, nkv, d = a["hidden_size"], a["num_heads"], a["num_kv_heads"], a["head_dim"]
        p = spec.prefix
        own = a.get("own_kv", True)
        m = {p + "q_proj.weight": TensorSpec((nq * d, h)), p + "o_proj.weight": TensorSpec((h, nq * d))}
        if own:
            m[p + "k_proj.weight"] = TensorSpec((nkv * d, h))
            m[p + "v_proj.weight"] = TensorSpec((nkv * d, h))
        if a.get("bias"):
            m[p + "q_proj.bias"] = TensorSpec((nq * d,), "float32")
            m[p + "o_proj.bias"] = TensorSpec((h,), "float32")
            if own:
                m[p + "k_proj.bias"] = TensorSpec((nkv * d,), "float32")
                m[p + "v_proj.bias"] = TensorSpec((nkv * d,), "float32")
        if a.get("qk_norm"):
            m[p + "query_layernorm.weight"] = TensorSpec((d,), "float32")
            if own:
                m[p + "key_layernorm.weight"] = TensorSpec((d,), "float32")
        return m

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.nq, self.nkv, self.d = int(a["num_heads"]), int(a["num_kv_heads"]), int(a["head_dim"])
        self.own_kv = bool(a.get("own_kv", True))
        self.window = int(a.get("window") or 0)
        self.scale = float(a.get("scale") or 1.0 / math.sqrt(self.d))
        self.eps = float(a.get("qk_norm_eps") or 0.0)
        if self.nq % self.nkv:
            raise ValueError(f"{p}: {self.nq} query heads are not a multiple of {self.nkv} kv heads")
        if self.d % 2 or self.d > 256:
            raise ValueError(f"{p}: head_dim {self.d} is not supported by the attention kernels "
                             "(even sizes up to 256)")
        names = ["q_proj"] + (["k_proj", "v_proj"] if self.own_kv else [])
        ws = [weights.pop(p + n + ".weight") for n in names]
        self.qkv_w = torch.cat(ws, dim=0).contiguous() if len(ws) > 1 else ws[0]
        self.qkv_b = (torch.cat([weights.pop(p + n + ".bias") for n in names]).contiguous()
                      if a.get("bias") else None)
        self.o_w = weights[p + "o_proj.weight"]
        self.o_b = weights.get(p + "o_proj.bias") if a.get("bias") else None
        self.q_norm = weights.get(p + "query_layernorm.weight") if a.get("qk_norm") else None
        self.k_norm = weights.get(p + "key_layernorm.weight") if a.get("qk_norm") and self.own_kv else None
        self.position = build_part(a["position"]) if a.get("position") is not None else None
        if self.position is not None:
            self.position.load(weights, rt)          # a position encoding may have tensors of its own
        self.qkv_cols = self.qkv_w.shape[0]
        rotary_dim = int(a.get("rotary_dim") or self.d)
        pairing, order = a.get("rope_pairing") or "half", a.get("qk_norm_order") or "after_rope"
        if rotary_dim % 2 or not 0 < rotary_dim <= self.d:
            raise ValueError(f"{p}: rotary_dim {rotary_dim} must be even and at most head_dim {self.d}")
        if pairing not in ("half", "interleaved") or order not in ("after_rope", "before_rope"):
            raise ValueError(f"{p}: rope_pairing is 'half' or 'interleaved', qk_norm_order 'after_rope' or "
                             f"'before_rope'; got {pairing!r}, {order!r}")
        # (rotated width, interleaved pairs, norm before the rotation, offset added to the norm weights)
        self.rope = (rotary_dim, pairing == "interleaved", order == "before_rope",
                     float(a.get("qk_norm_offset") or 0.0))
        self.max_splits = int(os.environ.get("CRANE_DECODE_SPLITS", "64"))

    def cache_need(self) -> CacheNeed:
        if not self.own_kv:
            return CacheNeed("none")
        return CacheNeed("kv", kv_heads=self.nkv, head_dim=self.d, window=self.window)

    def forward(self, h, ctx, cache, rt):
        n = h.shape[0]
        k = rt.kernels
        # (keys and values of more than a few MB stream through L2 between this product and the output
        # projection: asking for that one's weights now would only fetch them twice)
        kv_bytes = int(ctx.h_kv_len[:ctx.n_entries].sum()) * self.nkv * self.d * 4
        qkv = rt.linear(h, self.qkv_w, self.qkv_b, "attn_qkv", hint_next=kv_bytes < (8 << 20))
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.tables(rt, ctx.max_positions)
            if cos.shape[1] * 2 != self.rope[0]:
                raise ValueError(f"{self.prefix}: the position encoding gives tables for a rotated width of "
                                 f"{cos.shape[1] * 2}, the mixer rotates {self.rope[0]}")
        table = ctx.block_tables[cache.group]
        o = rt.ws.get("attn_o", n, self.nq * self.d, rt.dtype)
        decode = (not rt.exact and ctx.max_q_len == 1 and n == ctx.n_entries
                  and k.decode_attention_supports(self.d, self.nq, self.nkv))
        if decode and self.d % 4 == 0:
            # single decoded tokens: rotary encoding, head norms, the cache write, attention over
            # key slices (enough of them to fill the device) in one kernel, their merge in a second
            splits = k.decode_splits(ctx.n_entries, self.nkv, rt.num_sms, self.max_splits,
                                     max_keys=ctx.max_kv_len)
            # slices x entries never exceed two CTAs per SM, or the slices are 4 at most: that bounds
            # the slices' scratch rows
            rows = self.nq * max(2 * rt.num_sms // self.nkv + 1, 4 * rt.max_decode_rows)
            part_o = rt.ws.get("attn_part_o", rows, self.d, torch.float32, cap=rows)
            part_ml = rt.ws.get("attn_part_ml", rows, 2, torch.float32, cap=rows)
            k.paged_decode_attention_fused(qkv, self.qkv_cols, self.own_kv, cos, sin, self.q_norm,
                                           self.k_norm, self.eps, o, cache.k, cache.v, ctx.cu_q,
                                           ctx.kv_len, table, cache.page_size, self.nq, self.nkv,
                                           self.d, self.window, self.scale, splits, part_o, part_ml,
                                           rt.err, rope=self.rope)
            rt.launches += 1 if splits <= 8 else 2     # the merge is a launch of its own above 8 slices
            return rt.linear(o, self.o_w, self.o_b, "attn_out")
        q = rt.ws.get("attn_q", n, self.nq * self.d, rt.dtype)
        k.rope_norm_cache(qkv, self.qkv_cols, rt.dtype, ctx.positions, ctx.tok_entry, table, cos,
                          sin, self.q_norm, self.k_norm, self.eps, q, cache.k, cache.v,
                          cache.page_size, self.nq, self.nkv, self.d, self.own_kv,
                          self.position is not None, rt.err, rope=self.rope)
        use_mma = not rt.exact and k.prefill_attention_supports(self.d, self.nq, self.nkv)
        # Whole prompts of at most 64 tokens take the warp-level kernel (64-row tiles, several CTAs per
        # SM) also at head size 128.  Measured at 16 / 4 heads, tcgen05 against warp-level: 256 prompts of
        # 8 tokens 244 / 144 us, 64 of 32: 44 / 28 us, 32 of 64: 22 / 19 us; 21 of 96: 22 / 23 us, 16 of 128:
        # 16 / 21 us; 16 portions of 32 behind 2,000 cached keys 50 / 94 us.
        short = bool(getattr(ctx, "short_prompts", False)) and use_mma
        use_tc = (not rt.exact and rt.use_tc_attention and not short
                  and k.prefill_attention_tc_supports(self.d, self.nq, self.nkv, cache.page_size))
        # Decoded tokens beside prompt portions: the entries of one token go to the split-KV decode
        # kernel (which skips the others), the prompt portions to the prefill kernel (which skips them).
        singles = getattr(ctx, "single_entries", 0) if (use_tc or use_mma) and not decode else 0
        if singles and not k.decode_attention_supports(self.d, self.nq, self.nkv):
            singles = 0
        if decode or singles:
            if decode:
                splits = max(1, min(32, (2 * rt.num_sms) // max(1, ctx.n_entries * self.nkv)))
            else:
                # at most 8 slices: at head size 128 they merge inside a cluster without scratch
                splits = min(8, k.decode_splits(singles, self.nkv, rt.num_sms, self.max_splits))
            part_o = part_ml = None
            if splits > 1:
                rows = rt.max_decode_rows * self.nq * 32
                part_o = rt.ws.get("attn_part_o", rows, self.d, torch.float32, cap=rows)
                part_ml = rt.ws.get("attn_part_ml", rows, 2, torch.float32, cap=rows)
            k.paged_decode_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table,
                                     cache.page_size, self.nq, self.nkv, self.d, self.window,
                                     self.scale, splits, part_o, part_ml, rt.err)
            rt.launches += 3 if splits > 1 else 2
            if decode:
                return rt.linear(o, self.o_w, self.o_b, "attn_out")
            rt.launches -= 1                      # the rotary kernel is counted once, below
        if use_tc:
            tiles = query_tiles(ctx, 128, skip_single=bool(singles))
            k.prefill_attention_tc(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table, cache.page_size,
                                   tiles, self.nq, self.nkv, self.d, self.window, self.scale, rt.err,
                                   skip_single=bool(singles))
            rt.launches += 2
        elif use_mma:
            tiles = query_tiles(ctx, 64, skip_single=bool(singles))
            k.paged_prefill_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table,
                                      cache.page_size, tiles, self.nq, self.nkv, self.d, self.window,
                                      self.scale, rt.err, skip_single=bool(singles))
            rt.launches += 2
        else:
            k.paged_attention_simt(q, o, cache.k, cache.v, ctx.positions, ctx.tok_entry, table,
                                   cache.page_size, self.nq, self.nkv, self.d, self.window,
                                   self.scale, rt.err)
            rt.launches += 2
        return rt.linear(o, self.o_w, self.o_b, "attn_out")
