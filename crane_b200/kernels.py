"""Python face of the CUDA library: one method per kernel, tensors in, tensors out.

Every method launches on torch's current stream of the tensor's device and
checks the launch status.  There is no other implementation behind these
methods: if the library cannot be built or loaded, constructing ``Kernels``
raises.
"""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Union

import torch

from .csrc import build

P, I, L, F = c_void_p, c_int, c_longlong, c_float

_SIGNATURES = {
    "crane_embed_gather": [I, P, P, P, I, I, I, P, I, P, P],
    "crane_add_rmsnorm": [I, P, P, P, I, L, P, P, P, I, I, F, P],
    "crane_rope_norm_cache": [I, P, P, I, L, I, P, P, P, I, P, P, I, P, P, F, P, P, P, I, I, I, I,
                              I, I, I, I, I, I, I, F, P, P],
    "crane_silu_mul": [I, P, P, I, L, P, I, I, I, P],
    "crane_to_float": [I, P, P, L, P],
    "crane_sum_parts": [P, I, L, L, P, L, I, I, P],
    "crane_gemm_simt": [I, I, P, P, P, P, I, I, I, L, L, L, P],
    "crane_gemm_bf16_tcgen05": [P, P, P, P, I, I, I, L, L, L, I, I, I, I, I, L, I, P, L, P, P],
    "crane_gemm_bf16_pair": [P, P, P, P, I, I, I, L, L, L, I, I, I, P, P],
    "crane_paged_attention_simt": [I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P],
    "crane_paged_decode_attention_supports": [I, I, I],
    "crane_paged_decode_attention": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P, P],
    "crane_paged_prefill_attention_supports": [I, I, I],
    "crane_paged_prefill_attention": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P],
    "crane_paged_decode_attention_fused": [P, P, I, L, I, I, I, P, P, I, P, P, F, P, P, P, P, P, P, P, P,
                                           I, I, I, I, I, I, I, I, F, I, I, I, I, F, P, P],
    "crane_prefill_attention_tc_supports": [I, I, I, I],
    "crane_prefill_attention_tc": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P],
    "crane_repetition_penalty": [P, L, I, I, P, I, P, P, P],
    "crane_sample": [P, L, I, I, P, P, P, P, P, P, P],
}


class KernelError(RuntimeError):
    pass


class Partials:
    """A matrix product left as ``n`` float partial sums [n, rows, cols] (split
    along the inner dimension); the consumer adds them up in order."""

    def __init__(self, parts: torch.Tensor):
        self.parts = parts

    @property
    def shape(self):
        return self.parts.shape[1:]

    def sum(self, dtype=None):
        """The product itself: the slices added up in order (rounded once to ``dtype``)."""
        total = self.parts.sum(dim=0)
        return total if dtype is None else total.to(dtype)


Act = Union[torch.Tensor, Partials]


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 storage, got {dtype}")


def _split(a: Act):
    """(whole ptr, parts ptr, n_parts, part_stride) of a product result."""
    if isinstance(a, Partials):
        p = a.parts
        return None, p.data_ptr(), p.shape[0], p.stride(0)
    return a.data_ptr(), None, 0, 0


class Kernels:
    def __init__(self, head_sizes=()) -> None:
        self.head_sizes: set = set()      # head sizes whose warp-level attention kernels the loaded library holds
        self._bind(build.load_kernels([d for d in head_sizes if d in build.ATTENTION_HEAD_SIZES]))

    def _bind(self, lib) -> None:
        self.lib = lib
        for name, sig in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes = sig
            fn.restype = c_int
        # kernels of a step overlap their start with the end of the kernel before them
        self.lib.crane_set_pdl.argtypes = [c_int]
        self.lib.crane_set_pdl.restype = None
        self.lib.crane_set_pdl(0 if os.environ.get("CRANE_PDL", "1") == "0" else 1)
        self.head_sizes = {d for d in build.ATTENTION_HEAD_SIZES
                           if self.lib.crane_paged_decode_attention_supports(d, 1, 1)}

    def require_head_size(self, d: int) -> None:
        """Makes sure the loaded library holds the warp-level attention kernels of
        head size ``d`` (if there are any for it): a first call for a model
        compiles what that model needs, a model with another head size adds its
        two files.  The library that was loaded before stays loaded (graphs that
        were recorded with it keep working)."""
        if d in self.head_sizes or d not in build.ATTENTION_HEAD_SIZES:
            return
        self._bind(build.load_kernels(sorted(self.head_sizes | {d})))

    # While a model runs a step, every launch goes to the stream that was current when the step
    # began (looked up once, not per launch); outside a step the current stream is asked for.
    pinned_stream: Optional[int] = None

    def _stream(self, t: torch.Tensor) -> int:
        if self.pinned_stream is not None:
            return self.pinned_stream
        return torch.cuda.current_stream(t.device).cuda_stream

    @staticmethod
    def _check(code: int, what: str) -> None:
        if code != 0:
            raise KernelError(f"{what}: CUDA error {code}")

    # ---- elementwise ---------------------------------------------------
    def embed_gather(self, tokens, table, x, err, deferred=None) -> None:
        """``deferred`` int32 [R]: a token id <= -2 is read from its row -id - 2."""
        n, hidden = x.shape
        self._check(self.lib.crane_embed_gather(_dt(table.dtype), tokens.data_ptr(), table.data_ptr(),
                                                x.data_ptr(), n, hidden, table.shape[0],
                                                deferred.data_ptr() if deferred is not None else None,
                                                deferred.numel() if deferred is not None else 0,
                                                err.data_ptr(), self._stream(x)), "embed_gather")

    def add_rmsnorm(self, x, delta: Optional[Act], weight, eps: float, out, rows=None) -> None:
        """x += delta (if given); out = rmsnorm(x) * weight.  With ``rows`` only
        those rows of x are read (and x is not written)."""
        whole, parts, n_parts, stride = (None, None, 0, 0) if delta is None else _split(delta)
        n_rows = out.shape[0]
        self._check(self.lib.crane_add_rmsnorm(_dt(out.dtype), x.data_ptr(), whole, parts, n_parts,
                                               stride, weight.data_ptr(), _ptr(rows), out.data_ptr(),
                                               n_rows, x.shape[1], float(eps), self._stream(x)),
                    "add_rmsnorm")

    def rope_norm_cache(self, qkv: Act, qkv_cols: int, dtype, positions, tok_entry, block_table,
                        cos, sin, q_norm_w, k_norm_w, eps, q_out, k_pool, v_pool, page_size, nq,
                        nkv, d, has_kv: bool, rotary: bool, err, rope=None) -> None:
        """``rope``: (rotary_dim, interleaved pairs, norm before the rotation,
        norm weight offset); None: the whole head, contiguous halves, norm after,
        plain weights.  cos/sin are [positions, rotary_dim / 2]."""
        rd, inter, first, off = rope or (d, False, False, 0.0)
        whole, parts, n_parts, stride = _split(qkv)
        n_tokens = q_out.shape[0]
        num_pages = k_pool.shape[0] if k_pool is not None else 0
        max_blocks = block_table.shape[1] if block_table is not None else 0
        self._check(self.lib.crane_rope_norm_cache(
            _dt(dtype), whole, parts, n_parts, stride, qkv_cols, positions.data_ptr(),
            _ptr(tok_entry), _ptr(block_table), max_blocks, _ptr(cos), _ptr(sin),
            cos.shape[0] if cos is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
            q_out.data_ptr(), _ptr(k_pool), _ptr(v_pool), num_pages, page_size, n_tokens, nq, nkv,
            d, 1 if has_kv else 0, 1 if rotary else 0, int(rd), 1 if inter else 0, 1 if first else 0,
            float(off), err.data_ptr(), self._stream(q_out)), "rope_norm_cache")

    def silu_mul(self, gu: Act, out, blocked: bool = False) -> None:
        """out = silu(gate) * up.  ``gu`` rows are [gate | up], or, ``blocked``,
        16 gate columns then the 16 up columns of the same features, and so on."""
        whole, parts, n_parts, stride = _split(gu)
        self._check(self.lib.crane_silu_mul(_dt(out.dtype), whole, parts, n_parts, stride,
                                            out.data_ptr(), out.shape[0], out.shape[1],
                                            1 if blocked else 0, self._stream(out)), "silu_mul")

    def sum_parts(self, parts: "Partials", out) -> None:
        """out[rows, cols] (float) = the partial sums added up in slice order."""
        p = parts.parts
        assert p.dtype == torch.float32 and out.dtype == torch.float32 and out.shape == p.shape[1:]
        assert p.stride(2) == 1 and out.stride(1) == 1
        self._check(self.lib.crane_sum_parts(p.data_ptr(), p.shape[0], p.stride(0), p.stride(1),
                                             out.data_ptr(), out.stride(0), p.shape[1], p.shape[2],
                                             self._stream(out)), "sum_parts")

    def to_float(self, t, out) -> None:
        self._check(self.lib.crane_to_float(_dt(t.dtype), t.data_ptr(), out.data_ptr(), t.numel(),
                                            self._stream(t)), "to_float")

    # ---- matrix product on the FP32 cores ------------------------------
    def gemm_simt(self, a, w, bias, out) -> None:
        """out[M,N] = a[M,K] @ w[N,K]^T (+ bias); rows may be strided."""
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and out.shape == (M, N)
        assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
        self._check(self.lib.crane_gemm_simt(_dt(a.dtype), _dt(out.dtype), a.data_ptr(),
                                             w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
                                             a.stride(0), w.stride(0), out.stride(0),
                                             self._stream(a)), "gemm_simt")

    # ---- matrix product on the tensor cores (bfloat16) -------------------
    @staticmethod
    def tcgen05_takes(x, w) -> bool:
        """Whether the tensor-core kernel takes these operands: bfloat16, inner
        dimension and row pitches multiples of 8 elements, 16-byte aligned."""
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    @staticmethod
    def split_plan(k: int, want: int):
        """(k-blocks of the shortest slice, slices) for a requested number of
        slices: at most one slice per 64-wide k-block."""
        num_kb = (k + 63) // 64
        slices = max(1, min(want, num_kb))
        return num_kb // slices, slices

    @staticmethod
    def slices_for(tiles: int, k: int, sms: int, max_waves: int = 3) -> int:
        """How many slices of the inner dimension make ``tiles`` output tiles fill
        the device's SMs best: the fewest slices among those whose last wave of
        CTAs is (nearly) as full as it gets."""
        num_kb = (k + 63) // 64
        best, best_eff = 1, 0.0
        for s in range(1, min(num_kb, max(1, (max_waves * sms) // max(1, tiles))) + 1):
            ctas = tiles * s
            eff = ctas / (-(-ctas // sms) * sms)
            if eff > best_eff + 0.02:
                best, best_eff = s, eff
        return best

    PAIR_TILES = (256, 224, 192, 128)

    def gemm_pair(self, x, w, bias, out, err, bn: int = 256, silu_mul: bool = False,
                  tile_rows: int = 256) -> None:
        """out[M,N] (bf16) = x[M,K] @ w[N,K]^T (+ bias) for many tokens, every
        256 x ``bn`` tile computed by two SMs together (tcgen05 cta_group::2).
        ``silu_mul`` as in ``gemm_tcgen05``.  ``tile_rows`` 512: tiles of 512
        tokens x ``bn`` (192, 224 or 256) features, two accumulators per SM."""
        M, K = x.shape
        N = w.shape[0]
        assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and bn in self.PAIR_TILES
        assert tuple(out.shape) == ((M, N // 2) if silu_mul else (M, N))
        self._check(self.lib.crane_gemm_bf16_pair(
            x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, x.stride(0), w.stride(0),
            out.stride(0), bn, tile_rows, 1 if silu_mul else 0, err.data_ptr(), self._stream(x)), "gemm_pair")

    WIDE_TILES = (256, 224, 192, 160, 128)

    @classmethod
    def tile_width_for(cls, m: int, n: int, sms: int) -> int:
        """The width of the 128 x width output tiles of a many-token product that
        takes the fewest rounds of tiles over the SMs, times the width (plus a
        little per tile); the widest among equals."""
        best, best_cost = 256, None
        for bn in cls.WIDE_TILES:
            tiles = -(-m // 128) * -(-n // bn)
            cost = -(-tiles // sms) * (bn + 16)
            if best_cost is None or cost < best_cost:
                best, best_cost = bn, cost
        return best

    TALL_TILES = (256, 192)

    @classmethod
    def tall_width_for(cls, m: int, n: int, sms: int) -> int:
        """The width of 256 x width tiles on one SM where they beat the 128-row
        tiles of ``tile_width_for``, else 0: a product whose 128-row tiles need a
        second, partly empty round over the SMs and whose 256-row tiles need one
        (measured at 2048 x 3072 x 2048: 27.9 -> 25.1 us in 256 x 192 tiles; the
        factor below is that measurement)."""
        if m <= 128:
            return 0
        bn1 = cls.tile_width_for(m, n, sms)
        best, best_cost = 0, -(-(-(-m // 128) * -(-n // bn1)) // sms) * (bn1 + 16)
        for bn in cls.TALL_TILES:
            tiles = -(-m // 256) * -(-n // bn)
            cost = -(-tiles // sms) * 2 * (bn + 16) * 0.92
            if cost < best_cost:
                best, best_cost = bn, cost
        return best

    PAIR_MIN_FLOPS = 4e10      # below this the pair kernel's set-up outweighs its better feeding

    @classmethod
    def pair_width_for(cls, m: int, n: int, k: int, sms: int) -> int:
        """The tile width for ``gemm_pair``, or 0 where the single-SM kernel is the
        better choice (small products, fewer than 256 rows)."""
        if m < 256 or 2.0 * m * n * k < cls.PAIR_MIN_FLOPS:
            return 0
        best, best_cost = 0, None
        for bn in cls.PAIR_TILES:
            tiles = -(-m // 256) * -(-n // bn)
            cost = -(-tiles // (sms // 2)) * (bn + 16)
            if best_cost is None or cost < best_cost:
                best, best_cost = bn, cost
        return best

    TALL_PAIR_TILES = (256, 224, 192)

    @classmethod
    def pair_plan(cls, m: int, n: int, k: int, sms: int, silu_mul: bool = False):
        """(tile width, tile rows) for ``gemm_pair``, (0, 0) where the single-SM
        kernel is the better choice.

        A model of the time of one round of tiles, in microseconds, fitted to
        measurements of 13 shapes (2048 .. 8192 tokens, inner dimensions 2048 ..
        14336): the operand bytes a CTA moves through its shared memory ((256 +
        width) x 128 bytes per 64-wide k-block for its 128 rows of a 256-row
        tile, (512 + width) x 128 for its 256 rows of a 512-row tile) cost 1.2e-5
        us each, and 128 rows x width x 16 are multiplied in width / 2 clocks;
        the two overlap, not perfectly (a 3-norm).  Tiles of 512 rows move the
        least bytes per product but have no second accumulator to work into while
        the epilogue reads the first, so their epilogue adds to every round: they
        win with a long inner dimension (2048 x 3072 x 8192: 86.6 -> 74.6 us,
        8192^3: 807 -> 740 us) and lose with a short one and with the silu
        epilogue.  Among near-equal costs the wider 256-row tile is taken (it
        runs a little better than the model says)."""
        if not cls.pair_width_for(m, n, k, sms):
            return 0, 0
        pairs = sms // 2

        def norm3(a, b):
            return (a ** 3 + b ** 3) ** (1.0 / 3.0)

        cands = []
        for bn in cls.PAIR_TILES:
            rounds = -(-(-(-m // 256) * -(-n // bn)) // pairs)
            cands.append((rounds * norm3((256 + bn) * k * 1.2e-5, k * bn / 56000.0), bn, 256))
        for bn in cls.TALL_PAIR_TILES:
            rounds = -(-(-(-m // 512) * -(-n // bn)) // pairs)
            epilogue = bn * (0.024 if silu_mul else 0.018)
            cands.append((rounds * (norm3((512 + bn) * k * 1.2e-5, k * bn / 28000.0) + epilogue), bn, 512))
        least = min(c[0] for c in cands)
        near = [c for c in cands if c[0] <= 1.03 * least]
        _, bn, rows = min(near, key=lambda c: (c[2], -c[1]))
        return bn, rows

    def gemm_tcgen05(self, x, w, bias, out, err, split_k: int = 1, swap: bool = False,
                     bn: int = 128, silu_mul: bool = False, prefetch=None, tile_rows: int = 128) -> None:
        """out[M,N] = x[M,K] @ w[N,K]^T (+ bias).  ``swap``: the weight fills the
        128-row side of the MMA and ``bn`` (16..64) covers the tokens.  With
        ``split_k`` > 1 ``out`` is float [slices, M, N] of partial sums.
        ``silu_mul``: w's rows come as 16 gate rows then the 16 up rows of the same
        features, and out[M, N/2] = silu(gate) * up.  ``prefetch``: (address,
        bytes) of what the step's next product will stream, asked into L2 by the
        narrow-tile kernel while it runs (a hint; ignored by the other kernels).
        ``tile_rows`` 256: tiles of 256 tokens x ``bn`` (128, 192 or 256) features
        (bf16 output, no slices, no swap, no silu)."""
        M, K = x.shape
        N = w.shape[0]
        if silu_mul:
            assert out.shape == (M, N // 2) and out.stride(1) == 1 and split_k == 1 and not swap
            ld, stride = out.stride(0), 0
        elif split_k > 1:
            assert out.dtype == torch.float32 and out.dim() == 3 and out.shape[1:] == (M, N)
            ld, stride = out.stride(1), out.stride(0)
        else:
            assert out.shape == (M, N) and out.stride(1) == 1
            ld, stride = out.stride(0), 0
        a, b = (w, x) if swap else (x, w)
        self._check(self.lib.crane_gemm_bf16_tcgen05(
            a.data_ptr(), b.data_ptr(), _ptr(bias), out.data_ptr(), a.shape[0], b.shape[0], K,
            a.stride(0), b.stride(0), ld, bn, tile_rows, 1 if out.dtype == torch.float32 else 0,
            1 if swap else 0, split_k, stride, 1 if silu_mul else 0,
            prefetch[0] if prefetch else None, prefetch[1] if prefetch else 0, err.data_ptr(),
            self._stream(x)), "gemm_tcgen05")

    # ---- attention ------------------------------------------------------
    def paged_attention_simt(self, q, out, k_pool, v_pool, positions, tok_entry, block_table,
                             page_size, nq, nkv, d, window, scale, err) -> None:
        self._check(self.lib.crane_paged_attention_simt(
            _dt(q.dtype), q.data_ptr(), out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
            positions.data_ptr(), tok_entry.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], k_pool.shape[0], page_size, q.shape[0], nq, nkv, d, int(window),
            float(scale), err.data_ptr(), self._stream(q)), "paged_attention_simt")

    @staticmethod
    def decode_splits(entries: int, nkv: int, sms: int, cap: int = 64, max_keys: int = 1 << 30) -> int:
        """Key slices per (request, kv head) of the fused decode attention: enough CTAs to fill
        the device twice over (two fit on an SM), at most ``cap`` (the merge kernel takes 64);
        beyond that, the number of slices that fills the rounds over the SMs best.
        Measured in whole decode steps: 9 to 11 slices lose to 8, which merge themselves in a
        cluster without a second kernel; 33 to 40 lose to 32."""
        ctas, slots = max(1, entries * nkv), 2 * sms
        if ctas > slots:
            # More CTAs than fit at once.  The rounds over the SMs that are full run at the memory's
            # rate; a last round of few CTAs does not (about half the places have to be taken for
            # that), and it is as long as a full one.  Slices make the rounds shorter and the last one
            # fuller; they cost a little themselves (measured: 2 slices 2 %, 4 slices 7 %; 3, a
            # cluster of three, more).  The estimate below follows the measurements at a context of
            # 8,192 and 4 kv heads (ms per step with 1 / 2 / 4 slices): 80 requests 10.9 / 9.3 / 8.7,
            # 96 requests 11.1 / 9.7 / 10.1, 128 requests 12.2 / 12.2 / 13.0, 160 requests 16.7 / 15.6 /
            # 16.1, 192 requests 18.0 / - / 18.9.
            best, best_cost = 1, None
            for s, over in ((1, 1.0), (2, 1.02), (4, 1.07)):
                if s > cap:
                    break
                full, last = divmod(ctas * s, slots)
                cost = (full * slots + (max(last, slots // 2) if last else 0)) / s * over
                if best_cost is None or cost < best_cost:
                    best, best_cost = s, cost
            return best
        splits = max(1, min(cap, 64, slots // ctas))
        if splits > 8 and max_keys <= 2048:
            # few keys: 8 slices, which merge in their cluster, beat more slices and the merge kernel
            # (one request at a context of 256 / 1,024: 1.366 -> 1.284 / 1.380 -> 1.313 ms per step; four
            # requests: 1.440 -> 1.329 / 1.434 -> 1.387 ms; at 4,096 keys more slices win again)
            return 8
        while splits < 8 and splits & (splits - 1) and ctas * splits > 0.85 * slots:
            # 2 to 8 slices are a thread-block cluster, which has to find its places in one GPC: clusters
            # of 3 (5, 6, 7) that would take nearly every place do not all fit at once (24 requests of 4
            # kv heads at a context of 8,192: 288 CTAs in clusters of 3 4.74 ms per step, 192 in clusters
            # of 2 3.57 ms; 20 requests: 240 CTAs in clusters of 3 3.09 ms, 160 in clusters of 2 3.60 ms)
            splits -= 1
        if 8 < splits <= 11:
            return 8
        if 32 < splits <= 40:
            return 32
        return splits

    def decode_attention_supports(self, d: int, nq: int, nkv: int) -> bool:
        self.require_head_size(d)
        return bool(self.lib.crane_paged_decode_attention_supports(d, nq, nkv))

    def paged_decode_attention(self, q, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                               nq, nkv, d, window, scale, n_splits, part_o, part_ml, err) -> None:
        """The entries of exactly one token (bfloat16); entries with more or no
        rows are skipped.  ``part_o`` [entries * nq * n_splits * d] and ``part_ml``
        [entries * nq * n_splits * 2] floats are scratch for n_splits > 1."""
        n_entries = kv_len.shape[0]
        self.require_head_size(d)
        self._check(self.lib.crane_paged_decode_attention(
            q.data_ptr(), out.data_ptr(), _ptr(part_o), _ptr(part_ml), k_pool.data_ptr(),
            v_pool.data_ptr(), cu_q.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], k_pool.shape[0], page_size, n_entries, nq, nkv, d, int(window),
            float(scale), int(n_splits), err.data_ptr(), self._stream(q)), "paged_decode_attention")

    def prefill_attention_supports(self, d: int, nq: int, nkv: int) -> bool:
        self.require_head_size(d)
        return bool(self.lib.crane_paged_prefill_attention_supports(d, nq, nkv))

    def paged_prefill_attention(self, q, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                                total_q_tiles, nq, nkv, d, window, scale, err, skip_single=False) -> None:
        """Any mix of portions and single tokens (bfloat16).  ``total_q_tiles``:
        the sum over the entries of ceil(tokens / 64), or more.  ``skip_single``:
        entries of exactly one token are left to the decode kernel."""
        self.require_head_size(d)
        self._check(self.lib.crane_paged_prefill_attention(
            q.data_ptr(), out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(),
            kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1], k_pool.shape[0],
            page_size, kv_len.shape[0], int(total_q_tiles), nq, nkv, d, int(window), float(scale),
            1 if skip_single else 0, err.data_ptr(), self._stream(q)), "paged_prefill_attention")

    def prefill_attention_tc_supports(self, d: int, nq: int, nkv: int, page_size: int) -> bool:
        return bool(self.lib.crane_prefill_attention_tc_supports(d, nq, nkv, page_size))

    def prefill_attention_tc(self, q, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                             total_q_tiles, nq, nkv, d, window, scale, err, skip_single=False) -> None:
        """Flash attention on tcgen05 (head size 128).  ``total_q_tiles``: the sum
        over the entries of ceil(tokens / 128), or more.  ``skip_single`` as in
        ``paged_prefill_attention``."""
        self._check(self.lib.crane_prefill_attention_tc(
            q.data_ptr(), out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(),
            kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1], k_pool.shape[0],
            page_size, kv_len.shape[0], q.shape[0], int(total_q_tiles), nq, nkv, d, int(window),
            float(scale), 1 if skip_single else 0, err.data_ptr(), self._stream(q)), "prefill_attention_tc")

    def paged_decode_attention_fused(self, qkv: Act, qkv_cols, has_kv, cos, sin, q_norm_w, k_norm_w,
                                     eps, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                                     nq, nkv, d, window, scale, n_splits, part_o, part_ml, err,
                                     rope=None) -> None:
        """One token per entry, straight from the q/k/v product: rotary encoding,
        per-head norm, cache write and attention in one kernel, then the merge of
        the key slices.  ``rope`` as in ``rope_norm_cache``."""
        rd, inter, first, off = rope or (d, False, False, 0.0)
        whole, parts, n_parts, stride = _split(qkv)
        n_entries = kv_len.shape[0]
        self.require_head_size(d)
        self._check(self.lib.crane_paged_decode_attention_fused(
            whole, parts, n_parts, stride, qkv_cols, 1 if has_kv else 0, 1 if cos is not None else 0,
            _ptr(cos), _ptr(sin), cos.shape[0] if cos is not None else 0, _ptr(q_norm_w),
            _ptr(k_norm_w), float(eps), out.data_ptr(), _ptr(part_o), _ptr(part_ml),
            k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(), kv_len.data_ptr(),
            block_table.data_ptr(), block_table.shape[1], k_pool.shape[0], page_size, n_entries, nq,
            nkv, d, int(window), float(scale), int(n_splits), int(rd), 1 if inter else 0,
            1 if first else 0, float(off), err.data_ptr(), self._stream(out)),
            "paged_decode_attention_fused")

    # ---- sampling -------------------------------------------------------
    def repetition_penalty(self, logits, context, ctx_len, penalty) -> None:
        rows, vocab = logits.shape
        self._check(self.lib.crane_repetition_penalty(
            logits.data_ptr(), logits.stride(0), rows, vocab, context.data_ptr(), context.stride(0),
            ctx_len.data_ptr(), penalty.data_ptr(), self._stream(logits)), "repetition_penalty")

    def sample(self, logits, out, temperature=None, top_k=None, top_p=None, seed=None,
               counter=None) -> None:
        rows, vocab = logits.shape
        if temperature is not None and (seed is None or counter is None):
            raise KernelError("sampling with a temperature needs seed and counter per row")
        self._check(self.lib.crane_sample(
            logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_k),
            _ptr(top_p), _ptr(seed), _ptr(counter), out.data_ptr(), self._stream(logits)), "sample")


_kernels: Optional[Kernels] = None


def get_kernels(head_sizes=()) -> Kernels:
    """The process's kernels.  ``head_sizes``: head sizes that will be needed (a
    model's), so that a library compiled at this first call holds them at once."""
    global _kernels
    if _kernels is None:
        _kernels = Kernels(head_sizes)
    else:
        for d in head_sizes:
            _kernels.require_head_size(d)
    return _kernels
