"""What parts run with: the device, the model dtype, the kernels, long-lived
buffers, the device-side error word and the matrix product.

Matrix products: on the true 32-bit path always the FP32-core kernel of this
package (no tensor cores, so no reduced-precision mode can slip in).  On the
bfloat16 path the tcgen05 kernel of this package where it takes the shape, and
otherwise the vendor's library product, which is also what the reference uses
for every product (Candle's matmul, crane-core/src/models/hunyuan_dense/
modeling.rs:517-522, 645, 716, 732).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..kernels import Act, KernelError, Partials, get_kernels
from .base import Workspace

_ERR_NAMES = {1: "a token id outside the vocabulary", 2: "a block-table entry outside the page pool",
              4: "a position outside the rotary table", 8: "a bounded wait on the device ran out",
              16: "a state slot outside the pool"}


class DeviceFault(RuntimeError):
    pass


class Runtime:
    def __init__(self, device, dtype: torch.dtype, max_rows: int, max_decode_rows: int = 64, head_sizes=()):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError("the engine runs on a CUDA device only; there is no CPU path")
        if dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"model dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.exact = dtype == torch.float32
        self.kernels = get_kernels(head_sizes)       # (the model's head sizes: compiled at this first call if need be)
        self.ws = Workspace(self.device, max_rows)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.max_rows = max_rows
        self.max_decode_rows = max_decode_rows     # most single-token entries of a step
        self.launches = 0            # kernels of this package launched (a count for reports)
        self.use_tcgen05 = os.environ.get("CRANE_BF16_GEMM", "tcgen05") != "library"
        self.use_tc_attention = os.environ.get("CRANE_PREFILL_ATTENTION", "tcgen05") != "mma"
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        # Up to this many tokens a product streams the weights through the MMA's 128-row side
        # with the inner dimension in slices (partial sums), which keeps every SM busy on a
        # product too small to fill them with whole tiles; measured against the many-token
        # kernel at batch 96..256: 5 to 15 % faster steps.
        self.split_rows = 256
        self.silu_rows = 64          # above this the gate/up product takes the kernel with the fused silu-mul
        # The weights of a step's products in the order of use, learnt from the first steps: the products
        # of a single token are told what the next one will stream and ask for it into L2 at once
        # (CRANE_L2_PREFETCH=0: no hints).  A hint is given where the running product's weights and
        # the next one's together are at most this much: they must fit L2 beside each other.
        self.prefetch_cap = int(os.environ.get("CRANE_L2_PREFETCH_MB", "80")) << 20
        self.use_prefetch = os.environ.get("CRANE_L2_PREFETCH", "1") != "0"
        self._w_order = []           # (address, bytes) of the step's product weights, in order
        self._w_pos = 0

    # ---- device error word ---------------------------------------------
    def check_errors(self) -> None:
        """Reads the error word (synchronises) and raises if a kernel set it."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            what = [n for bit, n in _ERR_NAMES.items() if code & bit]
            raise DeviceFault("a kernel reported: " + "; ".join(what or [f"code {code}"]))

    # ---- what the next product will stream ---------------------------
    def begin_step(self) -> None:
        """A model's forward pass begins: its products come in the learnt order again."""
        self._w_pos = 0

    def _next_weights(self, w: torch.Tensor):
        """Notes that ``w`` is streamed now; returns (address, bytes) of the weights
        that followed it in the step before, or None while the order is learnt."""
        if not self.use_prefetch:
            return None
        order, pos, ptr = self._w_order, self._w_pos, w.data_ptr()
        self._w_pos = pos + 1
        if pos < len(order) and order[pos][0] == ptr:
            nxt = order[(pos + 1) % len(order)]
            # both products' weights have to lie in L2 side by side, or the running one's stream
            # throws out what was asked for (measured: with hints cut off at 48 MB, single tokens at
            # Hunyuan-4B and 7B sizes, whose products stream 100 to 235 MB, lost 11 %)
            if order[pos][1] + nxt[1] > self.prefetch_cap:
                return None
            return nxt
        del order[pos:]                                   # another path than last time: learn it
        order.append((ptr, w.numel() * w.element_size()))
        return None

    # ---- matrix product -------------------------------------------------
    def linear(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], name: str,
               out_dtype: Optional[torch.dtype] = None, cap: Optional[int] = None,
               hint_next: bool = True) -> Act:
        """x[M,K] @ w[N,K]^T (+ bias[N], float) -> [M,N] in ``out_dtype`` (the
        model dtype unless stated).  ``hint_next`` False: this product does not
        ask for the next product's weights (its caller streams so much between
        the two that they would not stay in L2)."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or self.dtype
        out = self.ws.get(name, M, N, out_dtype, cap)
        if self.exact:
            self.kernels.gemm_simt(x, w, bias, out)
            self.launches += 1
            return out
        return self._linear_bf16(x, w, bias, out, hint_next)

    def linear_silu_mul(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
        """out[M, N/2] = silu(gate) * up of x @ w^T in one kernel, for w whose rows
        alternate 16 gate / 16 up.  False if this step's shape has no such kernel
        (few tokens, where the product is computed in slices)."""
        M = x.shape[0]
        if self.exact or not self.use_tcgen05 or M <= self.silu_rows or not self.kernels.tcgen05_takes(x, w):
            return False
        if w.shape[0] % 32 or out.stride(0) % 8 or out.data_ptr() % 16:
            return False
        pair, rows = self.kernels.pair_plan(M, w.shape[0], x.shape[1], self.num_sms, silu_mul=True)
        if pair:
            self.kernels.gemm_pair(x, w, None, out, self.err, bn=pair, silu_mul=True, tile_rows=rows)
        else:
            self.kernels.gemm_tcgen05(x, w, None, out, self.err,
                                      bn=self.kernels.tile_width_for(M, w.shape[0], self.num_sms), silu_mul=True)
        self.launches += 1
        return True

    def _linear_bf16(self, x, w, bias, out, hint_next: bool = True) -> Act:
        k = self.kernels
        M, K = x.shape
        N = w.shape[0]
        if self.use_tcgen05 and k.tcgen05_takes(x, w):
            if M <= self.split_rows:
                # few tokens: the weight rows fill the MMA's 128-wide side (the tokens its 16 to
                # 256 wide side), and the inner dimension is cut into slices until every SM has a
                # tile to stream
                bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
                tiles = (N + 127) // 128
                # at most 8: the consumers of partial sums fetch eight slices at a time
                slices = min(k.slices_for(tiles, K, self.num_sms), 8)
                nxt = self._next_weights(w) if w.is_contiguous() else None
                # Measured in whole decode steps (Hunyuan-1.8B sizes): a single token gains 2.4 % at a
                # context of 2,048 and 4.6 % at 8,192; from two tokens on the hints cost 1 to 4 % (the
                # demand loads of the running product and the requests for the next one then share
                # a memory system that is already busier), so only a single token gives them.
                if not hint_next or M != 1:
                    nxt = None
                if slices > 1:
                    parts = self.ws.get("splitk:" + str(N), slices * self.split_rows, N,
                                        torch.float32, cap=slices * self.split_rows)
                    parts = parts[:slices * M].view(slices, M, N)
                    k.gemm_tcgen05(x, w, bias, parts, self.err, split_k=slices, swap=True, bn=bn, prefetch=nxt)
                    self.launches += 1
                    if out.dtype == torch.float32:
                        k.sum_parts(Partials(parts), out)      # float logits: the slices added in order
                        self.launches += 1
                        return out
                    return Partials(parts)
                k.gemm_tcgen05(x, w, bias, out, self.err, swap=True, bn=bn, prefetch=nxt)
            else:
                pair, pair_rows = k.pair_plan(M, N, K, self.num_sms) if out.dtype == torch.bfloat16 else (0, 0)
                bn = k.tile_width_for(M, N, self.num_sms)
                if not pair and out.dtype == torch.bfloat16 and M <= 4 * self.split_rows:
                    # A few hundred tokens and a long inner dimension (the down projection): 128 x 128
                    # tiles are too few for the SMs and re-read the operands too often.  Tiles of 128
                    # features x 256 tokens over slices of the inner dimension do better (measured
                    # at 2048 features x 6144: 31 -> 18 us at 512 tokens, 33 -> 26 us at 1024).
                    tiles = -(-N // 128) * -(-M // 256)
                    slices = min(self.num_sms // tiles, 4)
                    if slices >= 2 and K // slices >= 1536:
                        # at most 4 slices of 4 * split_rows tokens: the buffer never has to grow
                        parts = self.ws.get("splitk_wide:" + str(N), slices * M, N, torch.float32,
                                            cap=16 * self.split_rows).view(slices, M, N)
                        k.gemm_tcgen05(x, w, bias, parts, self.err, split_k=slices, swap=True, bn=256)
                        self.launches += 1
                        return Partials(parts)
                if out.dtype == torch.float32 and bn not in (128, 256):
                    bn = 256 if N >= 2048 else 128
                tall = 0 if pair or out.dtype != torch.bfloat16 else k.tall_width_for(M, N, self.num_sms)
                if pair:
                    k.gemm_pair(x, w, bias, out, self.err, bn=pair, tile_rows=pair_rows)   # two SMs per tile
                elif tall:
                    k.gemm_tcgen05(x, w, bias, out, self.err, bn=tall, tile_rows=256)
                else:
                    k.gemm_tcgen05(x, w, bias, out, self.err, bn=bn)
            self.launches += 1
            return out
        if out.dtype == torch.bfloat16 and bias is None:
            torch.mm(x, w.t(), out=out)
            return out
        # with a bias, or for a float result from bfloat16 operands: the FP32-core kernel, which adds
        # the float bias to the float accumulator and rounds once, as the tcgen05 kernels do
        k.gemm_simt(x, w, bias, out)
        self.launches += 1
        return out
