"""Helpers of the GPU tests: a paged cache laid out from dense keys/values with
pages in random order, and step metadata for the attention kernels."""
import numpy as np
import torch

DEV = "cuda:0"


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    want = want.to(torch.float64)
    return float((got.to(torch.float64) - want).abs().max() / want.abs().max().clamp_min(1e-30))


def paged_cache(ks, vs, page_size, dtype, extra_pages=3, seed=0):
    """ks, vs: per request [T_i, nkv, d] float tensors.  Returns k_pool, v_pool
    [pages, nkv, page_size, d] filled with garbage except where the requests'
    tokens live, and the block table [n, max_blocks] (unused entries -1)."""
    rng = np.random.default_rng(seed)
    nkv, d = ks[0].shape[1], ks[0].shape[2]
    blocks = [(k.shape[0] + page_size - 1) // page_size for k in ks]
    total = sum(blocks) + extra_pages
    order = rng.permutation(total)
    k_pool = torch.randn(total, nkv, page_size, d, device=DEV).mul_(50.0)    # garbage must never be read
    v_pool = torch.randn(total, nkv, page_size, d, device=DEV).mul_(50.0)
    table = -torch.ones(len(ks), max(blocks), dtype=torch.int32)
    nxt = 0
    for i, (k, v) in enumerate(zip(ks, vs)):
        for b in range(blocks[i]):
            page = int(order[nxt]); nxt += 1
            table[i, b] = page
            n = min(page_size, k.shape[0] - b * page_size)
            k_pool[page, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1).to(DEV)
            v_pool[page, :, :n] = v[b * page_size:b * page_size + n].transpose(0, 1).to(DEV)
    return k_pool.to(dtype), v_pool.to(dtype), table.to(DEV)


def attention_reference(q, k, v, pos, window=0, scale=None):
    """One query row q [nq, d] at position pos over k, v [T, nkv, d] in float64."""
    nq, d = q.shape
    nkv = k.shape[1]
    scale = scale if scale is not None else d ** -0.5
    lo = max(0, pos - window + 1) if window > 0 else 0
    out = torch.zeros(nq, d, dtype=torch.float64)
    for h in range(nq):
        g = h // (nq // nkv)
        s = (k[lo:pos + 1, g].double() @ q[h].double()) * scale
        p = torch.softmax(s, dim=0)
        out[h] = p @ v[lo:pos + 1, g].double()
    return out
