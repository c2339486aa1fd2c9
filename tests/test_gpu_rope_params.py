"""The parameters of the attention mixer that say how heads are rotated and
normalised: rotated width, pairing, norm before or after the rotation, (1 + w)
norm weights.  Hunyuan Dense uses the defaults; another architecture sets them
in its PartSpec and needs no change to a kernel.  Every value other than the
default against a NumPy restatement written here: the rotary kernel alone, the
fused decode kernel against the separate kernels, and the mixer part whole, in
portions and token by token."""
import math

import numpy as np
import pytest
import torch

import plain_hunyuan as ph
from gpu_helpers import DEV, paged_cache, rel_err

pytestmark = pytest.mark.gpu

VARIANTS = [dict(), dict(rotary_dim=0.5), dict(pairing="interleaved"), dict(order="before_rope"),
            dict(offset=1.0), dict(rotary_dim=0.25, pairing="interleaved", order="before_rope", offset=1.0)]


@pytest.fixture(scope="module")
def K():
    from crane_b200.kernels import get_kernels
    return get_kernels()


@pytest.fixture()
def err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def rotate_restated(x, positions, inv_freq, rotary_dim, interleaved):
    """x [T, heads, d] float64; the first rotary_dim elements of every head are
    rotated by angle p * inv_freq[i]: element pair (i, i + rotary_dim/2), or
    (2i, 2i + 1) when interleaved; the rest passes through."""
    out = x.copy()
    hr = rotary_dim // 2
    ang = positions.astype(np.float32)[:, None] * inv_freq[None, :].astype(np.float32)     # float32 product
    c, s = np.cos(ang.astype(np.float64))[:, None, :], np.sin(ang.astype(np.float64))[:, None, :]
    ia = np.arange(hr) * 2 if interleaved else np.arange(hr)
    ib = ia + 1 if interleaved else ia + hr
    a, b = x[..., ia], x[..., ib]
    out[..., ia] = a * c - b * s
    out[..., ib] = b * c + a * s
    return out


def norm_restated(x, w, eps, offset):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * (offset + w)


def heads_restated(x, positions, inv_freq, w, eps, rotary_dim, interleaved, norm_first, offset):
    if w is not None and norm_first:
        x = norm_restated(x, w, eps, offset)
    x = rotate_restated(x, positions, inv_freq, rotary_dim, interleaved)
    if w is not None and not norm_first:
        x = norm_restated(x, w, eps, offset)
    return x


def variant(d, v):
    rd = int(d * v.get("rotary_dim", 1.0)) // 2 * 2
    return rd, v.get("pairing", "half") == "interleaved", v.get("order", "after_rope") == "before_rope", v.get("offset", 0.0)


def tables(rd, n):
    inv = ph.rope_inv_freq(rd, 10000.0, 3.0)
    ang = (np.arange(n, dtype=np.float32)[:, None] * inv[None, :].astype(np.float32)).astype(np.float64)
    return inv, torch.from_numpy(np.cos(ang).astype(np.float32)).to(DEV), torch.from_numpy(np.sin(ang).astype(np.float32)).to(DEV)


@pytest.mark.parametrize("v", VARIANTS)
@pytest.mark.parametrize("dtype,d,nq,nkv,n_tok", [(torch.float32, 48, 3, 1, 13), (torch.bfloat16, 128, 6, 2, 40),
                                                  (torch.bfloat16, 64, 4, 2, 9), (torch.float32, 16, 2, 2, 5)])
def test_rotary_kernel_with_parameters(K, err, v, dtype, d, nq, nkv, n_tok):
    rd, inter, first, off = variant(d, v)
    eps, ps = 1e-5, 16
    torch.manual_seed(d + rd)
    positions = np.arange(7, 7 + n_tok)
    cols = (nq + 2 * nkv) * d
    qkv = torch.randn(n_tok, cols, device=DEV).to(dtype)
    blocks = (7 + n_tok + ps - 1) // ps
    table = torch.arange(blocks, dtype=torch.int32, device=DEV).flip(0).view(1, blocks).contiguous()
    k_pool = torch.zeros(blocks, nkv, ps, d, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    inv, cos, sin = tables(rd, 256)
    qw, kw = (1 + 0.1 * torch.randn(d)).to(DEV), (1 + 0.1 * torch.randn(d)).to(DEV)
    q_out = torch.empty(n_tok, nq * d, device=DEV, dtype=dtype)
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    K.rope_norm_cache(qkv, cols, dtype, i32(positions), i32(np.zeros(n_tok)), table, cos, sin, qw, kw, eps,
                      q_out, k_pool, v_pool, ps, nq, nkv, d, True, True, err, rope=(rd, inter, first, off))
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    x = qkv.double().cpu().numpy()
    q = heads_restated(x[:, :nq * d].reshape(n_tok, nq, d), positions, inv, qw.double().cpu().numpy(), eps, rd,
                       inter, first, off)
    k = heads_restated(x[:, nq * d:(nq + nkv) * d].reshape(n_tok, nkv, d), positions, inv,
                       kw.double().cpu().numpy(), eps, rd, inter, first, off)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert rel_err(q_out.cpu().view(n_tok, nq, d), torch.from_numpy(q)) < tol
    tab = table.cpu().numpy()[0]
    for t in range(n_tok):
        p = int(positions[t])
        assert rel_err(k_pool[int(tab[p // ps]), :, p % ps].cpu(), torch.from_numpy(k[t])) < tol
        assert torch.equal(v_pool[int(tab[p // ps]), :, p % ps].cpu(), qkv[t, (nq + nkv) * d:].view(nkv, d).cpu())
    if not v:
        # the defaults are the reference's convention, stated once more by the plain implementation
        a = ph.rope_angles(positions, inv)
        want = ph.rms_norm(ph.apply_rope(x[:, :nq * d].reshape(n_tok, nq, d), a), qw.double().cpu().numpy(), eps)
        assert np.abs(want - q).max() < 1e-12


@pytest.mark.parametrize("v", VARIANTS[1:])
@pytest.mark.parametrize("d,nq,nkv,page_size,splits,parts", [(128, 16, 4, 64, 8, 0), (128, 8, 2, 32, 12, 3),
                                                             (64, 8, 8, 16, 3, 0), (80, 10, 5, 16, 1, 2)])
def test_fused_decode_with_parameters_equals_the_separate_kernels(K, err, v, d, nq, nkv, page_size, splits, parts):
    from crane_b200.kernels import Partials
    rd, inter, first, off = variant(d, v)
    rope = (rd, inter, first, off)
    torch.manual_seed(d + splits)
    lens = [1, 32, 33, 64, 65, 700]
    n = len(lens)
    ks = [torch.randn(m, nkv, d).bfloat16().float() for m in lens]
    vs = [torch.randn(m, nkv, d).bfloat16().float() for m in lens]
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, torch.bfloat16, seed=splits)
    cols = (nq + 2 * nkv) * d
    qkv = torch.randn(n, cols, device=DEV)
    if parts:
        p = torch.randn(parts, n, cols, device=DEV)
        p[0] += qkv - p.sum(0)
        whole = p[0].clone()
        for i in range(1, parts):
            whole += p[i]
        src, whole = Partials(p), whole.bfloat16()
    else:
        src = whole = qkv.bfloat16()
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    pos, ent, cu, kvl = i32([m - 1 for m in lens]), i32(list(range(n))), i32(list(range(n + 1))), i32(lens)
    _, cos, sin = tables(rd, 1100)
    qw, kw = (1 + 0.1 * torch.randn(d)).to(DEV), (1 + 0.1 * torch.randn(d)).to(DEV)
    k1, v1 = k_pool.clone(), v_pool.clone()
    q = torch.empty(n, nq * d, device=DEV, dtype=torch.bfloat16)
    K.rope_norm_cache(whole, cols, torch.bfloat16, pos, ent, table, cos, sin, qw, kw, 1e-5, q, k1, v1, page_size,
                      nq, nkv, d, True, True, err, rope=rope)
    want = torch.empty_like(q)
    part_o = torch.empty(n * nq * splits * d, device=DEV)
    part_ml = torch.empty(n * nq * splits * 2, device=DEV)
    K.paged_decode_attention(q, want, k1, v1, cu, kvl, table, page_size, nq, nkv, d, 0, d ** -0.5, splits,
                             part_o, part_ml, err)
    k2, v2 = k_pool.clone(), v_pool.clone()
    got = torch.full_like(q, 9.0)
    K.paged_decode_attention_fused(src, cols, True, cos, sin, qw, kw, 1e-5, got, k2, v2, cu, kvl, table, page_size,
                                   nq, nkv, d, 0, d ** -0.5, splits, part_o, part_ml, err, rope=rope)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.equal(k2, k1) and torch.equal(v2, v1)
    assert rel_err(got, want.double()) < 4e-3


@pytest.mark.parametrize("v", VARIANTS[1:])
@pytest.mark.parametrize("dtype,d", [(torch.float32, 32), (torch.bfloat16, 128), (torch.bfloat16, 64)])
def test_attention_part_with_parameters(v, dtype, d):
    """The mixer part built from a PartSpec that sets the parameters: a whole
    sequence, the same in two portions, and its last tokens one by one (the
    fused decode kernel on the bfloat16 path), against the restatement."""
    from test_gpu_parts import build, make_ctx, np64, runtime, whole
    from crane_b200.config import PartSpec
    from crane_b200.parts import LayerCache
    rd, inter, first, off = variant(d, v)
    nq, nkv, h, T, ps, eps = 4, 2, 72, 45, 16, 1e-5
    rt = runtime(dtype)
    torch.manual_seed(d + rd)
    pos_spec = PartSpec("position", "rope", {"head_dim": d, "rotary_dim": rd, "theta": 10000.0, "alpha": 3.0,
                                             "max_positions": 4096})
    spec = PartSpec("mixer", "gqa_attention", {
        "hidden_size": h, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "bias": False, "qk_norm": True,
        "qk_norm_eps": eps, "window": 0, "own_kv": True, "position": pos_spec, "rotary_dim": rd,
        "rope_pairing": "interleaved" if inter else "half",
        "qk_norm_order": "before_rope" if first else "after_rope", "qk_norm_offset": off}, "a.")
    t = {"a.q_proj.weight": 0.15 * torch.randn(nq * d, h), "a.k_proj.weight": 0.15 * torch.randn(nkv * d, h),
         "a.v_proj.weight": 0.15 * torch.randn(nkv * d, h), "a.o_proj.weight": 0.15 * torch.randn(h, nq * d),
         "a.query_layernorm.weight": (0.0 if off else 1.0) + 0.1 * torch.randn(d),
         "a.key_layernorm.weight": (0.0 if off else 1.0) + 0.1 * torch.randn(d)}
    if dtype == torch.bfloat16:
        t = {k: (x.bfloat16().float() if x.dim() == 2 else x) for k, x in t.items()}
    part = build(spec, dict(t), rt)
    x = torch.randn(T, h, device=DEV).to(dtype)
    # the restatement of the layer
    w = {k: np64(x_) for k, x_ in t.items()}
    xs = np64(x)
    inv = ph.rope_inv_freq(rd, 10000.0, 3.0)
    positions = np.arange(T)
    q = heads_restated(ph.linear(xs, w["a.q_proj.weight"]).reshape(T, nq, d), positions, inv,
                       w["a.query_layernorm.weight"], eps, rd, inter, first, off)
    k = heads_restated(ph.linear(xs, w["a.k_proj.weight"]).reshape(T, nkv, d), positions, inv,
                       w["a.key_layernorm.weight"], eps, rd, inter, first, off)
    vv = ph.linear(xs, w["a.v_proj.weight"]).reshape(T, nkv, d)
    want = torch.from_numpy(ph.linear(ph.causal_attention(q, k, vv), w["a.o_proj.weight"]))
    need = part.cache_need()

    def cache():
        shape = (6, nkv, ps, d)
        return LayerCache(need, 0, torch.full(shape, 30.0, device=DEV, dtype=dtype),
                          torch.full(shape, 30.0, device=DEV, dtype=dtype), ps)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    rows = [[4, 1, 5, 2]]
    c = cache()
    out = whole(part.forward(x, make_ctx(rt, [(0, T)], ps, 6, 4, rows), c, rt), dtype)
    assert rel_err(out.cpu(), want) < tol
    c = cache()
    outs = [whole(part.forward(x[:23], make_ctx(rt, [(0, 23)], ps, 6, 4, rows), c, rt), dtype).clone(),
            whole(part.forward(x[23:40], make_ctx(rt, [(23, 17)], ps, 6, 4, rows), c, rt), dtype).clone()]
    for i in range(40, T):
        outs.append(whole(part.forward(x[i:i + 1], make_ctx(rt, [(i, 1)], ps, 6, 4, rows), c, rt), dtype).clone())
    assert rel_err(torch.cat(outs).cpu(), want) < tol
    rt.check_errors()
