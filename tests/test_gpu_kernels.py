"""Each kernel alone against a plain float64 computation of the same formula,
at sizes other than the tiny models': odd widths, head sizes in steps of 16,
vocabularies that are no power of two."""
import math

import numpy as np
import pytest
import torch

import plain_hunyuan as ph
from gpu_helpers import DEV, attention_reference, paged_cache, rel_err

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-6, torch.bfloat16: 1e-2}


def acc_tol(k):
    """Rounding of a float accumulation over k products, relative to the largest
    result: a few times sqrt(k) * 2^-24 (a wrong operand shows as 1e-3 or more)."""
    return max(2e-6, 6 * math.sqrt(k) * 2.0 ** -24)


@pytest.fixture(scope="module")
def K():
    from crane_b200.kernels import get_kernels
    return get_kernels()


@pytest.fixture()
def err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(100, 301), (2048, 1000)])
def test_embed_gather(K, err, dtype, hidden, vocab):
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    tokens = torch.tensor([0, vocab - 1, 5, 5, 17], dtype=torch.int32, device=DEV)
    x = torch.zeros(5, hidden, device=DEV)
    K.embed_gather(tokens, table, x, err)
    assert torch.equal(x, table[tokens.long()].float()) and int(err.item()) == 0
    bad = torch.tensor([vocab], dtype=torch.int32, device=DEV)
    K.embed_gather(bad, table, x[:1], err)
    assert int(err.item()) == 1                      # reported, not read


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [96, 2048, 4100])
def test_add_rmsnorm(K, dtype, hidden):
    n, eps = 7, 1e-5
    x = torch.randn(n, hidden, device=DEV)
    delta = torch.randn(n, hidden, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    want_x = x.double() + delta.double()
    want = torch.from_numpy(ph.rms_norm(want_x.cpu().numpy(), w.double().cpu().numpy(), eps))
    out = torch.empty(n, hidden, device=DEV, dtype=dtype)
    x1 = x.clone()
    K.add_rmsnorm(x1, delta, w, eps, out)
    assert rel_err(x1.cpu(), want_x.cpu()) < 1e-6          # the residual itself stays float
    assert rel_err(out.cpu(), want) < TOL[dtype]
    # norm only
    K.add_rmsnorm(x.clone(), None, w, eps, out)
    assert rel_err(out.cpu(), torch.from_numpy(ph.rms_norm(x.double().cpu().numpy(), w.double().cpu().numpy(), eps))) < TOL[dtype]
    # chosen rows: x must stay as it was
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    x2 = x.clone()
    out3 = torch.empty(3, hidden, device=DEV, dtype=dtype)
    K.add_rmsnorm(x2, delta, w, eps, out3, rows)
    assert torch.equal(x2, x) and rel_err(out3.cpu(), want[[5, 0, 5]]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(3, 10000), (64, 16384), (9, 32768), (2, 8200)])
def test_add_rmsnorm_of_rows_wider_than_8192(K, dtype, rows, hidden):
    """16 or 32 elements per thread at up to 1024 threads: the kernel must fit a
    block of that size (it once asked for more registers than such a block has)."""
    torch.manual_seed(hidden)
    x0 = torch.randn(rows, hidden, device=DEV) * 2
    delta = torch.randn(rows, hidden, device=DEV).to(dtype)
    w = torch.rand(hidden, device=DEV) + 0.5
    x = x0.clone()
    out = torch.empty(rows, hidden, device=DEV, dtype=dtype)
    K.add_rmsnorm(x, delta, w, 1e-5, out)
    want_x = x0 + delta.float()
    assert torch.equal(x, want_x)
    want = want_x.double() * torch.rsqrt((want_x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    assert rel_err(out, want) < (2e-6 if dtype == torch.float32 else 5e-3)
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, hidden, device=DEV, dtype=dtype)
    K.add_rmsnorm(x, None, w, 1e-5, out2, idx)
    assert rel_err(out2, want[[rows - 1, 0]]) < (2e-6 if dtype == torch.float32 else 5e-3)


def test_a_refused_launch_does_not_fail_the_next_one(K):
    from crane_b200.kernels import KernelError
    x = torch.randn(2, 40000, device=DEV)                      # wider than the norm kernels take
    with pytest.raises(KernelError):
        K.add_rmsnorm(x, None, torch.ones(40000, device=DEV), 1e-5, torch.empty_like(x))
    y = torch.randn(2, 64, device=DEV)
    out = torch.empty_like(y)
    K.add_rmsnorm(y, None, torch.ones(64, device=DEV), 1e-5, out)
    assert rel_err(out, y.double() * torch.rsqrt((y.double() ** 2).mean(-1, keepdim=True) + 1e-5)) < 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_rmsnorm_from_partial_sums(K, dtype):
    from crane_b200.kernels import Partials
    n, hidden = 5, 300
    x = torch.randn(n, hidden, device=DEV)
    parts = torch.randn(3, n, hidden, device=DEV)
    w = torch.ones(hidden, device=DEV)
    whole = parts.sum(0).to(dtype)
    a, b = torch.empty(n, hidden, device=DEV, dtype=dtype), torch.empty(n, hidden, device=DEV, dtype=dtype)
    xa, xb = x.clone(), x.clone()
    K.add_rmsnorm(xa, Partials(parts), w, 1e-6, a)
    K.add_rmsnorm(xb, whole, w, 1e-6, b)
    assert rel_err(a, b.float()) < TOL[dtype] and rel_err(xa, xb) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(300, 2048), (257, 768), (2048, 256)])
def test_add_rmsnorm_many_rows_a_warp_per_row(K, dtype, rows, hidden):
    """Many rows of a length that divides by 256 take the kernel with a warp per row."""
    torch.manual_seed(rows)
    x0 = torch.randn(rows, hidden, device=DEV) * 2
    delta = torch.randn(rows, hidden, device=DEV).to(dtype)
    w = torch.rand(hidden, device=DEV) + 0.5
    for d in (delta, None):
        x = x0.clone()
        out = torch.empty(rows, hidden, device=DEV, dtype=dtype)
        K.add_rmsnorm(x, d, w, 1e-5, out)
        want_x = x0 + (d.float() if d is not None else 0)
        assert torch.equal(x, want_x)
        want = want_x.double() * torch.rsqrt((want_x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
        assert rel_err(out, want) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,parts", [(1, 2048, 9), (8, 2048, 0), (33, 4096, 6), (64, 176, 3)])
def test_add_rmsnorm_few_rows_in_clusters(K, dtype, rows, hidden, parts):
    """Few rows of a length that divides by 16 take the kernel that shares a row
    among the CTAs of a cluster: same result as the plain formula, from a whole
    product and from partial sums."""
    from crane_b200.kernels import Partials
    torch.manual_seed(rows + hidden)
    x0 = torch.randn(rows, hidden, device=DEV) * 3
    w = torch.rand(hidden, device=DEV) + 0.5
    if parts:
        cut = torch.randn(parts, rows, hidden, device=DEV)
        total = cut[0].clone()
        for i in range(1, parts):
            total += cut[i]
        delta, dval = Partials(cut), total.to(dtype).float()
    else:
        delta = torch.randn(rows, hidden, device=DEV).to(dtype)
        dval = delta.float()
    x = x0.clone()
    out = torch.empty(rows, hidden, device=DEV, dtype=dtype)
    K.add_rmsnorm(x, delta, w, 1e-5, out)
    want_x = x0 + dval
    assert torch.equal(x, want_x)
    want = want_x.double() * torch.rsqrt((want_x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    assert rel_err(out, want) < (1e-6 if dtype == torch.float32 else 5e-3)
    out2 = torch.empty_like(out)
    K.add_rmsnorm(x, None, w, 1e-5, out2)                     # nothing to add: x stays
    assert torch.equal(x, want_x) and rel_err(out2, want) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(K, dtype):
    n, inter = 9, 353
    gu = (3 * torch.randn(n, 2 * inter, device=DEV)).to(dtype)
    out = torch.empty(n, inter, device=DEV, dtype=dtype)
    K.silu_mul(gu, out)
    g, u = gu[:, :inter].double().cpu().numpy(), gu[:, inter:].double().cpu().numpy()
    assert rel_err(out.cpu(), torch.from_numpy(ph.silu(g) * u)) < TOL[dtype]
    # the same with gate and up columns in alternating blocks of 16
    n2, i2 = 5, 352
    gate, up = (2 * torch.randn(n2, i2, device=DEV)).to(dtype), (2 * torch.randn(n2, i2, device=DEV)).to(dtype)
    blocked = torch.stack([gate.view(n2, -1, 16), up.view(n2, -1, 16)], dim=2).reshape(n2, 2 * i2).contiguous()
    out2 = torch.empty(n2, i2, device=DEV, dtype=dtype)
    K.silu_mul(blocked, out2, blocked=True)
    want2 = ph.silu(gate.double().cpu().numpy()) * up.double().cpu().numpy()
    assert rel_err(out2.cpu(), torch.from_numpy(want2)) < TOL[dtype]


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32),
                                                 (torch.bfloat16, torch.bfloat16),
                                                 (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K_", [(1, 301, 100), (37, 129, 352), (130, 64, 2048)])
def test_gemm_simt(K, in_dtype, out_dtype, M, N, K_):
    a = torch.randn(M, K_, device=DEV).to(in_dtype)
    w = torch.randn(N, K_, device=DEV).to(in_dtype)
    bias = torch.randn(N, device=DEV)
    out = torch.empty(M, N, device=DEV, dtype=out_dtype)
    K.gemm_simt(a, w, bias, out)
    want = a.double() @ w.double().T + bias.double()
    assert rel_err(out, want) < (3e-6 if out_dtype == torch.float32 else 1e-2)
    K.gemm_simt(a, w, None, out)
    assert rel_err(out, a.double() @ w.double().T) < (3e-6 if out_dtype == torch.float32 else 1e-2)


def test_gemm_simt_row_does_not_depend_on_the_batch(K):
    a = torch.randn(70, 333, device=DEV)
    w = torch.randn(150, 333, device=DEV)
    big, one = torch.empty(70, 150, device=DEV), torch.empty(1, 150, device=DEV)
    K.gemm_simt(a, w, None, big)
    K.gemm_simt(a[66:67], w, None, one)
    assert torch.equal(big[66:67], one)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,nq,nkv,qk_norm", [(16, 4, 2, True), (48, 6, 3, False), (128, 8, 2, True),
                                              (80, 5, 5, True)])
def test_rope_norm_cache(K, err, dtype, d, nq, nkv, qk_norm):
    page_size, n_tok, eps = 8, 13, 1e-5
    starts = [0, 21]                      # entry 0: positions 0..5; entry 1: positions 21..27
    counts = [6, 7]
    positions = torch.tensor(list(range(0, 6)) + list(range(21, 28)), dtype=torch.int32)
    tok_entry = torch.tensor([0] * 6 + [1] * 7, dtype=torch.int32)
    cols = (nq + 2 * nkv) * d
    qkv = torch.randn(n_tok, cols, device=DEV).to(dtype)
    table = torch.tensor([[3, -1, -1, -1], [7, 1, 5, 0]], dtype=torch.int32, device=DEV)
    k_pool = torch.zeros(9, nkv, page_size, d, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    inv = ph.rope_inv_freq(d, 10000.0, 7.0)
    ang = ph.rope_angles(np.arange(64), inv)
    cos = torch.from_numpy(np.cos(ang.astype(np.float64)).astype(np.float32)).to(DEV)
    sin = torch.from_numpy(np.sin(ang.astype(np.float64)).astype(np.float32)).to(DEV)
    qw = (1 + 0.1 * torch.randn(d)).to(DEV) if qk_norm else None
    kw = (1 + 0.1 * torch.randn(d)).to(DEV) if qk_norm else None
    q_out = torch.empty(n_tok, nq * d, device=DEV, dtype=dtype)
    K.rope_norm_cache(qkv, cols, dtype, positions.to(DEV), tok_entry.to(DEV), table, cos, sin, qw, kw,
                      eps, q_out, k_pool, v_pool, page_size, nq, nkv, d, True, True, err)
    assert int(err.item()) == 0
    x = qkv.double().cpu().numpy()
    q = x[:, :nq * d].reshape(n_tok, nq, d)
    k = x[:, nq * d:(nq + nkv) * d].reshape(n_tok, nkv, d)
    v = x[:, (nq + nkv) * d:].reshape(n_tok, nkv, d)
    a = ph.rope_angles(positions.numpy(), inv)
    q, k = ph.apply_rope(q, a), ph.apply_rope(k, a)
    if qk_norm:
        q = ph.rms_norm(q, qw.double().cpu().numpy(), eps)
        k = ph.rms_norm(k, kw.double().cpu().numpy(), eps)
    assert rel_err(q_out.cpu().view(n_tok, nq, d), torch.from_numpy(q)) < TOL[dtype]
    for t in range(n_tok):
        p, e = int(positions[t]), int(tok_entry[t])
        page, off = int(table[e, p // page_size]), p % page_size
        assert rel_err(k_pool[page, :, off].cpu(), torch.from_numpy(k[t])) < TOL[dtype]
        assert rel_err(v_pool[page, :, off].cpu(), torch.from_numpy(v[t])) < TOL[dtype]
    # nothing else was written: 13 tokens' worth of non-zero rows
    assert int((k_pool.float().abs().sum(-1) > 0).sum()) == n_tok * nkv
    # a block-table entry outside the pool is reported, not followed
    bad = table.clone(); bad[0, 0] = 99
    K.rope_norm_cache(qkv, cols, dtype, positions.to(DEV), tok_entry.to(DEV), bad, cos, sin, qw, kw,
                      eps, q_out, k_pool, v_pool, page_size, nq, nkv, d, True, True, err)
    assert int(err.item()) & 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,nq,nkv,page_size,window", [(16, 4, 2, 16, 0), (48, 6, 2, 8, 0),
                                                        (128, 8, 2, 64, 0), (32, 4, 4, 16, 37),
                                                        (256, 2, 1, 32, 0)])
def test_paged_attention_mixed_batch(K, err, dtype, d, nq, nkv, page_size, window):
    """Three requests: a prompt portion that starts in the middle of a page, a
    single decoded token far into a long context, and a whole short prompt."""
    torch.manual_seed(d + window)
    lens = [150, 333, 9]                   # cached length after the step
    q_lens = [45, 1, 9]
    ks = [torch.randn(n, nkv, d) for n in lens]
    vs = [torch.randn(n, nkv, d) for n in lens]
    # a far key that must dominate: request 1's token reads position 17 of 333
    qs = [torch.randn(ql, nq, d) for ql in q_lens]
    ks[1][17] *= 0.0
    ks[1][17, :, 0] = 40.0
    qs[1][0, :, 0] = 8.0 / (d ** -0.5) / 40.0 + 3.0         # score(17) stands out by far
    if dtype == torch.bfloat16:
        ks = [k.bfloat16().float() for k in ks]; vs = [v.bfloat16().float() for v in vs]
        qs = [q.bfloat16().float() for q in qs]
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, dtype)
    positions, tok_entry = [], []
    for e, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n)); tok_entry += [e] * ql
    q = torch.cat(qs).to(DEV).to(dtype).reshape(-1, nq * d)
    out = torch.empty_like(q)
    K.paged_attention_simt(q, out, k_pool, v_pool, torch.tensor(positions, dtype=torch.int32, device=DEV),
                           torch.tensor(tok_entry, dtype=torch.int32, device=DEV), table, page_size,
                           nq, nkv, d, window, d ** -0.5, err)
    assert int(err.item()) == 0
    row = 0
    for e, (n, ql) in enumerate(zip(lens, q_lens)):
        for i in range(ql):
            want = attention_reference(qs[e][i], ks[e], vs[e], n - ql + i, window)
            got = out[row].cpu().view(nq, d)
            assert rel_err(got, want) < (3e-6 if dtype == torch.float32 else 1.5e-2), (e, i)
            row += 1
    if window == 0:
        far = out[45].cpu().view(nq, d).double()
        assert rel_err(far[0], vs[1][17, 0].double()) < 2e-2       # the far key's value came through


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(K, err, dtype):
    """The key at position p - window must not be read, the one at p - window + 1 must."""
    d, nq, nkv, ps, window, n = 32, 2, 1, 16, 24, 100
    k = torch.zeros(n, nkv, d); v = torch.zeros(n, nkv, d)
    k[:, 0, 0] = 1.0
    v[:, 0, 0] = torch.arange(n).float()
    k[n - 1 - window, 0, 0] = 30.0        # just outside: would win if read
    k[n - window, 0, 0] = 5.0             # just inside
    q = torch.zeros(1, nq, d); q[..., 0] = 4.0 * d ** 0.5
    k_pool, v_pool, table = paged_cache([k], [v], ps, dtype)
    out = torch.empty(1, nq * d, device=DEV, dtype=dtype)
    K.paged_attention_simt(q.to(DEV).to(dtype).reshape(1, -1), out, k_pool, v_pool,
                           torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                           torch.zeros(1, dtype=torch.int32, device=DEV), table, ps, nq, nkv, d,
                           window, d ** -0.5, err)
    want = attention_reference(q[0], k, v, n - 1, window)
    assert rel_err(out.cpu().view(nq, d), want) < (3e-6 if dtype == torch.float32 else 1.5e-2)
    assert abs(float(out[0, 0]) - (n - window)) < 1.0


def _window_edge_request(pos0, q_len, nq, nkv, d, window):
    """Queries, keys and values of one request in which every query row has a
    key that would swamp its softmax JUST outside its window and its heaviest
    legitimate key JUST inside: row i (position p = pos0 + i) asks channel
    i mod d; key j answers 30 in the channel of the row whose window it has just
    left (j = p - window) and 5 in the channel of the row whose window starts at
    it (j = p - window + 1).  The window is shorter than d, so inside a row's
    window no other key answers its channel.  Channel 0 of the values is the
    key's position (from the request's first kept one), the rest small noise: a
    key too many pulls a row's output to p - window, a key too few to the middle
    of its window."""
    assert window + 2 <= d
    n = pos0 + q_len
    q = torch.zeros(q_len, nq, d)
    for i in range(q_len):
        q[i, :, i % d] = d ** 0.5                       # times 1 / sqrt(d): the key's channel value is the score
    k = torch.zeros(n, nkv, d)
    for j in range(n):
        k[j, :, (j + window - pos0) % d] = 30.0
        k[j, :, (j - 1 + window - pos0) % d] = 5.0
    v = 0.05 * torch.randn(n, nkv, d)
    v[:, :, 0] = (torch.arange(n).float() - max(0, pos0 - window - 2))[:, None]
    return q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()


def _check_window_edge(out_rows, reqs, window, nq, d):
    row = 0
    for (pos0, q_len), (q, k, v) in reqs:
        for i in range(q_len):
            want = attention_reference(q[i], k, v, pos0 + i, window)
            got = out_rows[row].double().cpu().view(nq, d)
            # channel 0 is a position: a wrong edge moves it by a fifth of the window or more
            assert (got[:, 0] - want[:, 0]).abs().max() < 0.02 * window + 0.01 * float(want[:, 0].abs().max()), \
                (pos0, i, got[:, 0], want[:, 0])
            assert rel_err(got, want) < 1.5e-2, (pos0, i)
            row += 1


WINDOW_EDGE_KERNELS = ["simt", "decode_1", "decode_3", "decode_12", "fused_1", "fused_3", "fused_12",
                       "prefill_mma", "prefill_tc"]


@pytest.mark.parametrize("kernel", WINDOW_EDGE_KERNELS)
@pytest.mark.parametrize("d,page_size,window", [(128, 64, 100), (128, 32, 33), (64, 16, 50)])
def test_window_edge_of_the_serving_kernels(K, err, kernel, d, page_size, window):
    """Every attention kernel that serves: the key at p - window is not read, the
    one at p - window + 1 is, for every row of a query tile (rows of one tile have
    different window starts), with the edge at the start of a tile, of a page, in
    their middle, and before the first key."""
    nq, nkv = 8, 2
    if kernel == "prefill_tc" and not K.prefill_attention_tc_supports(d, nq, nkv, page_size):
        pytest.skip("the tcgen05 flash attention is built for head size 128")
    torch.manual_seed(window)
    single = kernel.startswith(("decode", "fused"))
    if single:
        # the window's first key: position 0, 1, a tile's first (32), 33, a page's first and last, mid-tile
        first = [0, 1, 32, 33, page_size, 2 * page_size - 1, 4 * page_size, 77, 600, 1000]
        shapes = [(lo + window - 1, 1) for lo in first] + [(window // 2, 1)]      # the last: no key left out yet
    else:
        shapes = [(211, 300), (1333 - 1, 1), (0, 150), (65, 2), (window - 1, 3)]
    reqs = [((pos0, ql), _window_edge_request(pos0, ql, nq, nkv, d, window)) for pos0, ql in shapes]
    lens = [pos0 + ql for pos0, ql in shapes]
    q_lens = [ql for _, ql in shapes]
    ks, vs = [r[1][1].clone() for r in reqs], [r[1][2].clone() for r in reqs]
    if kernel.startswith("fused"):
        for k_, v_ in zip(ks, vs):                       # the new position's key and value come from the step
            k_[-1] = 77.0
            v_[-1] = 77.0
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, torch.bfloat16, seed=window)
    i32 = lambda x: torch.tensor(np.asarray(x), dtype=torch.int32, device=DEV)
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    q = torch.cat([r[1][0] for r in reqs]).to(DEV).bfloat16().reshape(-1, nq * d)
    out = torch.full_like(q, 9.0)
    scale = d ** -0.5
    n = len(shapes)
    if kernel == "simt":
        pos = np.concatenate([np.arange(p0, p0 + ql) for p0, ql in shapes])
        ent = np.concatenate([np.full(ql, e) for e, ql in enumerate(q_lens)])
        K.paged_attention_simt(q, out, k_pool, v_pool, i32(pos), i32(ent), table, page_size, nq, nkv, d,
                               window, scale, err)
    elif single:
        splits = int(kernel.split("_")[1])
        part_o = torch.empty(n * nq * splits * d, device=DEV)
        part_ml = torch.empty(n * nq * splits * 2, device=DEV)
        if kernel.startswith("decode"):
            K.paged_decode_attention(q, out, k_pool, v_pool, i32(cu), i32(lens), table, page_size, nq, nkv, d,
                                     window, scale, splits, part_o, part_ml, err)
        else:
            new_k = torch.stack([r[1][1][-1] for r in reqs]).reshape(n, nkv * d)
            new_v = torch.stack([r[1][2][-1] for r in reqs]).reshape(n, nkv * d)
            qkv = torch.cat([q, new_k.to(DEV).bfloat16(), new_v.to(DEV).bfloat16()], dim=1).contiguous()
            K.paged_decode_attention_fused(qkv, qkv.shape[1], True, None, None, None, None, 0.0, out, k_pool,
                                           v_pool, i32(cu), i32(lens), table, page_size, nq, nkv, d, window,
                                           scale, splits, part_o, part_ml, err)
    elif kernel == "prefill_mma":
        K.paged_prefill_attention(q, out, k_pool, v_pool, i32(cu), i32(lens), table, page_size,
                                  sum((x + 63) // 64 for x in q_lens), nq, nkv, d, window, scale, err)
    else:
        K.prefill_attention_tc(q, out, k_pool, v_pool, i32(cu), i32(lens), table, page_size,
                               sum((x + 127) // 128 for x in q_lens), nq, nkv, d, window, scale, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _check_window_edge(out, reqs, window, nq, d)


def test_argmax_ties_go_to_the_lowest_index(K):
    vocab = 120818
    logits = torch.randn(3, vocab, device=DEV)
    logits[0, 77777] = 50.0; logits[0, 1234] = 50.0
    logits[1, vocab - 1] = 60.0
    logits[2, :] = -1.0                                   # all equal
    out = torch.zeros(3, dtype=torch.int32, device=DEV)
    K.sample(logits, out)
    assert out.tolist() == [1234, vocab - 1, 0]


def test_repetition_penalty(K):
    vocab = 1000
    logits = torch.randn(2, vocab, device=DEV)
    want = logits.clone()
    ctx = torch.tensor([[5, 7, 5, 999, 0], [1, 2, 3, 4, 5]], dtype=torch.int32, device=DEV)
    ctx_len = torch.tensor([4, 0], dtype=torch.int32, device=DEV)
    pen = torch.tensor([1.3, 2.0], device=DEV)
    K.repetition_penalty(logits, ctx, ctx_len, pen)
    row = ph.apply_repetition_penalty(want[0].double().cpu().numpy(), 1.3, [5, 7, 5, 999])
    assert rel_err(logits[0].cpu(), torch.from_numpy(row)) < 1e-6
    assert torch.equal(logits[1], want[1])                # no context: untouched


def _host_opts(temp, topk, topp, seed, counter):
    t = lambda v, dt: torch.tensor(v, dtype=dt, device=DEV)
    return dict(temperature=t(temp, torch.float32), top_k=t(topk, torch.int32),
                top_p=t(topp, torch.float32), seed=t(seed, torch.int64), counter=t(counter, torch.int64))


def test_temperature_sampling_matches_the_restated_generator(K):
    vocab = 3001
    logits = 3 * torch.randn(4, vocab, device=DEV)
    out = torch.zeros(4, dtype=torch.int32, device=DEV)
    temps, seeds, counters = [0.8, 1.0, 0.0, 2.5], [1024, 7, 7, 99], [0, 5, 5, 123456]
    K.sample(logits, out, **_host_opts(temps, [0] * 4, [1.0] * 4, seeds, counters))
    for r in range(4):
        row = logits[r].double().cpu().numpy()
        if temps[r] <= 0:
            assert int(out[r]) == int(np.argmax(row))
            continue
        score = ph.gumbel_scores(row, temps[r], ph.uniform_noise(seeds[r], counters[r], vocab))
        # float32 logs on the device: the chosen token's score must be the maximum up to rounding
        assert score[int(out[r])] >= score.max() - 1e-4
    again = torch.zeros_like(out)
    K.sample(logits, again, **_host_opts(temps, [0] * 4, [1.0] * 4, seeds, counters))
    assert torch.equal(out, again)
    K.sample(logits, again, **_host_opts(temps, [0] * 4, [1.0] * 4, seeds, [c + 1 for c in counters]))
    assert not torch.equal(out, again)


def test_top_k_and_top_p(K):
    vocab = 5003
    logits = torch.randn(1, vocab, device=DEV)
    best = [4000, 17, 2500, 901]
    for i, b in enumerate(best):
        logits[0, b] = 10.0 - i                     # probabilities ~ .64 .24 .09 .03 among the top 4
    row = logits[0].double().cpu().numpy()
    seen_k, seen_p = set(), set()
    out = torch.zeros(1, dtype=torch.int32, device=DEV)
    for c in range(300):
        K.sample(logits, out, **_host_opts([1.0], [3], [1.0], [5], [c]))
        seen_k.add(int(out[0]))
        K.sample(logits, out, **_host_opts([1.0], [0], [0.7], [5], [c]))
        seen_p.add(int(out[0]))
    assert seen_k == set(best[:3])                                   # never outside the top 3
    keep = ph.top_k_top_p_keep(row, 1.0, 64, 0.7)
    assert seen_p == set(int(i) for i in keep) == set(best[:2])      # .64 <= .7, plus the one after


def test_top_p_in_a_vocabulary_smaller_than_the_candidate_list(K):
    """top-p applies also where top-k cannot restrict anything (a vocabulary of
    at most 64 entries, or top-k >= vocabulary)."""
    logits = torch.tensor([[0.0, 5.0, 1.0, -2.0, 4.0]], device=DEV)       # p ~ .72 .26 .01 ...
    out = torch.zeros(1, dtype=torch.int32, device=DEV)
    for topk in (0, 5, 64, 100):
        seen = set()
        for c in range(200):
            K.sample(logits, out, **_host_opts([1.0], [topk], [0.3], [9], [c]))
            seen.add(int(out[0]))
        assert seen == {1}, (topk, seen)          # .72 > .3: the first candidate alone
        seen = set()
        for c in range(200):
            K.sample(logits, out, **_host_opts([1.0], [topk], [0.8], [9], [c]))
            seen.add(int(out[0]))
        assert seen == {1, 4}, (topk, seen)       # .72 <= .8, plus the one after


def test_sampling_frequencies_follow_the_softmax(K):
    vocab = 7
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5, 1.5, -3.0]], device=DEV)
    p = torch.softmax(logits[0] / 0.9, 0).cpu().numpy()
    n = 4000
    counts = np.zeros(vocab)
    out = torch.zeros(1, dtype=torch.int32, device=DEV)
    big = logits.repeat(n, 1)
    outs = torch.zeros(n, dtype=torch.int32, device=DEV)
    K.sample(big, outs, **_host_opts([0.9] * n, [0] * n, [1.0] * n, [11] * n, list(range(n))))
    counts = np.bincount(outs.cpu().numpy(), minlength=vocab) / n
    # u is drawn from [1e-7, 0.999), as in the reference, which trims the upper tail a little
    assert np.abs(counts - p).max() < 0.03


@pytest.mark.parametrize("M,N,K_,bn", [(128, 128, 64, 128), (128, 256, 128, 256), (300, 520, 160, 128),
                                       (2048, 3072, 2048, 256), (77, 1000, 352, 128), (2048, 3072, 2048, 192),
                                       (300, 1000, 352, 224), (260, 520, 160, 160)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_many_tokens(K, err, M, N, K_, bn, out_dtype):
    a = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV)
    out = torch.full((M, N), 7.0, device=DEV, dtype=out_dtype)
    if out_dtype == torch.float32 and bn not in (128, 256):
        bn = 256                                  # the widths between 128 and 256 write bfloat16 only
    K.gemm_tcgen05(a, w, bias, out, err, bn=bn)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    want = a.double() @ w.double().T + bias.double()
    assert rel_err(out, want) < (acc_tol(K_) if out_dtype == torch.float32 else 5e-3)
    K.gemm_tcgen05(a, w, None, out, err, bn=bn)
    assert rel_err(out, a.double() @ w.double().T) < (acc_tol(K_) if out_dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("M,N,K_,bn", [(256, 256, 64, 256), (256, 512, 128, 256), (300, 520, 160, 128),
                                       (2048, 3072, 2048, 192), (700, 1000, 352, 224), (2048, 2048, 6144, 256)])
def test_gemm_on_pairs_of_sms(K, err, M, N, K_, bn):
    """The kernel in which two SMs share a 256-row tile: each loads half of the
    weights' rows, both halves must land in the right columns."""
    torch.manual_seed(M + N)
    a = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV)
    out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_pair(a, w, bias, out, err, bn=bn)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert rel_err(out, a.double() @ w.double().T + bias.double()) < 5e-3
    K.gemm_pair(a, w, None, out, err, bn=bn)
    assert rel_err(out, a.double() @ w.double().T) < 5e-3


@pytest.mark.parametrize("M,N,K_,bn", [(256, 256, 64, 256), (300, 520, 160, 128), (2048, 3072, 2048, 192),
                                       (700, 1000, 352, 192), (5000, 4100, 512, 256), (129, 192, 64, 192),
                                       (100, 200, 72, 128)])
def test_gemm_in_tiles_of_256_rows(K, err, M, N, K_, bn):
    """Tiles of 256 tokens on one SM (two accumulators of one tile): the second
    128 rows must land 128 rows further down, also where they reach past the end
    of the tokens, and a CTA that takes several tiles must keep them apart."""
    torch.manual_seed(M + N)
    a = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV)
    out = torch.full((M + 3, N), 7.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_tcgen05(a, w, bias, out[:M], err, bn=bn, tile_rows=256)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert rel_err(out[:M], a.double() @ w.double().T + bias.double()) < 5e-3
    assert bool((out[M:] == 7.0).all())                    # nothing written past the last row
    K.gemm_tcgen05(a, w, None, out[:M], err, bn=bn, tile_rows=256)
    assert rel_err(out[:M], a.double() @ w.double().T) < 5e-3
    # the same rows as the 128-row tiles give, bit for bit (same order of the sums)
    ref = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_tcgen05(a, w, None, ref, err, bn=bn if bn != 192 else 192)
    assert torch.equal(ref, out[:M])


@pytest.mark.parametrize("M,N,K_,bn", [(512, 256, 64, 256), (300, 520, 160, 192), (2048, 3072, 2048, 224),
                                       (700, 1000, 352, 224), (5000, 9000, 512, 256), (257, 192, 64, 192),
                                       (100, 200, 72, 256)])
def test_gemm_on_pairs_of_sms_in_tiles_of_512_rows(K, err, M, N, K_, bn):
    """Two SMs, two accumulators each: rows 0..127 and 256..383 of a tile in the
    first SM, 128..255 and 384..511 in the second; bit for bit what the 256-row
    tiles of the pair kernel give."""
    torch.manual_seed(M + N)
    a = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV)
    out = torch.full((M + 3, N), 7.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_pair(a, w, bias, out[:M], err, bn=bn, tile_rows=512)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert rel_err(out[:M], a.double() @ w.double().T + bias.double()) < 5e-3
    assert bool((out[M:] == 7.0).all())
    K.gemm_pair(a, w, None, out[:M], err, bn=bn, tile_rows=512)
    ref = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_pair(a, w, None, ref, err, bn=bn)
    assert torch.equal(ref, out[:M])
    # with the silu(gate) * up epilogue (N / 2 output columns; needs N % 32 == 0)
    if N % 32 == 0:
        o1 = torch.full((M, N // 2), 7.0, device=DEV, dtype=torch.bfloat16)
        o2 = torch.full((M, N // 2), 7.0, device=DEV, dtype=torch.bfloat16)
        ws = (w.float() * 0.05).bfloat16()
        K.gemm_pair(a, ws, None, o1, err, bn=bn, silu_mul=True, tile_rows=512)
        K.gemm_pair(a, ws, None, o2, err, bn=bn, silu_mul=True)
        assert torch.equal(o1, o2)
    torch.cuda.synchronize()
    assert int(err.item()) == 0


@pytest.mark.parametrize("M,I,K_,bn", [(256, 128, 64, 128), (300, 352, 160, 192), (2048, 6144, 2048, 224),
                                       (130, 1008, 64, 256)])
def test_gemm_on_pairs_of_sms_with_silu_mul(K, err, M, I, K_, bn):
    torch.manual_seed(I + M)
    a = torch.randn(M, K_, device=DEV).bfloat16()
    gate = (torch.randn(I, K_, device=DEV) * 0.05).bfloat16()
    up = (torch.randn(I, K_, device=DEV) * 0.05).bfloat16()
    w = torch.stack([gate.view(-1, 16, K_), up.view(-1, 16, K_)], dim=1).reshape(2 * I, K_).contiguous()
    out = torch.full((M, I), 7.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_pair(a, w, None, out, err, bn=bn, silu_mul=True)
    g = a.double() @ gate.double().T
    u = a.double() @ up.double().T
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert rel_err(out, g / (1 + torch.exp(-g)) * u) < 6e-3


@pytest.mark.parametrize("M,bn", [(1, 16), (8, 16), (16, 16), (17, 32), (33, 64), (64, 64), (100, 128), (200, 256)])
@pytest.mark.parametrize("N,K_,split", [(256, 128, 1), (3072, 2048, 6), (1000, 352, 3), (120818, 256, 1),
                                        (2048, 6144, 9)])
def test_gemm_tcgen05_few_tokens_swapped_and_split(K, err, M, bn, N, K_, split):
    from crane_b200.kernels import Partials
    a = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV)
    want = a.double() @ w.double().T + bias.double()
    out = torch.full((M, N), 7.0, device=DEV, dtype=torch.float32)
    K.gemm_tcgen05(a, w, bias, out, err, swap=True, bn=bn)
    assert rel_err(out, want) < acc_tol(K_)
    outb = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_tcgen05(a, w, bias, outb, err, swap=True, bn=bn)
    assert rel_err(outb, want) < 5e-3
    _, slices = K.split_plan(K_, split)
    if slices > 1:
        parts = torch.full((slices, M, N), 7.0, device=DEV)
        K.gemm_tcgen05(a, w, bias, parts, err, split_k=slices, swap=True, bn=bn)
        assert rel_err(parts.sum(0), want) < acc_tol(K_)
        # the consumers add the slices up themselves
        x = torch.zeros(M, N, device=DEV)
        normed = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        K.add_rmsnorm(x, Partials(parts), torch.ones(N, device=DEV), 1e-6, normed)
        assert rel_err(x, want) < 4e-3        # rounded once to bfloat16, like a whole product
    torch.cuda.synchronize()
    assert int(err.item()) == 0


@pytest.mark.parametrize("M,N,K_,slices", [(300, 384, 3072, 2), (512, 2048, 6144, 4), (1000, 260, 4608, 3)])
def test_gemm_tcgen05_hundreds_of_tokens_in_wide_slices(K, err, M, N, K_, slices):
    """A few hundred tokens, a long inner dimension: tiles of 128 features x 256
    tokens (several tiles of tokens) over slices, and the norm that adds them up."""
    from crane_b200.kernels import Partials
    a = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV).bfloat16()
    want = a.double() @ w.double().T
    parts = torch.full((slices, M, N), 7.0, device=DEV)
    K.gemm_tcgen05(a, w, None, parts, err, split_k=slices, swap=True, bn=256)
    assert rel_err(parts.sum(0), want) < acc_tol(K_)
    x = torch.zeros(M, N, device=DEV)
    normed = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K.add_rmsnorm(x, Partials(parts), torch.ones(N, device=DEV), 1e-6, normed)
    assert rel_err(x, want) < 4e-3
    torch.cuda.synchronize()
    assert int(err.item()) == 0


def test_gemm_tcgen05_refuses_what_it_cannot_take(K, err):
    from crane_b200.kernels import KernelError
    a = torch.randn(4, 100, device=DEV).bfloat16()        # inner dimension not a multiple of 8
    w = torch.randn(16, 100, device=DEV).bfloat16()
    assert not K.tcgen05_takes(a, w)
    with pytest.raises(KernelError):
        K.gemm_tcgen05(a, w, None, torch.empty(4, 16, device=DEV, dtype=torch.bfloat16), err)


@pytest.mark.parametrize("d,nq,nkv,page_size,window,splits", [
    (128, 16, 4, 64, 0, 1), (128, 16, 4, 64, 0, 7), (64, 8, 8, 16, 0, 3), (16, 4, 2, 8, 0, 2),
    (32, 8, 2, 16, 50, 4), (48, 6, 3, 32, 0, 32), (128, 32, 2, 128, 300, 5),
    (80, 10, 5, 16, 0, 3), (96, 6, 2, 32, 0, 1), (112, 4, 4, 16, 90, 4), (160, 4, 2, 16, 0, 2),
    (192, 6, 1, 32, 0, 5), (256, 8, 2, 64, 0, 6),
    # head size 128 with pages smaller than the kernel's 32-key tiles: a tile comes in several pieces
    (128, 8, 2, 16, 0, 3), (128, 16, 4, 16, 0, 8), (128, 4, 4, 8, 45, 2), (128, 8, 1, 16, 333, 12)])
def test_paged_decode_attention(K, err, d, nq, nkv, page_size, window, splits):
    """Single tokens of requests of very different lengths, one of them with a
    far key that must dominate; every slicing of the keys gives the same."""
    assert K.decode_attention_supports(d, nq, nkv)
    torch.manual_seed(d * 7 + splits)
    lens = [1, 31, 32, 33, 700, 1025]
    ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(nq, d).bfloat16().float() for _ in lens]
    far = 1025 - 40 if window else 11             # inside the window when there is one
    ks[5][far] = 0.0; ks[5][far, :, 1] = 30.0; qs[5][:, 1] = 6.0 * d ** 0.5 / 30.0 * 4
    ks[5] = ks[5].bfloat16().float(); qs[5] = qs[5].bfloat16().float()
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, torch.bfloat16, seed=splits)
    n = len(lens)
    q = torch.stack(qs).to(DEV).bfloat16().reshape(n, nq * d)
    out = torch.full_like(q, 9.0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    part_o = torch.empty(n * nq * splits * d, device=DEV)
    part_ml = torch.empty(n * nq * splits * 2, device=DEV)
    K.paged_decode_attention(q, out, k_pool, v_pool, i32(list(range(n + 1))), i32(lens), table, page_size,
                             nq, nkv, d, window, d ** -0.5, splits, part_o, part_ml, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    for e in range(n):
        want = attention_reference(qs[e], ks[e], vs[e], lens[e] - 1, window)
        assert rel_err(out[e].cpu().view(nq, d), want) < 1.5e-2, (e, lens[e])
    assert rel_err(out[5].cpu().view(nq, d)[0], vs[5][far, 0].double()) < 2e-2
    # the plain kernel agrees
    ref = torch.empty_like(q)
    K.paged_attention_simt(q, ref, k_pool, v_pool, i32([l - 1 for l in lens]), i32(list(range(n))), table,
                           page_size, nq, nkv, d, window, d ** -0.5, err)
    assert rel_err(out, ref.double()) < 1.5e-2


@pytest.mark.parametrize("d,nq,nkv,page_size,window", [(128, 8, 2, 64, 0), (64, 4, 4, 16, 0),
                                                        (16, 4, 2, 8, 0), (32, 4, 1, 16, 37),
                                                        (48, 6, 3, 32, 0), (128, 4, 1, 128, 100),
                                                        (80, 10, 5, 16, 0), (96, 6, 2, 32, 41), (112, 4, 4, 16, 0),
                                                        (160, 4, 2, 16, 0), (192, 6, 1, 32, 0), (256, 8, 2, 64, 70)])
def test_paged_prefill_attention_mixed_batch(K, err, d, nq, nkv, page_size, window):
    """A portion that starts in the middle of a page after 105 cached positions, a
    single decoded token far into a long context, a whole prompt of 200, a
    2-token portion and a 1-token request, in one launch."""
    torch.manual_seed(d + window)
    lens = [150, 333, 200, 67, 1]
    q_lens = [45, 1, 200, 2, 1]
    ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(ql, nq, d).bfloat16().float() for ql in q_lens]
    far = 333 - 20 if window else 17
    ks[1][far] = 0.0; ks[1][far, :, 0] = 40.0
    qs[1][0, :, 0] = 1.0 * d ** 0.5                  # score 40 at the far key
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, torch.bfloat16, seed=d)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).tolist()
    tiles = sum((n + 63) // 64 for n in q_lens)
    q = torch.cat(qs).to(DEV).bfloat16().reshape(-1, nq * d)
    out = torch.full_like(q, 9.0)
    K.paged_prefill_attention(q, out, k_pool, v_pool, i32(cu), i32(lens), table, page_size, tiles,
                              nq, nkv, d, window, d ** -0.5, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    row = 0
    for e, (n, ql) in enumerate(zip(lens, q_lens)):
        for i in range(ql):
            want = attention_reference(qs[e][i], ks[e], vs[e], n - ql + i, window)
            assert rel_err(out[row].cpu().view(nq, d), want) < 1.5e-2, (e, i)
            row += 1
    assert rel_err(out[45].cpu().view(nq, d)[0], vs[1][far, 0].double()) < 2e-2


@pytest.mark.parametrize("d,nq,nkv,page_size,window,splits,qk_norm,parts", [
    (128, 16, 4, 64, 0, 9, True, 0), (128, 16, 4, 64, 0, 1, True, 3), (64, 8, 8, 16, 0, 3, False, 0),
    (16, 4, 2, 8, 0, 2, True, 2), (32, 8, 2, 16, 50, 4, True, 0), (48, 6, 3, 32, 0, 32, False, 5),
    # head size 128, 2 to 8 slices: the slices merge in a thread-block cluster; 64: the most slices
    (128, 16, 4, 64, 0, 8, True, 6), (128, 8, 8, 32, 0, 2, False, 0), (128, 12, 4, 64, 100, 5, True, 0),
    (128, 16, 4, 64, 0, 64, True, 0),
    (80, 10, 5, 16, 0, 3, True, 0), (96, 6, 2, 32, 0, 1, False, 4), (112, 8, 4, 16, 90, 4, True, 2),
    (160, 4, 2, 16, 0, 2, True, 0), (192, 6, 1, 32, 0, 5, False, 0), (256, 8, 2, 64, 0, 6, True, 3),
    (128, 16, 4, 16, 0, 8, True, 6), (128, 8, 2, 16, 70, 3, True, 0), (128, 4, 4, 8, 0, 5, False, 2)])
def test_fused_decode_attention_equals_the_separate_kernels(K, err, d, nq, nkv, page_size, window,
                                                            splits, qk_norm, parts):
    """Rotary encoding, head norms, cache write, attention and merge in one
    kernel against rope_norm_cache + paged_decode_attention: same outputs, same
    keys and values in the pages.  Requests end at the first, a middle and the
    last row of a tile and of a page."""
    from crane_b200.kernels import Partials
    torch.manual_seed(d + splits)
    lens = [1, 32, 33, 64, 65, 700, 1024]           # cached length after the step
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
            whole += p[i]                       # in slice order, as the kernel adds them
        src, whole = Partials(p), whole.bfloat16()
    else:
        src = whole = qkv.bfloat16()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    pos, ent, cu, kvl = i32([m - 1 for m in lens]), i32(list(range(n))), i32(list(range(n + 1))), i32(lens)
    inv = ph.rope_inv_freq(d, 10000.0, 3.0)
    ang = ph.rope_angles(np.arange(1100), inv).astype(np.float64)
    cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(DEV)
    sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(DEV)
    qw = (1 + 0.1 * torch.randn(d)).to(DEV) if qk_norm else None
    kw = (1 + 0.1 * torch.randn(d)).to(DEV) if qk_norm else None
    # separate kernels
    k1, v1 = k_pool.clone(), v_pool.clone()
    q = torch.empty(n, nq * d, device=DEV, dtype=torch.bfloat16)
    K.rope_norm_cache(whole, cols, torch.bfloat16, pos, ent, table, cos, sin, qw, kw, 1e-5, q, k1, v1,
                      page_size, nq, nkv, d, True, True, err)
    want = torch.empty_like(q)
    part_o = torch.empty(n * nq * splits * d, device=DEV)
    part_ml = torch.empty(n * nq * splits * 2, device=DEV)
    K.paged_decode_attention(q, want, k1, v1, cu, kvl, table, page_size, nq, nkv, d, window, d ** -0.5,
                             splits, part_o, part_ml, err)
    for _ in range(2):
        k2, v2 = k_pool.clone(), v_pool.clone()
        got = torch.full_like(q, 9.0)
        K.paged_decode_attention_fused(src, cols, True, cos, sin, qw, kw, 1e-5, got, k2, v2, cu, kvl, table,
                                       page_size, nq, nkv, d, window, d ** -0.5, splits, part_o, part_ml, err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        assert torch.equal(k2, k1) and torch.equal(v2, v1)
        assert rel_err(got, want.double()) < 4e-3


@pytest.mark.parametrize("M,I,K_,bn", [(128, 128, 64, 128), (300, 352, 160, 128), (2048, 6144, 2048, 256),
                                       (2048, 6144, 2048, 224), (300, 352, 160, 192), (130, 1008, 64, 160)])
def test_gemm_tcgen05_with_silu_mul_epilogue(K, err, M, I, K_, bn):
    a = torch.randn(M, K_, device=DEV).bfloat16()
    gate = (torch.randn(I, K_, device=DEV) / K_ ** 0.5).bfloat16()
    up = (torch.randn(I, K_, device=DEV) / K_ ** 0.5).bfloat16()
    w = torch.stack([gate.view(-1, 16, K_), up.view(-1, 16, K_)], dim=1).reshape(2 * I, K_).contiguous()
    out = torch.full((M, I), 7.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_tcgen05(a, w, None, out, err, bn=bn, silu_mul=True)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    g, u = a.double() @ gate.double().T, a.double() @ up.double().T
    want = g / (1 + torch.exp(-g)) * u
    assert rel_err(out, want) < 5e-3


@pytest.mark.parametrize("nq,nkv,page_size,window", [(8, 2, 64, 0), (4, 4, 16, 0), (4, 1, 128, 300),
                                                     (16, 4, 32, 0), (8, 2, 256, 0), (4, 2, 512, 300),
                                                     (8, 4, 256, 77)])
def test_prefill_attention_tcgen05_mixed_batch(K, err, nq, nkv, page_size, window):
    """The tensor-core flash attention (head size 128) on a mixed batch: a portion
    of 300 rows after 211 cached positions, a single decoded token far into a long
    context, a whole prompt of 1000, a 2-token portion and a 1-token request."""
    d = 128
    assert K.prefill_attention_tc_supports(d, nq, nkv, page_size)
    torch.manual_seed(nq + window)
    lens = [511, 1333, 1000, 67, 1]
    q_lens = [300, 1, 1000, 2, 1]
    ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(ql, nq, d).bfloat16().float() for ql in q_lens]
    far = 1333 - 40 if window else 17
    ks[1][far] = 0.0; ks[1][far, :, 0] = 40.0
    qs[1][0, :, 0] = 1.0 * d ** 0.5
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, torch.bfloat16, seed=nq)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).tolist()
    tiles = sum((n + 127) // 128 for n in q_lens)
    q = torch.cat(qs).to(DEV).bfloat16().reshape(-1, nq * d)
    out = torch.full_like(q, 9.0)
    K.prefill_attention_tc(q, out, k_pool, v_pool, i32(cu), i32(lens), table, page_size, tiles, nq, nkv, d,
                           window, d ** -0.5, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    # against the warp-level kernel over all rows, and against the plain computation on samples
    ref = torch.full_like(q, -9.0)
    K.paged_prefill_attention(q, ref, k_pool, v_pool, i32(cu), i32(lens), table, page_size,
                              sum((n + 63) // 64 for n in q_lens), nq, nkv, d, window, d ** -0.5, err)
    assert rel_err(out, ref.double()) < 1.5e-2
    row = 0
    for e, (n, ql) in enumerate(zip(lens, q_lens)):
        for i in sorted({0, 1, ql // 2, ql - 1} & set(range(ql))):
            want = attention_reference(qs[e][i], ks[e], vs[e], n - ql + i, window)
            assert rel_err(out[row + i].cpu().view(nq, d), want) < 1.5e-2, (e, i)
        row += ql
    assert rel_err(out[300].cpu().view(nq, d)[0], vs[1][far, 0].double()) < 2e-2


@pytest.mark.parametrize("kernel,d,nq,nkv,page_size,window,splits", [
    ("tc", 128, 8, 2, 64, 0, 4), ("tc", 128, 16, 4, 32, 300, 8), ("mma", 128, 4, 4, 16, 0, 1),
    ("mma", 64, 8, 2, 16, 0, 3), ("mma", 80, 10, 5, 16, 90, 2)])
def test_single_tokens_and_portions_split_between_two_kernels(K, err, kernel, d, nq, nkv, page_size, window,
                                                              splits):
    """A mixed step as the attention part runs it: the entries of one token on the
    split-KV decode kernel, the others on a prefill kernel that skips them; every
    row is written by exactly one of the two."""
    torch.manual_seed(d + splits)
    lens = [511, 1333, 1000, 67, 1, 900]
    q_lens = [300, 1, 1000, 2, 1, 1]
    ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(ql, nq, d).bfloat16().float() for ql in q_lens]
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, torch.bfloat16, seed=d)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).tolist()
    n = len(lens)
    q = torch.cat(qs).to(DEV).bfloat16().reshape(-1, nq * d)
    out = torch.full_like(q, 9.0)
    part_o = torch.empty(n * nq * splits * d, device=DEV)
    part_ml = torch.empty(n * nq * splits * 2, device=DEV)
    K.paged_decode_attention(q, out, k_pool, v_pool, i32(cu), i32(lens), table, page_size, nq, nkv, d, window,
                             d ** -0.5, splits, part_o, part_ml, err)
    torch.cuda.synchronize()
    untouched = [r for e in range(n) if q_lens[e] != 1 for r in range(cu[e], cu[e + 1])]
    assert float(out[untouched].float().min()) == 9.0            # the decode kernel left the portions alone
    tile = 128 if kernel == "tc" else 64
    tiles = sum((x + tile - 1) // tile for x in q_lens if x != 1)
    fn = K.prefill_attention_tc if kernel == "tc" else K.paged_prefill_attention
    fn(q, out, k_pool, v_pool, i32(cu), i32(lens), table, page_size, tiles, nq, nkv, d, window, d ** -0.5,
       err, skip_single=True)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    row = 0
    for e, (m, ql) in enumerate(zip(lens, q_lens)):
        for i in sorted({0, 1, ql // 2, ql - 1} & set(range(ql))):
            want = attention_reference(qs[e][i], ks[e], vs[e], m - ql + i, window)
            assert rel_err(out[row + i].cpu().view(nq, d), want) < 1.5e-2, (e, i)
        row += ql
    # with more tiles than there are (a step padded to a shape), nothing else is written
    again = torch.full_like(q, 9.0)
    fn(q, again, k_pool, v_pool, i32(cu), i32(lens), table, page_size, tiles + 5, nq, nkv, d, window,
       d ** -0.5, err, skip_single=True)
    torch.cuda.synchronize()
    singles = [cu[e] for e in range(n) if q_lens[e] == 1]
    assert float(again[singles].float().min()) == 9.0
    assert torch.equal(again[untouched], out[untouched])


@pytest.mark.parametrize("qk_norm", [True, False])
def test_rope_norm_cache_wide_kernel_head_size_128(K, err, qk_norm):
    """The 16-byte-per-lane form taken for bf16 rows of head size 128 and 32 or more tokens."""
    d, nq, nkv, page_size, eps = 128, 6, 2, 16, 1e-5
    lens = [37, 1, 64]                              # three entries; tokens at the end of each request
    starts = [100, 0, 17]
    positions = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)])
    tok_entry = np.concatenate([np.full(n, i) for i, n in enumerate(lens)])
    n_tok = len(positions)
    cols = (nq + 2 * nkv) * d
    qkv = torch.randn(n_tok, cols, device=DEV).bfloat16()
    blocks = 12
    table = torch.from_numpy(np.random.default_rng(0).permutation(3 * blocks).astype(np.int32)).view(3, blocks).to(DEV)
    k_pool = torch.zeros(3 * blocks, nkv, page_size, d, device=DEV, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    inv = ph.rope_inv_freq(d, 10000.0, 1000.0)
    ang = ph.rope_angles(np.arange(256), inv).astype(np.float64)
    cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(DEV)
    sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(DEV)
    qw = (1 + 0.1 * torch.randn(d)).to(DEV) if qk_norm else None
    kw = (1 + 0.1 * torch.randn(d)).to(DEV) if qk_norm else None
    q_out = torch.empty(n_tok, nq * d, device=DEV, dtype=torch.bfloat16)
    i32 = lambda v: torch.tensor(np.asarray(v), dtype=torch.int32, device=DEV)
    K.rope_norm_cache(qkv, cols, torch.bfloat16, i32(positions), i32(tok_entry), table, cos, sin, qw, kw, eps,
                      q_out, k_pool, v_pool, page_size, nq, nkv, d, True, True, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    x = qkv.double().cpu().numpy()
    q = x[:, :nq * d].reshape(n_tok, nq, d)
    k = x[:, nq * d:(nq + nkv) * d].reshape(n_tok, nkv, d)
    v = x[:, (nq + nkv) * d:].reshape(n_tok, nkv, d)
    a = ph.rope_angles(positions, inv)
    q, k = ph.apply_rope(q, a), ph.apply_rope(k, a)
    if qk_norm:
        q = ph.rms_norm(q, qw.double().cpu().numpy(), eps)
        k = ph.rms_norm(k, kw.double().cpu().numpy(), eps)
    assert rel_err(q_out.cpu().view(n_tok, nq, d), torch.from_numpy(q)) < 1e-2
    tab = table.cpu().numpy()
    for t in range(n_tok):
        p, e = int(positions[t]), int(tok_entry[t])
        page, off = int(tab[e, p // page_size]), p % page_size
        assert rel_err(k_pool[page, :, off].cpu(), torch.from_numpy(k[t])) < 1e-2
        assert torch.equal(v_pool[page, :, off].cpu(), qkv[t, (nq + nkv) * d:].view(nkv, d).cpu())
    assert int((k_pool.float().abs().sum(-1) > 0).sum()) == n_tok * nkv


def test_the_two_heads_per_cta_attention_on_the_shapes_of_these_tests():
    """The tcgen05 flash attention picks between one and two query heads per CTA by
    the size of its grid; the shapes of this file are small and would all take
    the first.  Here the same tests run once more in a process that takes the
    two-head kernel wherever the group size is even."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, CRANE_PREFILL_PAIR="2")
    here = os.path.dirname(os.path.abspath(__file__))
    p = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
                        os.path.join(here, "test_gpu_kernels.py"), os.path.join(here, "test_gpu_long_context.py"),
                        "-k", "(tcgen05 or window_edge or split_between) and not two_heads_per_cta"],
                       capture_output=True, text=True, env=env, timeout=900)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-2000:]
    assert " passed" in p.stdout


def _dense_attention(qs, ks, vs, lens, q_lens, nq, nkv, d, window):
    """Every row of every entry in float64 on the device: [sum of q_lens, nq * d]."""
    outs = []
    for q, k, v, n, ql in zip(qs, ks, vs, lens, q_lens):
        q, k, v = q.to(DEV).double(), k.to(DEV).double(), v.to(DEV).double()
        kk, vv = k.repeat_interleave(nq // nkv, dim=1), v.repeat_interleave(nq // nkv, dim=1)
        s = torch.einsum("qhd,thd->hqt", q, kk) * d ** -0.5
        pos = torch.arange(n - ql, n, device=DEV)[:, None]
        t = torch.arange(n, device=DEV)[None, :]
        mask = t <= pos
        if window > 0:
            mask &= t > pos - window
        p = torch.softmax(s.masked_fill(~mask[None], float("-inf")), dim=-1)
        outs.append(torch.einsum("hqt,thd->qhd", p, vv).reshape(ql, nq * d))
    return torch.cat(outs)


def test_attention_kernels_at_random_shapes(K, err):
    """The split-KV decode kernel, the warp-level and the tcgen05 prefill kernel
    at shapes drawn at random: up to 8 entries of 1 to 4,200 keys, portions that
    end on, before and after the edges of the 64- and 128-row tiles, pages of 8
    to 512, odd group sizes, windows, 1 to 64 key slices."""
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    worst = 0.0
    for i in range(72):
        rng = np.random.default_rng(5000 + i)
        torch.manual_seed(5000 + i)
        kind = ["decode", "mma", "tc"][i % 3]
        d = 128 if kind == "tc" else int(rng.choice([64, 128, 128, 80, 256, 16, 48]))
        nkv = int(rng.choice([1, 2, 4, 5]))
        nq = nkv * int(rng.choice([1, 2, 4, 7, 8]))
        ps = int(rng.choice([8, 16, 32, 64, 128, 256, 512]))
        n_req = int(rng.integers(1, 9))
        lens = [int(rng.integers(1, 4200)) if rng.random() < 0.6 else int(rng.integers(1, 140)) for _ in range(n_req)]
        q_lens = [1] * n_req if kind == "decode" else \
            [int(min(n, rng.choice([1, 2, 63, 64, 65, 127, 128, 129, 300, 1000, n]))) for n in lens]
        window = 0 if rng.random() < 0.6 else int(rng.integers(1, 700))
        splits = int(rng.choice([1, 2, 3, 5, 8, 9, 16, 33, 64]))
        label = f"{i}: {kind} d={d} heads {nq}/{nkv} page {ps} keys {lens} rows {q_lens} window {window} slices {splits}"
        if kind == "tc" and not K.prefill_attention_tc_supports(d, nq, nkv, ps):
            continue
        ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
        vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
        qs = [torch.randn(ql, nq, d).bfloat16().float() for ql in q_lens]
        k_pool, v_pool, table = paged_cache(ks, vs, ps, torch.bfloat16, seed=i)
        cu = i32(np.concatenate([[0], np.cumsum(q_lens)]).tolist())
        q = torch.cat(qs).to(DEV).bfloat16().reshape(-1, nq * d)
        out = torch.full_like(q, 9.0)
        if kind == "decode":
            part_o = torch.empty(n_req * nq * splits * d, device=DEV)
            part_ml = torch.empty(n_req * nq * splits * 2, device=DEV)
            K.paged_decode_attention(q, out, k_pool, v_pool, cu, i32(lens), table, ps, nq, nkv, d, window,
                                     d ** -0.5, splits, part_o, part_ml, err)
        elif kind == "mma":
            K.paged_prefill_attention(q, out, k_pool, v_pool, cu, i32(lens), table, ps,
                                      sum((n + 63) // 64 for n in q_lens), nq, nkv, d, window, d ** -0.5, err)
        else:
            K.prefill_attention_tc(q, out, k_pool, v_pool, cu, i32(lens), table, ps,
                                   sum((n + 127) // 128 for n in q_lens), nq, nkv, d, window, d ** -0.5, err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0, label
        want = _dense_attention(qs, ks, vs, lens, q_lens, nq, nkv, d, window)
        e = float(((out.double() - want).abs().max(dim=1).values /
                   want.abs().max(dim=1).values.clamp_min(1e-30)).max())
        assert e < 1.5e-2, (label, e)
        worst = max(worst, e)
    print(f"worst row error {worst:.2e}")
