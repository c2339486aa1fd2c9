"""Attention and the whole model at the context lengths that serving and the
benchmark run at: thousands to a hundred thousand cached keys, 8 key slices
merged inside a cluster, 64 slices through scratch and the merge kernel, block
tables of hundreds of pages, positions beyond 8,192.

Among thousands of random keys one key more or less moves the output by less
than any tolerance.  So a few keys are planted that together carry most of a
row's softmax weight, each with a value of its own: at the first and last key of
the context, of pages, of 32-key tiles and of key slices, and around the
positions where a 16-bit or a page-times-stride product would wrap.  A planted
key that is dropped, read twice or read from the wrong place changes the output
by ten percent or more."""
import math

import numpy as np
import pytest
import torch

import plain_hunyuan as ph
import trace_tools as tt
from gpu_helpers import DEV, attention_reference, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from crane_b200.kernels import get_kernels
    return get_kernels()


@pytest.fixture()
def err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def planted_request(gen, n, q_len, nq, nkv, d, planted):
    """One request of n cached positions whose last q_len rows are queried.
    Every query row points along one direction u (plus noise); background keys
    score about N(0, 0.3); the planted keys lie along u with a score that gives
    them, together, a few times the weight of all background keys."""
    u = torch.randn(d, generator=gen)
    u /= u.norm()
    q = u[None, None, :] * d ** 0.5 + 0.3 * torch.randn(q_len, nq, d, generator=gen)
    k = 0.5 * torch.randn(n, nkv, d, generator=gen)
    v = torch.randn(n, nkv, d, generator=gen)
    planted = sorted({p for p in planted if 0 <= p < n})
    score = math.log(max(2.0, n / len(planted))) + 1.5
    for p in planted:
        k[p] = u[None, :] * score
        v[p] = 3.0 * torch.randn(nkv, d, generator=gen)
    return q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float(), planted


def pool_of(ks, vs, page_size, seed):
    """Pages in random order, as tests/gpu_helpers.paged_cache lays them out, but
    filled by one scatter per request (a long request has thousands of pages)."""
    rng = np.random.default_rng(seed)
    nkv, d = ks[0].shape[1], ks[0].shape[2]
    blocks = [(k.shape[0] + page_size - 1) // page_size for k in ks]
    total = sum(blocks) + 3
    order = rng.permutation(total)
    k_pool = torch.randn(total, nkv, page_size, d, device=DEV).mul_(50.0).bfloat16()    # garbage must never be read
    v_pool = torch.randn(total, nkv, page_size, d, device=DEV).mul_(50.0).bfloat16()
    table = -torch.ones(len(ks), max(blocks), dtype=torch.int32)
    nxt = 0
    for i, (k, v) in enumerate(zip(ks, vs)):
        pages = torch.from_numpy(order[nxt:nxt + blocks[i]].astype(np.int64))
        nxt += blocks[i]
        table[i, :blocks[i]] = pages.int()
        n = k.shape[0]
        full = n // page_size
        if full:
            kk = k[:full * page_size].view(full, page_size, nkv, d).permute(0, 2, 1, 3)
            vv = v[:full * page_size].view(full, page_size, nkv, d).permute(0, 2, 1, 3)
            k_pool[pages[:full].to(DEV)] = kk.to(DEV).bfloat16()
            v_pool[pages[:full].to(DEV)] = vv.to(DEV).bfloat16()
        rest = n - full * page_size
        if rest:
            pg = int(pages[full])
            k_pool[pg, :, :rest] = k[full * page_size:].transpose(0, 1).to(DEV).bfloat16()
            v_pool[pg, :, :rest] = v[full * page_size:].transpose(0, 1).to(DEV).bfloat16()
    return k_pool, v_pool, table.to(DEV)


def edge_positions(n, page_size, splits):
    """Positions where an indexing fault would show."""
    tiles = (n - 1) // 32 + 1
    per = (tiles + splits - 1) // splits
    out = [0, 1, 31, 32, page_size - 1, page_size, n - 2, n - 1, n // 2]
    for s in (1, 2, splits // 2, splits - 1):
        out += [s * per * 32 - 1, s * per * 32]                  # last key of a slice, first of the next
    for p in (4095, 4096, 8191, 8192, 16383, 16384, 32767, 32768, 65535, 65536, 131071):
        out += [p]
    return out


@pytest.mark.parametrize("lens,nq,nkv,splits,fused", [
    ([8192] * 8, 16, 4, 8, True),               # the benchmark's headline shape: 8 slices in a cluster
    ([8192], 16, 4, 64, True),                  # batch 1: 64 slices through scratch and the merge kernel
    ([8192, 8207, 5000], 16, 4, 12, False),     # the separate decode kernel, slices through scratch
    ([40000], 4, 1, 64, True),
    ([131072], 4, 1, 64, True),
    ([131072], 4, 1, 8, False)])
def test_decode_attention_at_long_contexts(K, err, lens, nq, nkv, splits, fused):
    d, ps = 128, 64
    gen = torch.Generator().manual_seed(len(lens) * 131 + splits)
    reqs = [planted_request(gen, n, 1, nq, nkv, d, edge_positions(n, ps, splits)) for n in lens]
    ks, vs = [r[1].clone() for r in reqs], [r[2].clone() for r in reqs]
    if fused:
        for k_, v_ in zip(ks, vs):                  # the last position's key and value come with the step
            k_[-1] = 77.0
            v_[-1] = 77.0
    k_pool, v_pool, table = pool_of(ks, vs, ps, seed=splits)
    n = len(lens)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    q = torch.cat([r[0] for r in reqs]).to(DEV).bfloat16().reshape(n, nq * d)
    out = torch.full_like(q, 9.0)
    part_o = torch.empty(n * nq * splits * d, device=DEV)
    part_ml = torch.empty(n * nq * splits * 2, device=DEV)
    cu, kvl = i32(list(range(n + 1))), i32(lens)
    if fused:
        new_k = torch.stack([r[1][-1] for r in reqs]).reshape(n, nkv * d).to(DEV).bfloat16()
        new_v = torch.stack([r[2][-1] for r in reqs]).reshape(n, nkv * d).to(DEV).bfloat16()
        qkv = torch.cat([q, new_k, new_v], dim=1).contiguous()
        K.paged_decode_attention_fused(qkv, qkv.shape[1], True, None, None, None, None, 0.0, out, k_pool,
                                       v_pool, cu, kvl, table, ps, nq, nkv, d, 0, d ** -0.5, splits, part_o,
                                       part_ml, err)
    else:
        K.paged_decode_attention(q, out, k_pool, v_pool, cu, kvl, table, ps, nq, nkv, d, 0, d ** -0.5,
                                 splits, part_o, part_ml, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    for e, (qq, kk, vv, planted) in enumerate(reqs):
        want = attention_reference(qq[0], kk, vv, lens[e] - 1)
        got = out[e].cpu().view(nq, d)
        assert rel_err(got, want) < 1.5e-2, (e, lens[e])
        # the check has teeth: without any one planted key the reference itself moves by far more
        drop = planted[len(planted) // 2]
        k2 = kk.clone(); k2[drop] = 0.0
        assert rel_err(attention_reference(qq[0], k2, vv, lens[e] - 1), want) > 5e-2


@pytest.mark.parametrize("cached,q_len,nq,nkv,page_size", [(0, 8192, 16, 4, 64), (16000, 512, 16, 4, 64),
                                                           (33000, 300, 4, 1, 128), (0, 8192, 4, 4, 32)])
def test_prefill_attention_tcgen05_at_long_contexts(K, err, cached, q_len, nq, nkv, page_size):
    """A whole prompt of 8,192 tokens (with 16 / 4 heads enough CTAs for the kernel
    that takes two heads per CTA; with 4 / 4 the kernel of one head per CTA), and
    portions behind 16,000 and 33,000 cached positions, on the tcgen05 flash
    attention; a handful of rows against float64."""
    d = 128
    n = cached + q_len
    gen = torch.Generator().manual_seed(n)
    q, k, v, planted = planted_request(gen, n, q_len, nq, nkv, d, edge_positions(n, page_size, 8) +
                                       [cached - 1, cached, cached + 127, cached + 128])
    k_pool, v_pool, table = pool_of([k], [v], page_size, seed=q_len)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    qd = q.to(DEV).bfloat16().reshape(q_len, nq * d)
    out = torch.full_like(qd, 9.0)
    K.prefill_attention_tc(qd, out, k_pool, v_pool, i32([0, q_len]), i32([n]), table, page_size,
                           (q_len + 127) // 128, nq, nkv, d, 0, d ** -0.5, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    rows = sorted({0, 1, 127, 128, q_len // 2, q_len - 129, q_len - 128, q_len - 2, q_len - 1} & set(range(q_len)))
    for i in rows:
        want = attention_reference(q[i], k, v, cached + i)
        assert rel_err(out[i].cpu().view(nq, d), want) < 1.5e-2, i
    # and all rows against the warp-level kernel
    ref = torch.full_like(qd, -9.0)
    K.paged_prefill_attention(qd, ref, k_pool, v_pool, i32([0, q_len]), i32([n]), table, page_size,
                              (q_len + 63) // 64, nq, nkv, d, 0, d ** -0.5, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert rel_err(out, ref.double()) < 1.5e-2


# two layers with heads of 128 (the serving kernels' size) in a narrow model, so that the plain
# implementation gets through 8,300 positions in seconds
LONG = {
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
    "vocab_size": 500, "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128, "hidden_act": "silu",
    "max_position_embeddings": 16384, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": {"alpha": 1000.0, "type": "dynamic"},
    "use_qk_norm": True, "tie_word_embeddings": True, "attention_bias": False,
}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_replay_of_a_request_beyond_8192_positions(dtype, tmp_path):
    """One request of 8,300 tokens through bin/trace_run: whole in one step, then
    most of it in one step and the last 32 tokens one by one (64 key slices, a
    block table of 130 pages), against the plain implementation."""
    from crane_b200.weights.random_init import write_model_folder
    folder = str(tmp_path / "model")
    write_model_folder(folder, LONG, 17, dtype, std=0.05, norm_std=0.05)
    cfg, w = ph.load_folder(folder)
    rng = np.random.default_rng(5)
    toks = rng.integers(0, cfg.vocab_size, 8300).tolist()
    plain = {"r0": ph.logits_all(cfg, w, toks)}
    tb = tt.TraceBuilder(64)
    tb.step([("r0", toks, [0, 1, 63, 64, 4095, 4096, 8191, 8192] + list(range(8260, 8300)))], end=["r0"])
    tt.trace_tail_decode(tb, {"r0": toks})
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, 64, str(tmp_path / "out"), timeout=900)
    worst = tt.compare(got, tb, plain, dtype, "8,300 positions")
    tt.compare_cuts([(got, tb)], dtype, "8,300 positions")
    print(f"8,300 positions {dtype}: worst relative error {worst:.3e}")
