"""Each part alone, built from a PartSpec with sizes of its own, against the
plain function of the same part."""
import numpy as np
import pytest
import torch

import plain_hunyuan as ph
from gpu_helpers import DEV, rel_err

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def runtime(dtype, rows=256):
    from crane_b200.parts import Runtime
    return Runtime(DEV, dtype, rows)


def build(spec, tensors, rt):
    """Part from its spec and float32 CPU tensors, through the loader's dtype policy."""
    from crane_b200.parts import build_part, part_class
    from crane_b200.weights import DictSource, load_weights
    man = part_class(spec).manifest(spec)
    assert set(man) == set(tensors), (sorted(man), sorted(tensors))
    w = load_weights(DictSource(tensors), man, {}, rt.dtype, rt.device)
    part = build_part(spec)
    part.load(w, rt)
    return part


def whole(act, dtype):
    """A part may hand its product on as partial sums; the test adds them up."""
    from crane_b200.kernels import Partials
    return act.sum(dtype) if isinstance(act, Partials) else act


def np64(t):
    return t.detach().double().cpu().numpy()


class Ctx:
    pass


def make_ctx(rt, entries, page_size, num_pages, max_blocks, table_rows):
    """entries: list of (start, count).  table_rows: block table rows per entry."""
    c = Ctx()
    pos, ent = [], []
    for i, (s, n) in enumerate(entries):
        pos += list(range(s, s + n)); ent += [i] * n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    c.n_tokens, c.n_entries, c.n_want = len(pos), len(entries), 0
    c.positions, c.tok_entry = i32(pos), i32(ent)
    c.block_tables = [i32(table_rows)]
    c.max_positions = 4096
    c.max_q_len = max(n for _, n in entries)
    c.max_kv_len = max(s + n for s, n in entries)
    c.kv_len = i32([s + n for s, n in entries])
    c.cu_q = i32(np.concatenate([[0], np.cumsum([n for _, n in entries])]).tolist())
    c.slots = i32(list(range(len(entries))))
    c.h_cu_q = c.cu_q.cpu().numpy(); c.h_kv_len = c.kv_len.cpu().numpy(); c.h_slots = c.slots.cpu().numpy()
    return c


@pytest.mark.parametrize("M,N,K_", [(5, 72, 100), (70, 33, 52), (300, 120, 36)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_on_widths_the_tensor_core_kernel_refuses_rounds_once(M, N, K_, out_dtype):
    """An inner dimension that is no multiple of 8 takes another product kernel;
    with a bias it still adds the float bias to the float sum and rounds the
    result once, as the tensor-core kernels do: the same layer gives the same
    value whichever kernel its shape selects.  A float result from split-K
    slices is summed in float by the engine's own kernel."""
    rt = runtime(torch.bfloat16, rows=512)
    torch.manual_seed(M + N)
    x = torch.randn(M, K_, device=DEV).bfloat16()
    w = (torch.randn(N, K_, device=DEV) / K_ ** 0.5).bfloat16()
    bias = 3.0 * torch.randn(N, device=DEV)
    assert not rt.kernels.tcgen05_takes(x, w)
    for b in (bias, None):
        got = whole(rt.linear(x, w, b, "t", out_dtype=out_dtype), out_dtype)
        want = x.double() @ w.double().T + (b.double() if b is not None else 0.0)
        torch.cuda.synchronize()
        # one rounding to bfloat16 (2^-9 relative) or float accumulation error only
        tol = 2.0 ** -8 if out_dtype == torch.bfloat16 else 1e-5
        assert ((got.double() - want).abs() <= tol * want.abs() + 1e-4).all()     # (+ cancellation in the float sum)


@pytest.mark.parametrize("M,N,K_", [(798, 320, 8960), (1024, 128, 6144), (300, 2048, 6144), (513, 136, 7000)])
def test_linear_of_hundreds_of_tokens_in_wide_slices_has_room_for_every_slice(M, N, K_):
    """A narrow output and a long inner dimension take 4 slices of up to 1,024
    tokens: the buffer of partial sums must hold all of them."""
    from crane_b200.kernels import Partials
    rt = runtime(torch.bfloat16, rows=1024)
    torch.manual_seed(M + N)
    x = torch.randn(M, K_, device=DEV).bfloat16()
    w = (torch.randn(N, K_, device=DEV) / K_ ** 0.5).bfloat16()
    got = rt.linear(x, w, None, "o")
    if K_ % 8 == 0:
        assert isinstance(got, Partials)
    torch.cuda.synchronize()
    assert rel_err(whole(got, torch.bfloat16), x.double() @ w.double().T) < 5e-3
    rt.check_errors()


def test_linear_at_random_shapes():
    """Products drawn at random through the runtime's choice of kernel (few
    tokens with the weights on the wide side and slices of the inner dimension,
    wide slices for hundreds of tokens, one SM or two per tile, tiles of once or
    twice the rows, the silu epilogue, the kernels for shapes the tensor-core
    kernels refuse), with and without a bias, bfloat16 and float results."""
    from crane_b200.kernels import Partials
    rt = runtime(torch.bfloat16, rows=8192)
    worst = 0.0
    for i in range(160):
        rng = np.random.default_rng(9000 + i)
        torch.manual_seed(9000 + i)
        M = int(rng.choice([1, 2, 7, 8, 16, 17, 33, 64, 65, 100, 128, 129, 200, 256, 257, 300, 512, 700, 798,
                            1000, 1024, 1025, 1500, 2048, 3000, 4096, 5000]))
        N = int(rng.choice([8, 16, 64, 100, 128, 136, 256, 320, 384, 1000, 1001, 2048, 3072, 4096, 6144, 12288]))
        K_ = int(rng.choice([64, 72, 128, 136, 256, 1000, 1536, 2048, 3072, 4096, 6144, 8960, 14336]))
        if M * N * K_ > 4096 * 12288 * 4096:
            K_ = 2048
        bias = torch.randn(N, device=DEV) if rng.random() < 0.4 else None
        out_dtype = torch.float32 if rng.random() < 0.25 else torch.bfloat16
        silu = rng.random() < 0.25 and N % 32 == 0 and bias is None and out_dtype == torch.bfloat16
        label = f"{i}: {M} x {N} x {K_}, bias {bias is not None}, {out_dtype}, silu {silu}"
        x = torch.randn(M, K_, device=DEV).bfloat16()
        w = (torch.randn(N, K_, device=DEV) / K_ ** 0.5).bfloat16()
        want = x.double() @ w.double().T + (bias.double() if bias is not None else 0.0)
        if silu:
            got = torch.full((M, N // 2), 7.0, device=DEV, dtype=torch.bfloat16)
            if not rt.linear_silu_mul(x, w, got):
                continue
            gu = want.view(M, N // 32, 2, 16)                # the weights' rows: 16 of gate, 16 of up, ...
            g, u = gu[:, :, 0].reshape(M, N // 2), gu[:, :, 1].reshape(M, N // 2)
            want = g / (1 + torch.exp(-g)) * u
        else:
            got = whole(rt.linear(x, w, bias, "t" + str(i % 3), out_dtype=out_dtype), out_dtype)
        torch.cuda.synchronize()
        rt.check_errors()
        e = rel_err(got, want)
        assert e < (6e-3 if out_dtype == torch.bfloat16 else 2e-5 * max(1.0, (K_ / 256) ** 0.5)), (label, e)
        worst = max(worst, e)
    print(f"worst error {worst:.2e}")


def test_float_logits_from_split_k_slices():
    """A head narrow enough to be computed in slices of the inner dimension: the
    float result is the slices' sum in float (no rounding to bfloat16 between)."""
    rt = runtime(torch.bfloat16, rows=512)
    torch.manual_seed(3)
    x = torch.randn(6, 2048, device=DEV).bfloat16()
    w = (torch.randn(384, 2048, device=DEV) / 45.0).bfloat16()
    before = rt.launches
    got = rt.linear(x, w, None, "head", out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert rt.launches - before == 2                      # the sliced product and the sum of its slices
    want = x.double() @ w.double().T
    assert rel_err(got, want) < 2e-6
    rt.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    from crane_b200.config import PartSpec
    rt = runtime(dtype)
    w = 1 + 0.2 * torch.randn(200)
    part = build(PartSpec("norm", "rms_norm", {"size": 200, "eps": 3e-4}, "n."), {"n.weight": w}, rt)
    x = torch.randn(11, 200, device=DEV)
    delta = torch.randn(11, 200, device=DEV).to(dtype)
    want_x = np64(x) + np64(delta)
    out = part.forward(x, delta, rt)
    assert rel_err(x.cpu(), torch.from_numpy(want_x)) < 1e-6
    assert rel_err(out.cpu(), torch.from_numpy(ph.rms_norm(want_x, np64(w), 3e-4))) < TOL[dtype]
    assert part.weight.dtype == torch.float32


def test_rope_tables_follow_the_reference_arithmetic():
    from crane_b200.config import PartSpec
    from crane_b200.parts import build_part
    rt = runtime(torch.float32)
    for d, theta, alpha in [(128, 10000.0, 1000.0), (48, 5e4, 0.0), (16, 1e6, 3.5)]:
        part = build_part(PartSpec("position", "rope", {"head_dim": d, "theta": theta, "alpha": alpha,
                                                        "max_positions": 300}))
        assert np.array_equal(part.inv_freq(), ph.rope_inv_freq(d, theta, alpha))
        cos, sin = part.tables(rt, 200)
        assert cos.shape == (200, d // 2) and cos.dtype == torch.float32
        ang = ph.rope_angles(np.arange(200), ph.rope_inv_freq(d, theta, alpha)).astype(np.float64)
        assert np.abs(cos.cpu().numpy() - np.cos(ang)).max() < 1e-7
        assert np.abs(sin.cpu().numpy() - np.sin(ang)).max() < 1e-7


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from crane_b200.config import PartSpec
    rt = runtime(dtype)
    h, i = 72, 200
    t = {"f.gate_proj.weight": 0.2 * torch.randn(i, h), "f.up_proj.weight": 0.2 * torch.randn(i, h),
         "f.down_proj.weight": 0.2 * torch.randn(h, i)}
    if dtype == torch.bfloat16:
        t = {k: v.bfloat16().float() for k, v in t.items()}
    part = build(PartSpec("ffn", "swiglu", {"hidden_size": h, "intermediate_size": i}, "f."), dict(t), rt)
    x = torch.randn(13, h, device=DEV).to(dtype)
    out = whole(part.forward(x, None, rt), dtype)
    want = ph.swiglu(np64(x), np64(t["f.gate_proj.weight"]), np64(t["f.up_proj.weight"]),
                     np64(t["f.down_proj.weight"]))
    assert rel_err(out.cpu(), torch.from_numpy(want)) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from crane_b200.config import PartSpec
    rt = runtime(dtype)
    v, h = 301, 40
    table = torch.randn(v, h)
    emb = build(PartSpec("embed", "token_embedding", {"vocab_size": v, "hidden_size": h}, "e."),
                {"e.weight": table}, rt)
    toks = torch.tensor([300, 0, 7], dtype=torch.int32, device=DEV)
    x = torch.empty(3, h, device=DEV)
    emb.forward(toks, x, rt)
    assert torch.equal(x.cpu(), table.to(dtype).float()[[300, 0, 7]])
    head_w = torch.randn(v, h)
    if dtype == torch.bfloat16:
        head_w = head_w.bfloat16().float()
    head = build(PartSpec("head", "lm_head", {"vocab_size": v, "hidden_size": h, "tied_to": None}, "l."),
                 {"l.weight": head_w}, rt)
    hid = torch.randn(5, h, device=DEV).to(dtype)
    logits = head.forward(hid, rt)
    assert logits.dtype == torch.float32 and logits.shape == (5, v)
    assert rel_err(logits.cpu(), torch.from_numpy(np64(hid) @ np64(head_w).T)) < (1e-5 if dtype == torch.float32 else 1e-5)
    # tied: shares the embedding's tensor, expects none of its own
    from crane_b200.parts import build_part, part_class
    tied = PartSpec("head", "lm_head", {"vocab_size": v, "hidden_size": h, "tied_to": "e.weight"}, "l.")
    assert part_class(tied).manifest(tied) == {}
    tp = build_part(tied); tp.load({"e.weight": emb.table}, rt)
    assert tp.weight.data_ptr() == emb.table.data_ptr()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,qk_norm,bias", [(6, 2, 48, True, True), (4, 4, 16, False, False),
                                                   (8, 2, 128, True, False)])
def test_attention_part_whole_and_in_two_portions(dtype, nq, nkv, d, qk_norm, bias):
    """The mixer alone: a whole sequence in one call, then the same sequence
    cut in two portions over the same pages, both against the plain layer."""
    from crane_b200.config import PartSpec
    from crane_b200.parts import CacheNeed, LayerCache
    rt = runtime(dtype)
    h, T, ps = 80, 50, 16
    pos_spec = PartSpec("position", "rope", {"head_dim": d, "theta": 20000.0, "alpha": 2.0,
                                             "max_positions": 4096})
    spec = PartSpec("mixer", "gqa_attention", {
        "hidden_size": h, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "bias": bias,
        "qk_norm": qk_norm, "qk_norm_eps": 1e-5, "window": 0, "own_kv": True, "position": pos_spec}, "a.")
    t = {"a.q_proj.weight": 0.15 * torch.randn(nq * d, h), "a.k_proj.weight": 0.15 * torch.randn(nkv * d, h),
         "a.v_proj.weight": 0.15 * torch.randn(nkv * d, h), "a.o_proj.weight": 0.15 * torch.randn(h, nq * d)}
    if bias:
        t.update({"a.q_proj.bias": 0.1 * torch.randn(nq * d), "a.k_proj.bias": 0.1 * torch.randn(nkv * d),
                  "a.v_proj.bias": 0.1 * torch.randn(nkv * d), "a.o_proj.bias": 0.1 * torch.randn(h)})
    if qk_norm:
        t.update({"a.query_layernorm.weight": 1 + 0.1 * torch.randn(d),
                  "a.key_layernorm.weight": 1 + 0.1 * torch.randn(d)})
    if dtype == torch.bfloat16:
        t = {k: (v.bfloat16().float() if v.dim() == 2 else v) for k, v in t.items()}
    part = build(spec, dict(t), rt)
    need = part.cache_need()
    assert need == CacheNeed("kv", kv_heads=nkv, head_dim=d, window=0)
    x = torch.randn(T, h, device=DEV).to(dtype)

    cfg = ph.PlainConfig(vocab_size=1, hidden_size=h, intermediate_size=1, num_hidden_layers=1,
                         num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d,
                         max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=20000.0,
                         rope_alpha=2.0, attention_bias=bias, use_qk_norm=qk_norm,
                         tie_word_embeddings=True, use_cla=False, cla_share_factor=1)
    want, _ = ph.attention_layer(np64(x), cfg, {k: np64(v) for k, v in t.items()}, "a.", np.arange(T))
    want = torch.from_numpy(want)

    def cache():
        shape = (6, nkv, ps, d)
        return LayerCache(need, 0, torch.full(shape, 30.0, device=DEV, dtype=dtype),
                          torch.full(shape, 30.0, device=DEV, dtype=dtype), ps)
    rows = [[4, 1, 5, 2]]
    c = cache()
    out = whole(part.forward(x, make_ctx(rt, [(0, T)], ps, 6, 4, rows), c, rt), dtype)
    assert rel_err(out.cpu(), want) < TOL[dtype]
    c = cache()
    a = whole(part.forward(x[:23], make_ctx(rt, [(0, 23)], ps, 6, 4, rows), c, rt), dtype).clone()
    b = whole(part.forward(x[23:], make_ctx(rt, [(23, T - 23)], ps, 6, 4, rows), c, rt), dtype)
    assert rel_err(torch.cat([a, b]).cpu(), want) < TOL[dtype]
    rt.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_arrangement(dtype, model_folders):
    """A whole block: residual, norms, mixer and feed-forward in the reference's order."""
    import tiny_configs
    from crane_b200.config import HunyuanDenseConfig, build_spec
    from crane_b200.parts import LayerCache, block_class
    from crane_b200.parts.model import model_manifest
    from crane_b200.weights import load_weights, open_folder
    name = "float32" if dtype == torch.float32 else "bfloat16"
    folder = model_folders("B", name)
    rt = runtime(dtype)
    mc = HunyuanDenseConfig.from_dict(tiny_configs.B)
    spec = build_spec(mc)
    w = load_weights(open_folder(folder), model_manifest(spec), spec.ignored_tensors, dtype, DEV)
    block = block_class("prenorm_residual")(spec.layers[1])
    for p in block.parts():
        p.load(w, rt)
    T, ps = 37, 16
    x0 = torch.randn(T, 160, device=DEV)
    pending = (0.5 * torch.randn(T, 160, device=DEV)).to(dtype)
    need = block.mixer.cache_need()
    shape = (4, need.kv_heads, ps, need.head_dim)
    cache = LayerCache(need, 0, torch.zeros(shape, device=DEV, dtype=dtype),
                       torch.zeros(shape, device=DEV, dtype=dtype), ps)
    x = x0.clone()
    out = block.forward(x, pending, make_ctx(rt, [(0, T)], ps, 4, 3, [[2, 0, 3]]), cache, rt)
    pc, pw = ph.load_folder(folder)
    want, _ = ph.decoder_layer(np64(x0) + np64(pending), pc, pw, 1, np.arange(T))
    got = x.double().cpu() + whole(out, dtype).double().cpu()   # the block leaves its last addition pending
    assert rel_err(got, torch.from_numpy(want)) < TOL[dtype]
