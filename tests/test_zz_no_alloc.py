"""The entry point that allocates nothing (csrc/no_alloc.h), called through its
exported C symbol, against the entry point that takes the caller's scratch
buffers: two calls in a row that share the library's built-in scratch array.

It serves callers that cannot allocate device memory while they run: a host
program that has given the whole device to its own arena, or a serving loop
that cannot afford the device-wide synchronisation of cudaMalloc / cudaFree.
This file is collected last, so a run that stops at the first failure has
already run every other test."""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from gpu_helpers import DEV, attention_reference, paged_cache, rel_err

pytestmark = pytest.mark.gpu

TOL = 1.5e-2          # the bfloat16 attention tolerance of tests/test_gpu_kernels.py
SCRATCH_FLOATS = 1 << 20


@pytest.fixture(scope="module")
def lib():
    from crane_b200.csrc import build
    lib = ctypes.CDLL(build.build_kernels())
    fn = lib.crane_paged_decode_attention_noalloc
    P, I = c_void_p, c_int
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, c_float, I, P, P]
    fn.restype = c_int
    lib.crane_noalloc_strerror.argtypes = [c_int]
    lib.crane_noalloc_strerror.restype = ctypes.c_char_p
    return lib


def _case(seed, lens, d, nq, nkv, page_size):
    torch.manual_seed(seed)
    ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(nq, d).bfloat16().float() for _ in lens]
    k_pool, v_pool, table = paged_cache(ks, vs, page_size, torch.bfloat16, seed=seed)
    q = torch.stack(qs).to(DEV).bfloat16().reshape(len(lens), nq * d)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return ks, vs, qs, k_pool, v_pool, table, q, i32(list(range(len(lens) + 1))), i32(lens)


def _call(lib, q, out, k_pool, v_pool, cu_q, kv_len, table, page_size, nq, nkv, d, splits, err):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.crane_paged_decode_attention_noalloc(
        q.data_ptr(), out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(),
        kv_len.data_ptr(), table.data_ptr(), table.shape[1], k_pool.shape[0], page_size,
        kv_len.shape[0], nq, nkv, d, 0, d ** -0.5, splits, err.data_ptr(), stream)


def test_calls_in_a_row_match_the_allocating_entry_point(lib):
    """Every call here has more than 8 key slices at head size 128, or another
    head size, so its partial results do go through the built-in array and the
    merge kernel (2 to 8 slices at head size 128 merge inside a cluster and
    would never touch it).  Each call lays its slots out differently from the
    one before and finds that call's leftovers in the array; entries shorter
    than the number of slices have slices without keys."""
    from crane_b200.kernels import get_kernels
    K = get_kernels()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    cases = ((1, [700, 33, 1025, 5], 12, 128, 16, 4, 64),       # 4 x 16 x 12 x 130 = 99,840 floats
             (2, [90, 2048, 64], 9, 128, 16, 4, 64),
             (3, [300, 5, 77], 5, 64, 8, 2, 16),                # the kernel that copies with cp.async
             (4, [40, 1500], 33, 128, 8, 1, 32))
    for seed, lens, splits, d, nq, nkv, ps in cases:
        ks, vs, qs, k_pool, v_pool, table, q, cu_q, kv_len = _case(seed, lens, d, nq, nkv, ps)
        n = len(lens)
        assert n * nq * splits * (d + 2) <= SCRATCH_FLOATS
        got = torch.full_like(q, 9.0)
        assert _call(lib, q, got, k_pool, v_pool, cu_q, kv_len, table, ps, nq, nkv, d, splits, err) == 0
        want = torch.full_like(q, -9.0)
        part_o = torch.empty(n * nq * splits * d, device=DEV)
        part_ml = torch.empty(n * nq * splits * 2, device=DEV)
        K.paged_decode_attention(q, want, k_pool, v_pool, cu_q, kv_len, table, ps, nq, nkv, d, 0,
                                 d ** -0.5, splits, part_o, part_ml, err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        assert torch.equal(got, want)              # the same kernels on the same data: the same bits
        for e in range(n):
            ref = attention_reference(qs[e], ks[e], vs[e], lens[e] - 1)
            assert rel_err(got[e].cpu().view(nq, d), ref) < TOL


def test_a_call_beyond_the_built_in_scratch_is_refused_in_words(lib):
    d, nq, nkv, ps = 128, 16, 4, 64
    lens = [40] * 64
    ks, vs, qs, k_pool, v_pool, table, q, cu_q, kv_len = _case(3, lens, d, nq, nkv, ps)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full_like(q, 9.0)
    splits = 16                                    # 64 * 16 * 16 * 130 floats > 2^20
    assert 64 * nq * splits * (d + 2) > SCRATCH_FLOATS
    code = _call(lib, q, out, k_pool, v_pool, cu_q, kv_len, table, ps, nq, nkv, d, splits, err)
    assert code == -2
    msg = lib.crane_noalloc_strerror(code).decode()
    assert "exceed" in msg and "1048576" in msg
    torch.cuda.synchronize()
    assert float(out.float().min()) == 9.0         # nothing was launched
    # slice counts outside 1..64 are an argument out of range, whatever the sizes
    for bad in (0, 65):
        code = _call(lib, q[:1], out[:1], k_pool, v_pool, cu_q[:2], kv_len[:1], table, ps, nq, nkv, d, bad, err)
        assert code == -3 and "1..64" in lib.crane_noalloc_strerror(code).decode()
    torch.cuda.synchronize()
    assert float(out.float().min()) == 9.0
    # one slice needs no scratch at all and is always taken
    assert _call(lib, q, out, k_pool, v_pool, cu_q, kv_len, table, ps, nq, nkv, d, 1, err) == 0
    torch.cuda.synchronize()
    assert rel_err(out[7].cpu().view(nq, d), attention_reference(qs[7], ks[7], vs[7], 39)) < TOL
