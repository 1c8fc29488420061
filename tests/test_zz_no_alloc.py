"""The attention entry point for callers that cannot allocate device memory
(``mf_attention_paged_noalloc``): called through its exported C symbol, its output must
equal the ordinary entry point's, on two calls in a row that share the fixed scratch array,
and a request beyond the array's size must be refused.

Such callers exist where cudaMalloc is not allowed: in a real-time loop that may not block
on the allocator, inside a host application that owns all device memory, or under a fixed
memory budget.  This file is named so that it is collected last."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, lens, nh, nk, hd, n_pages=40):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    width = max(-(-n // 64) for n in lens)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((B, width), -1, dtype=torch.int32)
    for b, n in enumerate(lens):
        for lp in range(-(-n // 64)):
            table[b, lp] = perm.pop()
    kc = torch.randn(n_pages, nk, 64, hd, generator=g).bfloat16().cuda()
    vc = torch.randn(n_pages, nk, 64, hd, generator=g).bfloat16().cuda()
    q = torch.randn(B, nh, hd, generator=g).bfloat16().cuda()
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    row_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    return q, kc, vc, row_seq, row_pos, table.cuda(), width


def _call_noalloc(lib, q, kc, vc, row_seq, row_pos, table, width, out, nh, nk, hd, n_chunks, dtype):
    fn = lib.mf_attention_paged_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = ([ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p] +
                   [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p])
    return fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), row_seq.data_ptr(), row_pos.data_ptr(),
              table.data_ptr(), width, 0, out.data_ptr(), q.shape[0], nh, nk, hd, 0, 256, n_chunks,
              1.0 / math.sqrt(hd), dtype, torch.cuda.current_stream().cuda_stream)


def test_no_alloc_entry_point_equals_the_ordinary_one_twice_in_a_row():
    from minfer_b200.kernels import api as K
    from minfer_b200.kernels.build import load_library
    lib = load_library("attention")
    lib.mf_attention_noalloc_capacity.restype = ctypes.c_longlong
    capacity = lib.mf_attention_noalloc_capacity()
    assert capacity == 4 << 20

    # two calls in a row with different shapes: the second must not see the first's leftovers
    for seed, lens, nh, nk, hd in ((1, [600, 1, 257, 64], 28, 4, 128), (2, [300, 700], 6, 2, 64)):
        q, kc, vc, row_seq, row_pos, table, width = _case(seed, lens, nh, nk, hd)
        n_chunks = 4
        want = torch.empty(len(lens), nh * hd, dtype=torch.bfloat16, device="cuda")
        partial = torch.empty(len(lens) * nh * n_chunks * (hd + 2), device="cuda")
        K.attention_paged(q, kc, vc, row_seq, row_pos, table, width, 0, want, partial, nh, nk, hd,
                          0, 256, n_chunks, 1.0 / math.sqrt(hd))
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()      # the call itself must not take any
        rc = _call_noalloc(lib, q, kc, vc, row_seq, row_pos, table, width, got, nh, nk, hd,
                           n_chunks, K.BF16)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        err = float((got.float() - want.float()).abs().max()) / 3.0
        assert err < 2e-2                    # the tolerance of the bfloat16 kernel tests
        assert torch.equal(got, want)        # in fact the same kernels: the same bits

    # float32 through the generic kernel as well
    q, kc, vc, row_seq, row_pos, table, width = _case(3, [500, 90], 4, 1, 32)
    q, kc, vc = q.float(), kc.float(), vc.float()
    want = torch.empty(2, 4 * 32, device="cuda")
    partial = torch.empty(2 * 4 * 2 * 34, device="cuda")
    K.attention_paged(q, kc, vc, row_seq, row_pos, table, width, 0, want, partial, 4, 1, 32, 0, 256,
                      2, 1.0 / math.sqrt(32))
    got = torch.zeros_like(want)
    assert _call_noalloc(lib, q, kc, vc, row_seq, row_pos, table, width, got, 4, 1, 32, 2, K.F32) == 0
    torch.cuda.synchronize()
    assert float((got - want).abs().max()) < 2e-5 * 3.0


def test_no_alloc_entry_point_refuses_more_than_its_array_holds():
    from minfer_b200.kernels import api as K
    from minfer_b200.kernels.build import load_library
    lib = load_library("attention")
    q, kc, vc, row_seq, row_pos, table, width = _case(4, [64], 28, 4, 128)
    out = torch.zeros(1, 28 * 128, dtype=torch.bfloat16, device="cuda")
    too_many_chunks = (4 << 20) // (28 * 130) + 1
    rc = _call_noalloc(lib, q, kc, vc, row_seq, row_pos, table, width, out, 28, 4, 128,
                       too_many_chunks, K.BF16)
    assert rc == 2005
    # sizes whose product would not fit 64 bits are refused the same way, not multiplied out
    fn = lib.mf_attention_paged_noalloc
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), row_seq.data_ptr(), row_pos.data_ptr(),
            table.data_ptr(), width, 0, out.data_ptr(), 2 ** 31 - 1, 2 ** 31 - 4, 4, 128, 0, 256,
            6000, 0.1, K.BF16, torch.cuda.current_stream().cuda_stream)
    assert rc == 2005
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0          # nothing was launched
