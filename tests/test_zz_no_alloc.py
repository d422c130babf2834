"""The entry point for callers that cannot allocate device memory (csrc/attention_decode_noalloc.h):
called through its exported C symbol, twice in a row, it must give what the ordinary entry point
gives with scratch from the caller. The file name makes pytest collect it last, so that a run
that stops at the first failure has run every other test first."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def test_no_alloc_decode_attention_matches_the_ordinary_entry_point():
    from glassbox_b200 import kernels
    from test_kernels_gpu import make_cache, ref_attention, tol

    lib = kernels.lib()
    fn = lib.gb_attention_decode_noalloc
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn.argtypes = [P, LL, P, LL, P, P, P, I, P, P, I, I, I, I, I, LL, F, I, I, P, P]
    fn.restype = I
    lib.gb_attention_decode_noalloc_bytes.argtypes = [I, I, I, I, I]
    lib.gb_attention_decode_noalloc_bytes.restype = LL

    nh, nkv, hd, ps, window, splits = 9, 3, 64, 16, None, 3
    lens = [700, 65, 31, 1, 300]
    dtype = torch.bfloat16
    k, v, tables, dense = make_cache(dtype, len(lens), lens, nkv, hd, ps, seed=12)
    n = len(lens)
    row_seq = torch.arange(n, dtype=torch.int32, device=DEV)
    positions = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    assert 0 < lib.gb_attention_decode_noalloc_bytes(n, nh, nkv, hd, splits) <= 8 << 20

    for call in range(2):                                   # two calls in a row share the built-in scratch
        q = torch.randn(n, nh, hd, generator=torch.Generator().manual_seed(call)).to(dtype)
        qd = q.to(DEV).reshape(n, nh * hd)
        want = torch.empty(n, nh * hd, device=DEV, dtype=dtype)
        kernels.attention_decode_mma(qd, want, k, v, tables, row_seq, positions, nh, nkv, hd, ps, hd ** -0.5, window,
                                     splits, torch.empty(n * nh * 4 * splits * hd, device=DEV),
                                     torch.empty(n * nh * 4 * splits * 2, device=DEV),
                                     torch.zeros(n * nkv, dtype=torch.int32, device=DEV), status)
        got = torch.full((n, nh * hd), 7.0, device=DEV, dtype=dtype)
        rc = fn(qd.data_ptr(), qd.stride(0), got.data_ptr(), got.stride(0), k.data_ptr(), v.data_ptr(),
                tables.data_ptr(), tables.shape[1], row_seq.data_ptr(), positions.data_ptr(), n, nh, nkv, hd, ps,
                k.shape[0], hd ** -0.5, 0, splits, status.data_ptr(), stream)
        assert rc == 0, lib.gb_last_error().decode()
        torch.cuda.synchronize()
        assert int(status) == 0
        assert (got.float() - want.float()).abs().max() <= tol(dtype, 2)
        ref = ref_attention(q, dense, list(range(n)), [l - 1 for l in lens], nh, nkv, hd ** -0.5, window)
        assert (got.cpu().double().reshape(n, nh, hd) - ref).abs().max() <= tol(dtype, 2)

    # a call that would not fit the built-in array is refused, loudly, and nothing runs
    big = lib.gb_attention_decode_noalloc_bytes(64, 32, 8, 128, 64)
    assert big > 8 << 20
    rc = fn(qd.data_ptr(), qd.stride(0), got.data_ptr(), got.stride(0), k.data_ptr(), v.data_ptr(), tables.data_ptr(),
            tables.shape[1], row_seq.data_ptr(), positions.data_ptr(), 64, 32, 8, 128, ps, k.shape[0], 0.1, 0, 64,
            status.data_ptr(), stream)
    assert rc != 0 and "scratch" in lib.gb_last_error().decode()
