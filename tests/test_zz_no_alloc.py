"""The allocation-free GEMM entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need a split-K GEMM: an
FFN process whose device budget was fixed at admission time, or a plain C host without an allocator.
``xp_gemm_noalloc`` keeps the split-K workspace in a fixed array inside the library. Its output must
equal the ordinary entry point's (same kernel, same split factor), on two calls in a row — the
second call reuses the array with the first call's leftovers in it. This file sorts last so that a
run stopping at the first failure has already seen every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE, BAD_ARGUMENT = -1000, -1002


def _lib():
    from crosspool_b200 import native

    lib = native.kernels()
    lib.xp_gemm_noalloc.restype = C.c_int
    lib.xp_gemm_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.xp_gemm_noalloc_required_bytes.restype = C.c_longlong
    lib.xp_gemm_noalloc_required_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int]
    lib.xp_gemm_noalloc_status.restype = C.c_int
    lib.xp_gemm_noalloc_status.argtypes = [C.POINTER(C.c_uint), C.c_void_p]
    lib.xp_gemm_noalloc_strerror.restype = C.c_char_p
    lib.xp_gemm_noalloc_strerror.argtypes = [C.c_int]
    return lib


@pytest.mark.parametrize("rows,n,k,splits", [(8, 512, 2048, 4), (40, 1024, 3072, 3), (130, 256, 1024, 2), (5, 256, 512, 1)])
def test_matches_the_allocating_entry_point_twice_in_a_row(rows, n, k, splits):
    from crosspool_b200.ops import gemm

    lib = _lib()
    g = torch.Generator(device="cuda").manual_seed(rows + n + k)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x = (torch.randn(rows, k, device="cuda", generator=g) * 0.5).bfloat16()
        w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
        want = gemm.linear(x, w, splits=splits)
        got = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
        rc = lib.xp_gemm_noalloc(w.data_ptr(), x.data_ptr(), got.data_ptr(), n, k, rows, splits, stream)
        assert rc == 0, lib.xp_gemm_noalloc_strerror(rc)
        torch.cuda.synchronize()
        gemm.check_status(x.device)                      # the allocating call's status word
        st = C.c_uint(99)
        assert lib.xp_gemm_noalloc_status(C.byref(st), stream) == 0 and st.value == 0   # and this entry point's own
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        ref = x.float() @ w.float().t()
        torch.testing.assert_close(got.float(), ref, atol=2e-2, rtol=2e-2)


def test_refuses_problems_beyond_the_fixed_scratch_without_launching():
    lib = _lib()
    rows, n, k, splits = 256, 8192, 8192, 8
    assert lib.xp_gemm_noalloc_required_bytes(n, k, rows, splits) > (8 << 20)
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros(rows, k, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(n, k, dtype=torch.bfloat16, device="cuda")
    rc = lib.xp_gemm_noalloc(w.data_ptr(), x.data_ptr(), out.data_ptr(), n, k, rows, splits,
                             torch.cuda.current_stream().cuda_stream)
    assert rc == TOO_LARGE
    assert b"scratch" in lib.xp_gemm_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())  # nothing ran
    assert lib.xp_gemm_noalloc(None, x.data_ptr(), out.data_ptr(), n, k, rows, 1, None) == BAD_ARGUMENT
