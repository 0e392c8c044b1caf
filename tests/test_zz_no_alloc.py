"""The allocation-free split-K GEMM entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory when they need a product: an engine
that planned all of its memory up front, or an embedding without PyTorch's allocator. For them
the library exports `kmoss_gemm_splitk_noalloc`, whose partial-sum scratch is a fixed array
inside the library. This test calls it twice in a row (the scratch keeps the first call's
contents) and compares each result with the regular entry point, `ops.native.gemm` with the
same split count, whose scratch is an ordinary torch tensor.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(x, y):
    return ((x.float() - y.float()).norm() / y.float().norm().clamp_min(1e-12)).item()


def _symbol():
    from kohakumosstrainer_b200.ops import native

    native.load()
    lib = ctypes.CDLL(str(native.library_path()))
    fn = lib.kmoss_gemm_splitk_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_long, ctypes.c_long, ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def test_two_calls_match_the_regular_entry_point():
    from kohakumosstrainer_b200.ops import native

    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(11)
    # adapter-gradient shapes: d_up[out, r] = dY^T[out, tokens] . T[tokens, r], both operands MN-major
    for (M, N, K, splits) in ((3072, 16, 8192, 8), (1024, 64, 4096, 5)):
        dy = torch.randn(K, M, device="cuda", generator=g).bfloat16()
        t = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        out = torch.full((M, N), float("nan"), device="cuda")
        rc = fn(dy.data_ptr(), t.data_ptr(), out.data_ptr(), M, N, K, dy.stride(0), t.stride(0), out.stride(0), 1, 1,
                splits, stream)
        assert rc == 0
        expect = native.gemm(dy, t, a_mn=True, b_mn=True, out_dtype=torch.float32, splits=splits)
        torch.cuda.synchronize()
        assert torch.isfinite(out).all()
        assert _rel(out, expect) < 2e-3
        assert _rel(out, dy.float().t() @ t.float()) < 2e-3
    native.check_status()


def test_rejects_sizes_beyond_the_scratch():
    fn = _symbol()
    a = torch.zeros(8, 8, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8, 8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # 64 splits x 4096 x 4096 x 4 bytes = 4 GiB of partial sums: far beyond 16 MiB
    assert fn(a.data_ptr(), a.data_ptr(), out.data_ptr(), 4096, 4096, 4096, 4096, 4096, 4096, 0, 0, 64, stream) == -1
    assert fn(a.data_ptr(), a.data_ptr(), out.data_ptr(), 8, 8, 8, 8, 8, 8, 0, 0, 1, stream) == -2
    assert fn(None, a.data_ptr(), out.data_ptr(), 8, 8, 8, 8, 8, 8, 0, 0, 2, stream) == -2
