"""The product entry point that allocates nothing, called through its exported C symbol.

Some embedders cannot call cudaMalloc once they are running: they gave all the device memory they
may use to their own pools, or they must not synchronise the device.  For them the library exports
``tge_gemm_tcgen05_static_scratch``, which keeps the partial sums of its k-splits in a buffer that is
part of the library image.  This test calls it twice in a row through ctypes, with different shapes
and data (the second call meets whatever the first left in the shared buffer), and compares each
result with the regular entry point's.  It is collected last so that a run that stops at the first
failure has already run every other test; it passes alone in a fresh process as well.
"""
import ctypes

import pytest
import torch

from helpers import TOL, rel_error

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GEMM_STORE, GEMM_STORE_F32, GEMM_ADD_F32, GEMM_SWIGLU = 0, 1, 2, 3


def _symbol():
    from aegean_tge_b200 import ops
    lib = ops.core()
    fn = lib.tge_gemm_tcgen05_static_scratch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p]
    return ops, lib, fn


def _call(fn, x, w, bias, out, epilogue, status):
    M, K = x.shape
    return fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), None if bias is None else bias.data_ptr(),
              out.data_ptr(), out.stride(0), M, w.shape[0], K, epilogue, status.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_the_regular_entry_point_twice_in_a_row():
    ops, lib, fn = _symbol()
    status = ops.status_word()
    gen = torch.Generator().manual_seed(21)
    # two shapes with few output tiles and a long k: both are cut along k, so both use the scratch
    cases = [(8, 512, 2048, GEMM_STORE_F32), (24, 384, 3584, GEMM_ADD_F32)]
    for M, N, K, epilogue in cases:
        assert lib.tge_gemm_tcgen05_scratch_floats(M, N, K) > 0, "the case must use scratch to mean anything"
        x = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(DEV)
        w = (torch.randn(N, K, generator=gen) * 0.05).to(torch.bfloat16).to(DEV)
        bias = torch.randn(N, generator=gen).to(DEV)
        start = torch.randn(M, N, generator=gen).to(DEV)
        expected = start.clone()
        ops.linear(x, w, bias, epilogue, out=expected)                    # the existing entry point
        got = start.clone()
        rc = _call(fn, x, w, bias, got, epilogue, status)
        assert rc == 2, lib.tge_last_error()                              # product kernel + reduction kernel
        ops.check_status()
        assert rel_error(got, expected) < TOL[torch.float32]
        assert rel_error(got, (x.double() @ w.double().T + bias.double()
                               + (start.double() if epilogue == GEMM_ADD_F32 else 0.0))) < TOL[torch.float32]


def test_static_scratch_with_the_other_epilogues_and_the_two_sm_plan():
    """The reductions that read the shared buffer in other ways: the gated epilogue (pairs of partial sums), the
    bfloat16 store, and a product of more than 128 tokens that pairs two SMs on a tile and still cuts along k."""
    ops, lib, fn = _symbol()
    status = ops.status_word()
    gen = torch.Generator().manual_seed(22)
    plan = (ctypes.c_int * 4)()
    lib.tge_gemm_tcgen05_describe.restype = None
    lib.tge_gemm_tcgen05_describe.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    paired = None
    for M, N, K in ((160, 512, 4096), (192, 768, 8192), (256, 512, 8192), (144, 256, 16384)):
        lib.tge_gemm_tcgen05_describe(M, N, K, plan)
        if plan[0] == 1 and plan[3] > 1 and lib.tge_gemm_tcgen05_scratch_floats(M, N, K) <= 4 * 1024 * 1024:
            paired = (M, N, K)
            break
    cases = [(8, 512, 2048, GEMM_SWIGLU), (24, 384, 3584, GEMM_STORE)]
    if paired is not None:          # (the pair kernel can be switched off by the environment; then there is no such plan)
        cases.append((*paired, GEMM_STORE_F32))
    for M, N, K, epilogue in cases:
        assert lib.tge_gemm_tcgen05_scratch_floats(M, N, K) > 0
        x = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(DEV)
        w = (torch.randn(N, K, generator=gen) * 0.05).to(torch.bfloat16).to(DEV)
        bias = None if epilogue == GEMM_SWIGLU else torch.randn(N, generator=gen).to(DEV)
        shape = (M, N // 2) if epilogue == GEMM_SWIGLU else (M, N)
        dtype = torch.float32 if epilogue == GEMM_STORE_F32 else torch.bfloat16
        expected = ops.linear(x, w, bias, epilogue)
        got = torch.zeros(shape, dtype=dtype, device=DEV)
        rc = _call(fn, x, w, bias, got, epilogue, status)
        assert rc == 2, lib.tge_last_error()
        ops.check_status()
        assert torch.equal(got, expected)                 # the same kernels, the same order of sums
        product = x.double() @ w.double().T
        if epilogue == GEMM_SWIGLU:
            gate, up = product[:, 0::2], product[:, 1::2]
            reference = gate / (1.0 + torch.exp(-gate)) * up
        else:
            reference = product + bias.double()
        assert rel_error(got, reference) < TOL[dtype]


def test_static_scratch_refuses_what_does_not_fit():
    ops, lib, fn = _symbol()
    M, N, K = 256, 3584, 18944                    # cut in five along k: 4.6 M partial sums, the buffer holds 4 Mi
    assert lib.tge_gemm_tcgen05_scratch_floats(M, N, K) > 4 * 1024 * 1024
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
    out = torch.full((M, N), 7.0, device=DEV)
    rc = _call(fn, x, w, None, out, GEMM_STORE_F32, ops.status_word())
    assert rc < 0 and rc != -100
    message = lib.tge_last_error().decode()
    assert "built-in buffer holds 4194304" in message
    assert float(out.min()) == 7.0                # nothing was launched
