"""GPU check of the tcgen05 building blocks (shared-memory descriptors for K-major and MN-major 128-byte
swizzled bf16 tiles, instruction descriptor, TMEM allocate / load): one CTA computes a 128 x N x 128
product on the 5th-generation tensor cores; the result must equal the fp32 product of the same bf16 data."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


CASES = [  # M, N, NB (rows of B in shared memory), n_off, a_mn, b_mn, neg_b
    (128, 64, 64, 0, 0, 0, 0), (128, 64, 64, 0, 1, 0, 0), (128, 64, 64, 0, 0, 1, 0), (128, 64, 64, 0, 1, 1, 1),
    (128, 128, 128, 0, 0, 0, 0), (128, 128, 128, 0, 1, 0, 0), (128, 128, 128, 0, 0, 1, 0), (128, 128, 128, 0, 1, 1, 1),
    (64, 64, 64, 0, 0, 0, 0), (64, 64, 64, 0, 1, 1, 0), (64, 128, 128, 0, 1, 0, 0),
    (128, 16, 64, 16, 1, 0, 0), (128, 16, 64, 48, 1, 0, 0), (128, 16, 64, 32, 1, 1, 0), (128, 16, 64, 0, 0, 1, 0),
    (64, 16, 64, 16, 0, 0, 0),
    (128, 32, 64, 0, 0, 1, 0), (128, 32, 64, 32, 1, 1, 0), (64, 32, 64, 0, 0, 1, 0), (128, 32, 64, 16, 1, 0, 0),
]


@pytest.mark.parametrize("M,N,NB,n_off,a_mn,b_mn,neg_b", CASES)
def test_umma_gemm(M, N, NB, n_off, a_mn, b_mn, neg_b):
    from kda_b200 import build
    lib = C.CDLL(build.DEBUG_LIB)          # development checks live in their own library, not in libkda_b200.so
    fn = lib.kda_b200_debug_umma_gemm
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                   C.c_int, C.c_int, C.c_int]
    g = torch.Generator().manual_seed(N + 2 * a_mn + b_mn + M + n_off)
    A = torch.randn(128, 128, generator=g).bfloat16().cuda()      # M = 64 uses the first 64 rows
    B = torch.randn(NB, 128, generator=g).bfloat16().cuda()
    D = torch.full((M, N), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = fn(A.data_ptr(), B.data_ptr(), D.data_ptr(), N, a_mn, b_mn, neg_b, status.data_ptr(),
            torch.cuda.current_stream().cuda_stream, M, NB, n_off)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded mbarrier wait gave up"
    ref = A[:M].float() @ B[n_off:n_off + N].float().t()
    if neg_b:
        ref = -ref
    assert torch.isfinite(D).all()
    assert (D - ref).abs().max().item() <= 1e-3 * ref.abs().max().item()
