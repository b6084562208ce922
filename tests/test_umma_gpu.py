"""GPU check of the tcgen05 building blocks (shared-memory descriptors for K-major and MN-major 128-byte
swizzled bf16 tiles, instruction descriptor, TMEM allocate / load): one CTA computes a 128 x N x 128
product on the 5th-generation tensor cores; the result must equal the fp32 product of the same bf16 data."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N", [64, 128])
@pytest.mark.parametrize("a_mn,b_mn,neg_b", [(0, 0, 0), (1, 0, 0), (0, 1, 0), (1, 1, 1)])
def test_umma_gemm(N, a_mn, b_mn, neg_b):
    from kda_b200 import _lib
    lib = _lib.load()
    fn = lib.kda_b200_debug_umma_gemm
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    g = torch.Generator().manual_seed(N + 2 * a_mn + b_mn)
    A = torch.randn(128, 128, generator=g).bfloat16().cuda()
    B = torch.randn(N, 128, generator=g).bfloat16().cuda()
    D = torch.full((128, N), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = fn(A.data_ptr(), B.data_ptr(), D.data_ptr(), N, a_mn, b_mn, neg_b, status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded mbarrier wait gave up"
    ref = A.float() @ B.float().t()
    if neg_b:
        ref = -ref
    assert torch.isfinite(D).all()
    assert (D - ref).abs().max().item() <= 1e-3 * ref.abs().max().item()
