"""The device status word of the chunked kernels is visible to the host: a bounded wait that runs out and a
cu_seqlens that does not fit the tensors both end in a KdaError in checked mode (KDA_B200_CHECK=1) instead of
silently incomplete outputs, and the GPU stays usable afterwards.  Nothing here faults or hangs a GPU: the wait
that gives up is a wait on a barrier that nothing arrives at, with the library's own poll limit."""
import ctypes as C
import os

import pytest
import torch

from kda_b200.inputs import make_inputs

pytestmark = pytest.mark.gpu


def _debug_lib():
    from kda_b200 import build
    lib = C.CDLL(build.DEBUG_LIB)
    lib.kda_b200_debug_wait_giveup.restype = C.c_int
    lib.kda_b200_debug_wait_giveup.argtypes = [C.c_void_p, C.c_uint, C.c_void_p]
    return lib


def test_a_wait_that_runs_out_is_reported_and_the_gpu_stays_usable():
    from kda_b200 import _lib, chunk_kda
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    assert _lib.chunk_status(ws.data_ptr()) == 0
    rc = _debug_lib().kda_b200_debug_wait_giveup(ws.data_ptr(), 0x2, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert _lib.chunk_status(ws.data_ptr()) == 0x2          # the host sees the bit after the stream has drained
    with pytest.raises(_lib.KdaError, match="a product did not complete"):
        _lib.check_chunk_status(ws.data_ptr(), "test")
    # the context is intact: an ordinary call still works and reports nothing
    d = {n: t.cuda() for n, t in make_inputs(1, 100, 2, 128, 128, torch.bfloat16, seed=1, h0_std=0.02).items() if t is not None}
    with torch.no_grad():
        o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"])
    assert torch.isfinite(o.float()).all()


@pytest.mark.parametrize("cu_list", [[0, 300], [0, 150, 100, 200], [-64, 200]])
def test_inconsistent_cu_seqlens_is_reported_not_executed(cu_list):
    """cu_seqlens beyond the tensors, not monotone, or negative: the tables kernel sets KDA_STATUS_BAD_CU_SEQLENS and
    leaves empty tables, so no kernel reads or writes past a buffer; o keeps its previous contents."""
    from kda_b200 import _lib
    lib = _lib.load()
    tokens, H, N = 200, 2, len(cu_list) - 1
    d = {n: t.cuda().contiguous() for n, t in make_inputs(1, tokens, H, 128, 128, torch.bfloat16, seed=2, h0_std=0.02, n_states=N).items()
         if t is not None}
    cu = torch.tensor(cu_list, dtype=torch.int32, device="cuda")
    ws = torch.empty(lib.kda_chunk_workspace_bytes(tokens, N, H, 128, 128, 0), dtype=torch.uint8, device="cuda")
    o = torch.full_like(d["v"], 7.0)
    a = _lib.ChunkArgs(q=d["q"].data_ptr(), k=d["k"].data_ptr(), v=d["v"].data_ptr(), g=d["g"].data_ptr(), beta=d["beta"].data_ptr(),
                       h0=d["h0"].data_ptr(), cu_seqlens=cu.data_ptr(), o=o.data_ptr(), workspace=ws.data_ptr(),
                       workspace_bytes=ws.numel(), tokens=tokens, N=N, H=H, K=128, V=128, io_dtype=_lib.KDA_BF16, scale=0.1)
    assert lib.kda_chunk_fwd(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    assert _lib.chunk_status(ws.data_ptr()) == 0x100
    assert bool((o == 7.0).all())


def test_checked_mode_raises_through_the_operator():
    from kda_b200 import _lib, chunk_kda
    assert os.environ.get("KDA_B200_CHECK") == "1"          # set for every GPU test by conftest
    d = {n: t.cuda() for n, t in make_inputs(1, 200, 2, 128, 128, torch.bfloat16, seed=3).items() if t is not None}
    cu = torch.tensor([0, 120, 260], dtype=torch.int32, device="cuda")          # 260 > 200 tokens
    with torch.no_grad(), pytest.raises(_lib.KdaError, match="cu_seqlens"):
        chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], cu_seqlens=cu)
