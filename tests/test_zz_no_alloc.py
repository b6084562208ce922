"""GPU test of kda_chunk_fwd_noalloc, the forward entry point for callers that cannot allocate device
memory (a serving process whose pool is frozen, a no-allocation region, a C caller with no allocator).

It is called through the C ABI exactly as such a caller would: inputs and outputs are passed, no
workspace.  Its results must equal those of kda_chunk_fwd (same kernels, so bit for bit — tighter than
the 2e-2 / 0.9999 bf16 tolerance of the other tests) on two calls in a row of different sizes, the
second of which finds the first call's bytes still in the shared array.  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from kda_b200.inputs import make_inputs

pytestmark = pytest.mark.gpu


def _call(lib, fn, d, cu, N, H, tokens, ws):
    from kda_b200 import _lib
    o = torch.empty_like(d["v"])
    ht = torch.empty(N, H, 128, 128, dtype=torch.float32, device="cuda")
    a = _lib.ChunkArgs(q=d["q"].data_ptr(), k=d["k"].data_ptr(), v=d["v"].data_ptr(), g=d["g"].data_ptr(),
                       beta=d["beta"].data_ptr(), h0=d["h0"].data_ptr(), cu_seqlens=cu.data_ptr(), o=o.data_ptr(),
                       ht=ht.data_ptr(), workspace=(ws.data_ptr() if ws is not None else None),
                       workspace_bytes=(ws.numel() if ws is not None else 0), tokens=tokens, N=N, H=H, K=128, V=128,
                       io_dtype=_lib.KDA_BF16, use_qk_l2norm=0, save_for_backward=0, scale=128 ** -0.5)
    rc = fn(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, o, ht


def test_noalloc_matches_regular_entry_point_twice():
    from kda_b200 import _lib
    lib = _lib.load()
    H = 2
    for call, (lens, seed) in enumerate((([200, 70], 41), ([100], 42))):
        tokens, N = sum(lens), len(lens)
        d = make_inputs(1, tokens, H, 128, 128, torch.bfloat16, seed=seed, h0_std=0.02, n_states=N)
        d = {n: t.cuda().contiguous() for n, t in d.items() if t is not None}
        cu = torch.tensor([0] + [sum(lens[:i + 1]) for i in range(N)], dtype=torch.int32, device="cuda")
        need = lib.kda_chunk_workspace_bytes(tokens, N, H, 128, 128, 0)
        assert need <= _lib.NOALLOC_SCRATCH_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc1, o1, h1 = _call(lib, lib.kda_chunk_fwd, d, cu, N, H, tokens, ws)
        before = torch.cuda.memory_allocated()
        rc2, o2, h2 = _call(lib, lib.kda_chunk_fwd_noalloc, d, cu, N, H, tokens, None)
        assert rc1 == 0 and rc2 == 0, (call, rc1, rc2)
        assert torch.cuda.memory_allocated() - before == o2.numel() * 2 + h2.numel() * 4   # only the outputs
        assert torch.isfinite(o2.float()).all() and torch.isfinite(h2).all()
        assert torch.equal(o1, o2), call
        assert torch.equal(h1, h2), call
        assert _lib.chunk_status(None) == 0 and _lib.chunk_status(ws.data_ptr()) == 0      # no bounded wait gave up
        del o1, h1, o2, h2, ws, d      # so that the next round's allocator bookkeeping starts clean


def test_noalloc_rejects_what_does_not_fit():
    from kda_b200 import _lib
    lib = _lib.load()
    d = {n: t.cuda() for n, t in make_inputs(1, 64, 2, 128, 128, torch.bfloat16, seed=1, h0_std=0.02).items() if t is not None}
    cu = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    a = _lib.ChunkArgs(q=d["q"].data_ptr(), k=d["k"].data_ptr(), v=d["v"].data_ptr(), g=d["g"].data_ptr(),
                       beta=d["beta"].data_ptr(), cu_seqlens=cu.data_ptr(), o=d["v"].data_ptr(),
                       tokens=1 << 20, N=1, H=32, K=128, V=128, io_dtype=_lib.KDA_BF16, scale=1.0)
    assert lib.kda_chunk_fwd_noalloc(C.byref(a), None) == -7          # KDA_E_LIMIT, nothing launched
    assert b"maximum" in lib.kda_b200_strerror(-7)
    a.tokens, a.H, a.save_for_backward = 64, 2, 1
    assert lib.kda_chunk_fwd_noalloc(C.byref(a), None) == -2          # forward only
    assert lib.kda_chunk_fwd_noalloc(None, None) == -1
