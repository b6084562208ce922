"""Test helper: calls the chunked entry points through the C ABI with every output and scratch buffer placed
inside a larger sentinel-filled allocation, so that a write outside a buffer shows up as a damaged margin
(compute-sanitizer's job, done by hand).  Not a test module."""
import ctypes as C

import torch

MARGIN = 4096          # bytes on each side of every guarded buffer; keeps 256-byte alignment
SENTINEL = 0xA5


class Guarded:
    """A device buffer of `nbytes` with MARGIN sentinel bytes before and after it."""

    def __init__(self, nbytes: int, device="cuda"):
        self.nbytes = int(nbytes)
        pad = (-self.nbytes) % 256
        self.raw = torch.full((MARGIN + self.nbytes + pad + MARGIN,), SENTINEL, dtype=torch.uint8, device=device)
        self.body = self.raw[MARGIN:MARGIN + self.nbytes]

    def view(self, dtype, shape):
        return self.body.view(dtype).view(shape)

    def ptr(self) -> int:
        return self.body.data_ptr()

    def margins_intact(self) -> bool:
        lo, hi = self.raw[:MARGIN], self.raw[MARGIN + self.nbytes:]
        return bool((lo == SENTINEL).all()) and bool((hi == SENTINEL).all())


def guarded_like(shape, dtype, device="cuda"):
    n = 1
    for s in shape:
        n *= s
    g = Guarded(n * torch.empty((), dtype=dtype).element_size(), device)
    return g, g.view(dtype, shape)


def chunk_fwd_bwd_guarded(d, cu, noalloc=False, l2=False):
    """Forward (+ backward unless `noalloc`) of the chunked kernels through the C ABI on the inputs in dict `d`
    (device tensors q,k,v,g,beta,h0,do,dht with a leading batch axis of 1 or more) and int32 device `cu`.
    Returns (outputs dict, list of (name, Guarded))."""
    from kda_b200 import _lib
    lib = _lib.load()
    H, K, V = d["v"].shape[-2], d["q"].shape[-1], d["v"].shape[-1]
    tokens = d["q"].shape[0] * d["q"].shape[1]
    N = cu.numel() - 1
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    guards, out = [], {}

    def mk(name, shape, dtype):
        g, t = guarded_like(shape, dtype)
        guards.append((name, g))
        out[name] = t
        return t

    o = mk("o", d["v"].shape, torch.bfloat16)
    ht = mk("ht", (N, H, K, V), torch.float32)
    save = 0 if noalloc else (1 | (2 if l2 else 0))
    a = _lib.ChunkArgs(q=d["q"].data_ptr(), k=d["k"].data_ptr(), v=d["v"].data_ptr(), g=d["g"].data_ptr(),
                       beta=d["beta"].data_ptr(), h0=d["h0"].data_ptr(), cu_seqlens=cu.data_ptr(), o=o.data_ptr(),
                       ht=ht.data_ptr(), tokens=tokens, N=N, H=H, K=K, V=V, io_dtype=_lib.KDA_BF16, use_qk_l2norm=int(l2),
                       save_for_backward=save, scale=K ** -0.5, HQ=d["q"].shape[-2])
    if noalloc:
        rc = lib.kda_chunk_fwd_noalloc(C.byref(a), st)
        torch.cuda.synchronize()
        assert rc == 0, rc
        assert _lib.chunk_status(None) == 0
        return out, guards
    ws = Guarded(lib.kda_chunk_workspace_bytes(tokens, N, H, K, V, save))
    guards.append(("workspace", ws))
    a.workspace, a.workspace_bytes = ws.ptr(), ws.nbytes
    rc = lib.kda_chunk_fwd(C.byref(a), st)
    torch.cuda.synchronize()
    assert rc == 0, rc
    assert _lib.chunk_status(ws.ptr()) == 0
    flags = int(l2) | (2 if d["q"].shape[-2] != H else 0) | (4 if l2 else 0)
    bws = Guarded(lib.kda_chunk_bwd_workspace_bytes(tokens, N, H, K, V, flags))
    guards.append(("bwd_workspace", bws))
    a.bwd_workspace, a.bwd_workspace_bytes = bws.ptr(), bws.nbytes
    a.d_o, a.d_ht = d["do"].data_ptr(), d["dht"].data_ptr()
    a.dq = mk("dq", d["q"].shape, torch.bfloat16).data_ptr()
    a.dk = mk("dk", d["k"].shape, torch.bfloat16).data_ptr()
    a.dv = mk("dv", d["v"].shape, torch.bfloat16).data_ptr()
    a.dg = mk("dg", d["g"].shape, torch.float32).data_ptr()
    a.dbeta = mk("dbeta", d["beta"].shape, torch.float32).data_ptr()
    a.dh0 = mk("dh0", (N, H, K, V), torch.float32).data_ptr()
    rc = lib.kda_chunk_bwd(C.byref(a), st)
    torch.cuda.synchronize()
    assert rc == 0, rc
    assert _lib.chunk_status(ws.ptr()) == 0
    return out, guards
