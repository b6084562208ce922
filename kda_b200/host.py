"""Host-resident batches: forward+backward of `chunk_kda` for inputs that live in pinned host memory.

The (sequence, head) recurrences of a batch are independent, so an equal-length batch is cut along the
batch axis (and, with strided copies, along the head axis) and the pieces are pipelined over three CUDA
streams: piece s+1 is copied host->device while piece s is computed and the results of piece s-1 are copied
device->host.  PCIe is full duplex, so a step
costs about max(bytes in, bytes out) / link bandwidth instead of their sum plus the compute time.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .ops import chunk_kda

_IN = ("q", "k", "v", "g", "beta", "h0", "do", "dht")
_OUT = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")


# which axis of each tensor is the head axis (None: no head axis to cut)
_HEAD_AXIS = dict(q=2, k=2, v=2, g=2, beta=2, do=2, o=2, dq=2, dk=2, dv=2, dg=2, dbeta=2, h0=1, dht=1, ht=1, dh0=1)


def _copy_heads(dst: torch.Tensor, src: torch.Tensor, b0: int, b1: int, h0: int, h1: int, name: str, to_device: bool, stream) -> None:
    """One strided copy of batch rows [b0, b1) and heads [h0, h1) between a full pinned host tensor and a dense device
    slice (`to_device`: src is the host tensor, dst the device slice; else the other way round)."""
    full, part = (src, dst) if to_device else (dst, src)
    ax = _HEAD_AXIS[name]
    H = full.shape[ax]
    inner = 1
    for d in full.shape[ax + 1:]:
        inner *= d
    es = full.element_size()
    width = (h1 - h0) * inner * es
    pitch = H * inner * es
    rows = b1 - b0
    for d in full.shape[1:ax]:
        rows *= d
    off = (b0 * (full[0].numel()) + h0 * inner) * es
    fptr = full.data_ptr() + off
    lib = _lib.load()
    if to_device:
        _lib.check(lib.kda_copy_rows_async(C.c_void_p(part.data_ptr()), width, C.c_void_p(fptr), pitch, width, rows,
                                           C.c_void_p(stream.cuda_stream)), "kda_copy_rows_async")
    else:
        _lib.check(lib.kda_copy_rows_async(C.c_void_p(fptr), pitch, C.c_void_p(part.data_ptr()), width, width, rows,
                                           C.c_void_p(stream.cuda_stream)), "kda_copy_rows_async")


class HostPipeline:
    """Re-usable pipeline for one device; keeps its streams and staging buffers between calls."""

    def __init__(self, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._stage = {}
        self._slot_free = [None, None]      # per staging slot: the event after which its tensors may be overwritten
        self._end = None                    # the event behind the last step's last copy-out

    def _staging(self, slot, name, shape, dtype):
        key = (slot, name, tuple(shape), dtype)
        buf = self._stage.get(key)
        if buf is None:
            buf = torch.empty(shape, dtype=dtype, device=self.device)
            self._stage[key] = buf
        return buf

    def synchronize(self) -> None:
        """Blocks until the results of every step issued so far have landed in host memory."""
        if self._end is not None:
            self._end.synchronize()

    def fwd_bwd(self, host_in: dict, host_out: dict | None = None, slices: int | None = None, head_groups: int | None = None,
                wait: bool = True, **kwargs) -> dict:
        """host_in: pinned CPU tensors q,k,v,g,beta,do (+ h0, dht); returns pinned CPU tensors
        o, ht, dq, dk, dv, dg, dbeta (+ dh0).  Blocks until every result has landed in host memory -- unless
        `wait=False`: then the call returns as soon as the step is queued, the results are valid after `synchronize()`,
        and the next step's copy-in overlaps this step's copy-out (a training loop over host-resident batches keeps both
        directions of the link busy; give consecutive steps different `host_out` buffers if step i's results are read
        while step i+1 runs).

        The batch is cut into `slices` along the batch axis and every slice into `head_groups` along the head axis
        (strided copies): the pipeline's fill and drain cost one piece each way, so more, smaller pieces bring the step
        closer to bytes / link bandwidth.  Defaults: one slice per batch row, no cut along the heads (a head cut needs
        q and v to have the same head count)."""
        B, H = host_in["q"].shape[0], host_in["v"].shape[2]
        n = B if slices is None else max(1, min(int(slices), B))
        G = 1 if head_groups is None else max(1, int(head_groups))
        assert H % G == 0 and (G == 1 or host_in["q"].shape[2] == H), "head_groups must divide H (and needs HV == H)"
        hg = H // G
        pieces = [(i * B // n, (i + 1) * B // n, j * hg, (j + 1) * hg) for i in range(n) for j in range(G)]
        has_h0 = host_in.get("h0") is not None
        if host_out is None:
            host_out = {}
        compute = torch.cuda.current_stream(self.device)
        if wait:
            start = torch.cuda.Event()
            start.record(compute)
            self.s_in.wait_event(start)
            self.s_out.wait_event(start)
        done_ev = [None] * len(pieces)
        keep = []
        for s, (b0, b1, h0, h1) in enumerate(pieces):
            slot = s & 1
            with torch.cuda.stream(self.s_in):
                if self._slot_free[slot] is not None:
                    self.s_in.wait_event(self._slot_free[slot])   # the staging slot is free again (also across steps)
                dev = {}
                for name in _IN:
                    t = host_in.get(name)
                    if t is None:
                        continue
                    shape = list(t.shape)
                    shape[0] = b1 - b0
                    if G > 1:
                        shape[_HEAD_AXIS[name]] = h1 - h0
                    dst = self._staging(slot, name, shape, t.dtype)
                    if G > 1:
                        _copy_heads(dst, t, b0, b1, h0, h1, name, True, self.s_in)
                    else:
                        dst.copy_(t[b0:b1], non_blocking=True)
                    dev[name] = dst
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            compute.wait_event(ev_in)
            leaves = [dev[nm].requires_grad_(True) for nm in ("q", "k", "v", "g", "beta")]
            if has_h0:
                leaves.append(dev["h0"].requires_grad_(True))
            o, ht = chunk_kda(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], initial_state=dev.get("h0"),
                              output_final_state=True, **kwargs)
            grads = torch.autograd.grad([o, ht], leaves, [dev["do"], dev.get("dht", torch.zeros_like(ht))])
            outs = dict(o=o.detach(), ht=ht.detach(), dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3], dbeta=grads[4])
            if has_h0:
                outs["dh0"] = grads[5]
            for nm in ("q", "k", "v", "g", "beta", "h0"):
                if nm in dev:
                    dev[nm].requires_grad_(False)
            done_ev[s] = torch.cuda.Event()
            done_ev[s].record(compute)
            self._slot_free[slot] = done_ev[s]
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done_ev[s])
                for name, t in outs.items():
                    full = host_out.get(name)
                    if full is None:
                        shape = list(t.shape)
                        shape[0] = B
                        shape[_HEAD_AXIS[name]] = host_in["q" if name in ("dq", "dk") else "v"].shape[2]
                        full = torch.empty(shape, dtype=t.dtype, pin_memory=True)
                        host_out[name] = full
                    if G > 1:
                        _copy_heads(full, t.contiguous(), b0, b1, h0, h1, name, False, self.s_out)
                    else:
                        full[b0:b1].copy_(t, non_blocking=True)
                    t.record_stream(self.s_out)
            keep.append(outs)
        end = torch.cuda.Event()
        end.record(self.s_out)
        self._end = end
        if wait:
            compute.wait_event(end)      # the caller's stream sees the step as one unit
            end.synchronize()
        return host_out


_default: dict = {}


def _pipe() -> HostPipeline:
    dev = torch.cuda.current_device()
    pipe = _default.get(dev)
    if pipe is None:
        pipe = _default[dev] = HostPipeline(torch.device("cuda", dev))
    return pipe


def chunk_kda_fwd_bwd_host(host_in: dict, host_out: dict | None = None, slices: int | None = None,
                           head_groups: int | None = None, wait: bool = True, **kwargs) -> dict:
    """Module-level convenience over a per-device `HostPipeline` (see `HostPipeline.fwd_bwd`)."""
    return _pipe().fwd_bwd(host_in, host_out, slices, head_groups, wait, **kwargs)


def host_synchronize() -> None:
    """Waits for every step queued with `wait=False` on the current device."""
    _pipe().synchronize()
