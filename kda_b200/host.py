"""Host-resident batches: forward+backward of `chunk_kda` for inputs that live in pinned host memory.

The (sequence, head) recurrences of a batch are independent, so an equal-length batch is cut along the
batch axis and the slices are pipelined over three CUDA streams: slice s+1 is copied host->device while
slice s is computed and the results of slice s-1 are copied device->host.  PCIe is full duplex, so a step
costs about max(bytes in, bytes out) / link bandwidth instead of their sum plus the compute time.
"""
from __future__ import annotations

import torch

from .ops import chunk_kda

_IN = ("q", "k", "v", "g", "beta", "h0", "do", "dht")
_OUT = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")


class HostPipeline:
    """Re-usable pipeline for one device; keeps its streams and staging buffers between calls."""

    def __init__(self, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._stage = {}

    def _staging(self, slot, name, like):
        key = (slot, name, tuple(like.shape), like.dtype)
        buf = self._stage.get(key)
        if buf is None:
            buf = torch.empty(like.shape, dtype=like.dtype, device=self.device)
            self._stage[key] = buf
        return buf

    def fwd_bwd(self, host_in: dict, host_out: dict | None = None, slices: int | None = None, **kwargs) -> dict:
        """host_in: pinned CPU tensors q,k,v,g,beta,do (+ h0, dht); returns pinned CPU tensors
        o, ht, dq, dk, dv, dg, dbeta (+ dh0).  Blocks until every result has landed in host memory."""
        B = host_in["q"].shape[0]
        n = B if slices is None else max(1, min(int(slices), B))
        bounds = [(i * B // n, (i + 1) * B // n) for i in range(n)]
        has_h0 = host_in.get("h0") is not None
        if host_out is None:
            host_out = {}
        compute = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(compute)
        self.s_in.wait_event(start)
        self.s_out.wait_event(start)
        done_ev = [None] * n
        keep = []
        for s, (b0, b1) in enumerate(bounds):
            slot = s & 1
            with torch.cuda.stream(self.s_in):
                if s >= 2:
                    self.s_in.wait_event(done_ev[s - 2])          # the staging slot is free again
                dev = {}
                for name in _IN:
                    t = host_in.get(name)
                    if t is None:
                        continue
                    src = t[b0:b1]
                    dst = self._staging(slot, name, src)
                    dst.copy_(src, non_blocking=True)
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
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done_ev[s])
                for name, t in outs.items():
                    full = host_out.get(name)
                    if full is None:
                        shape = (B,) + tuple(t.shape[1:])
                        full = torch.empty(shape, dtype=t.dtype, pin_memory=True)
                        host_out[name] = full
                    full[b0:b1].copy_(t, non_blocking=True)
                    t.record_stream(self.s_out)
            keep.append(outs)
        end = torch.cuda.Event()
        end.record(self.s_out)
        compute.wait_event(end)          # the caller's stream sees the step as one unit
        end.synchronize()
        return host_out


_default: dict = {}


def chunk_kda_fwd_bwd_host(host_in: dict, host_out: dict | None = None, slices: int | None = None, **kwargs) -> dict:
    """Module-level convenience over a per-device `HostPipeline`."""
    dev = torch.cuda.current_device()
    pipe = _default.get(dev)
    if pipe is None:
        pipe = _default[dev] = HostPipeline(torch.device("cuda", dev))
    return pipe.fwd_bwd(host_in, host_out, slices, **kwargs)
