"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark workloads.

q, k ~ N(0,1) then L2-normalised per head-row; v ~ N(0,1); beta = sigmoid(N(0,1)) [B,T,H];
g = -exp(a_h) * softplus(x), x ~ N(0,1) [B,T,H,K], a_h = log U(1,16) per head (the decay
parameter initialisation of fla/layers/kda.py:178).  Everything is generated on the CPU from one
`torch.Generator` so that a given (workload, seed) is the same tensor on every machine, then cast.
"""
from __future__ import annotations

import dataclasses
import math

import torch


@dataclasses.dataclass(frozen=True)
class Workload:
    name: str
    B: int
    T: int
    H: int
    K: int
    V: int
    dtype: torch.dtype
    backward: bool
    h0_std: float           # 0 -> zero initial state
    n_seqs: int = 0          # >0 -> variable-length packed (B must be 1, T = sum of lengths)
    min_len: int = 0
    max_len: int = 0
    steps: int = 1           # decode: consecutive single-token steps


WORKLOADS = {
    # CPU-runnable fp32 forward
    "fwd_fp32_small": Workload("fwd_fp32_small", 1, 256, 2, 64, 64, torch.float32, False, 0.0),
    # bf16 forward prefill at the production head shape
    "prefill_bf16": Workload("prefill_bf16", 4, 4096, 32, 128, 128, torch.bfloat16, False, 0.02),
    # bf16 training forward+backward (the headline metric's workload)
    "train_bf16": Workload("train_bf16", 8, 8192, 32, 128, 128, torch.bfloat16, True, 0.02),
    # variable-length packed forward+backward
    "varlen_bf16": Workload("varlen_bf16", 1, 0, 32, 128, 128, torch.bfloat16, True, 0.02,
                            n_seqs=64, min_len=128, max_len=16384),
    # float32 training (the exact token-recurrent kernels); not one of the five stated workloads: a measurement case
    "train_fp32": Workload("train_fp32", 8, 2048, 32, 128, 128, torch.float32, True, 0.02),
    # decode: 1024 sequences, one token each, 256 consecutive steps
    "decode": Workload("decode", 1024, 1, 32, 128, 128, torch.bfloat16, False, 0.02, steps=256),
}


def varlen_lengths(n_seqs: int, min_len: int, max_len: int, seed: int = 0) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(min_len, max_len + 1, (n_seqs,), generator=gen).tolist()


def cu_seqlens_from_lengths(lengths) -> torch.Tensor:
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + int(n))
    return torch.tensor(cu, dtype=torch.int32)


def make_inputs(B, T, H, K, V, dtype=torch.bfloat16, seed=0, h0_std=0.0, n_states=None,
                backward=False, device="cpu", generate_on_device=False):
    """Returns a dict with q,k,v,g,beta,(h0),(do,dht).  q/k/v/do in `dtype`; g, beta, h0, dht fp32.

    By default the values come from a CPU generator (the same tensors on every machine) and are then moved to
    `device`.  `generate_on_device=True` draws them on `device` from that device's own seeded generator instead:
    the same distributions, a different (still seeded) stream -- for the largest workloads, whose float32
    staging tensors would need tens of GB of host memory and minutes of CPU time."""
    gdev = device if generate_on_device else "cpu"
    gen = torch.Generator(device=gdev).manual_seed(seed)
    rn = lambda *shape: torch.randn(*shape, generator=gen, device=gdev)      # noqa: E731
    q = rn(B, T, H, K)
    q = (q / q.norm(dim=-1, keepdim=True)).to(dtype)
    k = rn(B, T, H, K)
    k = (k / k.norm(dim=-1, keepdim=True)).to(dtype)
    v = rn(B, T, H, V).to(dtype)
    beta = torch.sigmoid(rn(B, T, H))
    a = torch.log(1.0 + 15.0 * torch.rand(H, generator=gen, device=gdev))            # a_h = log U(1,16)
    g = -torch.exp(a).view(1, 1, H, 1) * torch.nn.functional.softplus(rn(B, T, H, K))
    out = dict(q=q, k=k, v=v, g=g.float(), beta=beta.float())
    N = B if n_states is None else n_states
    if h0_std > 0:
        out["h0"] = (rn(N, H, K, V) * h0_std).float()
    else:
        out["h0"] = None
    if backward:
        out["do"] = rn(B, T, H, V).to(dtype)
        out["dht"] = (rn(N, H, K, V) * 0.01).float()
    if device != "cpu" and not generate_on_device:
        out = {n: (t.to(device) if t is not None else None) for n, t in out.items()}
    return out


def make_workload(name: str, seed: int = 0, device="cpu", scale_down: int = 1, generate_on_device=False):
    """Inputs of a named workload.  `scale_down` divides B (or the number of packed sequences) to
    make a smaller case with the same per-sequence shape.  The packed lengths always come from the CPU generator."""
    w = WORKLOADS[name]
    if w.n_seqs:
        lengths = varlen_lengths(max(1, w.n_seqs // scale_down), w.min_len, w.max_len, seed)
        cu = cu_seqlens_from_lengths(lengths)
        d = make_inputs(1, int(cu[-1]), w.H, w.K, w.V, w.dtype, seed, w.h0_std, n_states=len(lengths),
                        backward=w.backward, device=device, generate_on_device=generate_on_device)
        d["cu_seqlens"] = cu.to(device) if device != "cpu" else cu
        return d
    d = make_inputs(max(1, w.B // scale_down), w.T, w.H, w.K, w.V, w.dtype, seed, w.h0_std,
                    backward=w.backward, device=device, generate_on_device=generate_on_device)
    d["cu_seqlens"] = None
    return d


# ---- algorithmic work per (token, head), chunk C = 64:  GEMM = 2mnk, triangular products counted full,
# ---- the 64x64 unit-lower-triangular inverse counted as (2/3) C^2 per token; recompute not counted.

def flops_per_token_head(K=128, V=128, C=64, backward=True) -> float:
    fwd = 2 * C * (3 * K + 2 * V) + 6 * K * V + (2.0 / 3.0) * C * C
    bwd = 12 * K * V + 12 * C * K + 8 * C * V + 4 * C * C
    return fwd + (bwd if backward else 0.0)


def min_hbm_bytes_per_token_head(K=128, V=128, backward=True) -> int:
    fwd = 2 * K + 2 * K + 2 * V + 4 * K + 4 + 2 * V              # q,k,v bf16 + g fp32 + beta fp32 in, o bf16 out
    bwd = (2 * K + 2 * K + 2 * V + 4 * K + 4 + 2 * V) + (2 * K + 2 * K + 2 * V + 4 * K + 4)
    return fwd + (bwd if backward else 0)


def decode_bytes_per_seq_head(K=128, V=128) -> int:
    return 2 * K * V * 4 + (2 * K + 2 * K + 2 * V + 4 * K + 4 + 2 * V)


def default_scale(K: int) -> float:
    return 1.0 / math.sqrt(K)
