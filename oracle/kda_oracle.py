"""CPU oracle for Kimi Delta Attention (KDA).  TEST INFRASTRUCTURE ONLY.

This module restates the KDA recurrence on the CPU in float64.  It is the checker for the CUDA
path: only the tests, the smoke entry and the benchmark's CPU-baseline leg may import it.  The
shipped package never imports it and has no CPU fallback.

Parity status: the NVlabs/kda repository contains no implementation, test or golden vector for this
operator ("parity unpinned" by that repository).  The recurrence restated here is the published one,

    S_t = (I - beta_t k_t k_t^T) Diag(exp g_t) S_{t-1} + beta_t k_t v_t^T,      o_t = scale * S_t^T q_t

and its operation order (decay, then delta update, then read-out with the updated state) follows the
token loop of flash-linear-attention 0.5.1 (git bb324a3), fla/ops/kda/naive.py:59-63 and
fla/ops/kda/fused_recurrent.py:146-192.  The oracle is pinned against outputs of that package's
`naive_recurrent_kda`, generated in the build container and committed under tests/golden/ together
with the generating script.

Everything here is differentiable torch code, so float64 autograd through `recurrent_kda` is the
gradient oracle.
"""
from __future__ import annotations

import torch

L2_EPS = 1e-6  # fla/modules/l2norm.py:138-187 uses rsqrt(sum(x^2) + 1e-6)


def l2norm(x: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(sum(x^2) + eps) over the last dim (fla/modules/l2norm.py:138-187)."""
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + L2_EPS)


def _scan_one(q, k, v, g, beta, scale, S):
    """One batch of equal-length sequences.  q,k,g: [B,T,H,K]; v: [B,T,H,V]; beta: [B,T,H];
    S: [B,H,K,V].  Returns (o [B,T,H,V], S_final).  fla/ops/kda/naive.py:57-63."""
    T = q.shape[1]
    outs = []
    for t in range(T):
        q_t, k_t, v_t, g_t, b_t = q[:, t], k[:, t], v[:, t], g[:, t], beta[:, t]
        S = S * g_t.exp().unsqueeze(-1)                                    # Diag(exp g_t) S
        resid = v_t - torch.einsum("bhk,bhkv->bhv", k_t, S)                # v_t - S^T k_t
        S = S + torch.einsum("bhk,bhv->bhkv", b_t.unsqueeze(-1) * k_t, resid)
        outs.append(scale * torch.einsum("bhk,bhkv->bhv", q_t, S))        # o_t = scale S_t^T q_t
    o = torch.stack(outs, dim=1) if outs else q.new_zeros(q.shape[0], 0, q.shape[2], v.shape[-1])
    return o, S


def recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                  cu_seqlens=None, use_qk_l2norm=False, dtype=torch.float64):
    """Token-by-token KDA in `dtype` (float64 by default).

    Shapes follow the operator API (fla/ops/kda/chunk.py:167-188): q,k,g [B,T,H,K], v [B,T,H,V],
    beta [B,T,H], initial_state [N,H,K,V]; with `cu_seqlens` (length N+1) B must be 1 and every
    sequence is scanned on its own from its own initial state.  Returns (o, final_state) in `dtype`.
    """
    q, k, v, g, beta = (x.to(dtype) for x in (q, k, v, g, beta))
    if use_qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    if cu_seqlens is None:
        S0 = q.new_zeros(B, H, K, V) if initial_state is None else initial_state.to(dtype)
        o, S = _scan_one(q, k, v, g, beta, scale, S0)
        return o, (S if output_final_state else None)
    if B != 1:
        raise ValueError("cu_seqlens requires batch size 1")
    cu = [int(x) for x in cu_seqlens]
    N = len(cu) - 1
    if initial_state is not None and initial_state.shape[0] != N:
        raise ValueError("initial_state.shape[0] must equal the number of sequences")
    outs, finals = [], []
    for n in range(N):
        s, e = cu[n], cu[n + 1]
        S0 = q.new_zeros(1, H, K, V) if initial_state is None else initial_state[n:n + 1].to(dtype)
        o_n, S_n = _scan_one(q[:, s:e], k[:, s:e], v[:, s:e], g[:, s:e], beta[:, s:e], scale, S0)
        outs.append(o_n)
        finals.append(S_n)
    o = torch.cat(outs, dim=1)
    return o, (torch.cat(finals, dim=0) if output_final_state else None)


def recurrent_kda_grads(q, k, v, g, beta, do, dht=None, scale=None, initial_state=None,
                        cu_seqlens=None, use_qk_l2norm=False):
    """float64 autograd through `recurrent_kda`.  Returns dict with o, ht, dq, dk, dv, dg, dbeta, dh0.
    The loss is <o, do> + <ht, dht>, i.e. `do`/`dht` are the upstream gradients."""
    leaves = [x.detach().to(torch.float64).requires_grad_(True) for x in (q, k, v, g, beta)]
    h0 = None
    if initial_state is not None:
        h0 = initial_state.detach().to(torch.float64).requires_grad_(True)
    o, ht = recurrent_kda(*leaves, scale=scale, initial_state=h0, output_final_state=True,
                          cu_seqlens=cu_seqlens, use_qk_l2norm=use_qk_l2norm)
    loss = (o * do.to(torch.float64)).sum()
    if dht is not None:
        loss = loss + (ht * dht.to(torch.float64)).sum()
    wrt = leaves + ([h0] if h0 is not None else [])
    grads = torch.autograd.grad(loss, wrt)
    out = dict(o=o.detach(), ht=ht.detach(), dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3],
               dbeta=grads[4], dh0=(grads[5] if h0 is not None else None))
    return out


# ------------------------------------------------------------------------------------------------
# error measures used by every parity test
# ------------------------------------------------------------------------------------------------

def max_norm_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max|x - ref| / max|ref|   (the 'fp32 mode' and 'bf16 relative error' measure)."""
    x, ref = x.detach().double().cpu(), ref.detach().double().cpu()
    denom = ref.abs().max().item()
    if denom == 0.0:
        return (x - ref).abs().max().item()
    return (x - ref).abs().max().item() / denom


def rel_l2_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """||x - ref||_2 / ||ref||_2."""
    x, ref = x.detach().double().cpu(), ref.detach().double().cpu()
    denom = ref.norm().item()
    if denom == 0.0:
        return (x - ref).norm().item()
    return (x - ref).norm().item() / denom


def cosine(x: torch.Tensor, ref: torch.Tensor) -> float:
    x, ref = x.detach().double().cpu().flatten(), ref.detach().double().cpu().flatten()
    nx, nr = x.norm().item(), ref.norm().item()
    if nx == 0.0 and nr == 0.0:
        return 1.0
    if nx == 0.0 or nr == 0.0:
        return 0.0
    return float((x @ ref).item() / (nx * nr))


def assert_bf16_parity(x: torch.Tensor, ref: torch.Tensor, name: str = "", rel: float = 2e-2, cos: float = 0.9999) -> None:
    """The bf16-mode bar, read both ways: max|x - ref| / max|ref| <= rel AND ||x - ref||_2 / ||ref||_2 <= rel, and
    cosine >= cos; every value finite."""
    assert torch.isfinite(x.detach().float()).all(), f"{name}: non-finite values"
    e_max, e_l2, c = max_norm_err(x, ref), rel_l2_err(x, ref), cosine(x, ref)
    assert e_max <= rel and e_l2 <= rel and c >= cos, f"{name}: max-normalised {e_max:.3e}, relative L2 {e_l2:.3e}, cosine {c:.6f}"


# ---- gate front end -------------------------------------------------------------------------------------
def kda_gate(g_raw, A_log, dt_bias=None, lower_bound=None, dtype=torch.float64):
    """Decay activation in front of the operator, differentiable, in `dtype`.

    g = -exp(A_log[h]) * softplus(g_raw + dt_bias[h, k])                    (fla/ops/kda/gate.py:26-55)
    g = lower_bound * sigmoid(exp(A_log[h]) * (g_raw + dt_bias[h, k]))      (fla/ops/kda/gate.py:58-69)
    g_raw [..., H, K]; A_log [H]; dt_bias [H*K] or None.  softplus switches to the identity above 20
    (fla/ops/utils/softplus.py:17-26), which in float64 differs from log1p(exp(x)) by < 3e-9.
    """
    H, K = g_raw.shape[-2:]
    x = g_raw.to(dtype)
    if dt_bias is not None:
        x = x + dt_bias.to(dtype).view(H, K)
    a = A_log.to(dtype).view(H, 1).exp()
    if lower_bound is None:
        return -a * torch.where(x > 20.0, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))
    return lower_bound * torch.sigmoid(a * x)


def beta_sigmoid(beta_raw, dtype=torch.float64):
    """beta = sigmoid(beta_raw) (fla/ops/kda/chunk.py:58-61)."""
    return torch.sigmoid(beta_raw.to(dtype))
