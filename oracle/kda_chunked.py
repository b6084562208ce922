"""Chunked restatement of KDA forward and backward in float64.  TEST INFRASTRUCTURE ONLY.

The CUDA kernels evaluate the recurrence chunk by chunk (64 tokens) with the UT/WY transform and
hand-derived gradients.  This file writes exactly those formulas with dense float64 tensors so that
they can be checked against float64 autograd through the token-by-token oracle
(oracle/kda_oracle.py) on the CPU, independently of any GPU.  The forward decomposition is the one of
flash-linear-attention 0.5.1 (fla/ops/kda/naive.py:69-166, fla/ops/kda/chunk_fwd.py:20-134); the
backward identities were derived for this project and are pinned by tests/test_oracle.py.

Per chunk (G = inclusive cumsum of g inside the chunk, Gam = exp(G), D[t,j] = exp(G_t - G_j), j<=t):
    Akk[t,j] = beta_t <k_t * D[t,j], k_j>  (j<t)        Aqk[t,j] = scale <q_t * D[t,j], k_j>  (j<=t)
    Tm = (I + Akk)^-1      w = Tm (beta * k * Gam)      u = Tm (beta * v)
    qg = scale q Gam       kg = k exp(G_last - G)
    v_new = u - w h        o = qg h + Aqk v_new         h' = Diag(Gam_last) h + kg^T v_new
"""
from __future__ import annotations

import torch

C = 64


def _pad(x, n):
    if x.shape[0] == n:
        return x
    pad = x.new_zeros((n - x.shape[0],) + tuple(x.shape[1:]))
    return torch.cat([x, pad], 0)


def chunk_quantities(q, k, v, g, beta, scale):
    """All state-independent per-chunk quantities for one (sequence, head) chunk (padded to C)."""
    G = g.cumsum(0)
    Gam = G.exp()
    diff = G[:, None, :] - G[None, :, :]                                     # [t, j, K]
    idx = torch.arange(C)
    low = idx[:, None] >= idx[None, :]
    D = torch.where(low[:, :, None], diff, torch.full_like(diff, -float("inf"))).exp()
    rawkk = torch.einsum("tk,tjk,jk->tj", k, D, k)
    rawqk = torch.einsum("tk,tjk,jk->tj", q, D, k)
    strict = idx[:, None] > idx[None, :]
    Akk = torch.where(strict, beta[:, None] * rawkk, torch.zeros_like(rawkk))
    Aqk = torch.where(low, scale * rawqk, torch.zeros_like(rawqk))
    Tm = torch.linalg.inv(torch.eye(C, dtype=q.dtype) + Akk)
    kgam = k * Gam
    w = Tm @ (beta[:, None] * kgam)
    u = Tm @ (beta[:, None] * v)
    qg = scale * q * Gam
    decay_to_end = (G[-1:, :] - G).exp()
    kg = k * decay_to_end
    return dict(G=G, Gam=Gam, D=D, rawkk=rawkk, Akk=Akk, Aqk=Aqk, Tm=Tm, kgam=kgam, w=w, u=u, qg=qg,
                kg=kg, decay_to_end=decay_to_end, low=low, strict=strict)


def chunked_forward(q, k, v, g, beta, scale, h0):
    """One (sequence, head): q,k,g [T,K], v [T,V], beta [T], h0 [K,V].  Returns o, ht, saved."""
    T = q.shape[0]
    NT = (T + C - 1) // C
    h = h0.clone()
    o = q.new_zeros(T, v.shape[1])
    saved = []
    for c in range(NT):
        s, e = c * C, min(T, (c + 1) * C)
        qc, kc, vc, gc, bc = (_pad(x[s:e], C) for x in (q, k, v, g, beta))
        cq = chunk_quantities(qc, kc, vc, gc, bc, scale)
        v_new = cq["u"] - cq["w"] @ h
        oc = cq["qg"] @ h + cq["Aqk"] @ v_new
        o[s:e] = oc[: e - s]
        saved.append(dict(cq=cq, h=h.clone(), v_new=v_new, q=qc, k=kc, v=vc, beta=bc, s=s, e=e))
        h = cq["Gam"][-1][:, None] * h + cq["kg"].T @ v_new
    return o, h, saved


def chunked_backward(saved, do, dht, scale):
    """Hand-derived gradients.  do [T,V], dht [K,V].  Returns dq, dk, dv, dg, dbeta, dh0."""
    T = do.shape[0]
    K = saved[0]["q"].shape[1]
    V = do.shape[1]
    dq = do.new_zeros(T, K)
    dk = do.new_zeros(T, K)
    dv = do.new_zeros(T, V)
    dg = do.new_zeros(T, K)
    db = do.new_zeros(T)
    dh_next = dht.clone()                              # gradient w.r.t. the state at the chunk's END
    for sv in reversed(saved):
        cq, h, v_new, qc, kc, vc, bc, s, e = (sv[n] for n in ("cq", "h", "v_new", "q", "k", "v", "beta", "s", "e"))
        doc = _pad(do[s:e], C)
        Tm, D = cq["Tm"], cq["D"]
        # --- reverse state scan step
        dv_new = cq["Aqk"].T @ doc + cq["kg"] @ dh_next
        dh = cq["Gam"][-1][:, None] * dh_next + cq["qg"].T @ doc - cq["w"].T @ dv_new
        # --- state-dependent pieces
        dqg = doc @ h.T
        dAqk = torch.where(cq["low"], doc @ v_new.T, torch.zeros(C, C, dtype=do.dtype))
        dkg = v_new @ dh_next.T
        dw = -dv_new @ h.T
        du = dv_new
        # --- through w = Tm (beta kgam), u = Tm (beta v)
        dbv = Tm.T @ du
        dbk = Tm.T @ dw
        dvc = bc[:, None] * dbv
        dkgam = bc[:, None] * dbk
        dbc = (dbv * vc).sum(-1) + (dbk * cq["kgam"]).sum(-1)
        dT = du @ (bc[:, None] * vc).T + dw @ (bc[:, None] * cq["kgam"]).T
        dAkk = torch.where(cq["strict"], -(Tm.T @ dT @ Tm.T), torch.zeros(C, C, dtype=do.dtype))
        dbc = dbc + (dAkk * cq["rawkk"]).sum(-1)
        dAkk_b = dAkk * bc[:, None]
        # --- q, k: "pos" parts see x*Gam, "neg" parts see x/Gam
        dqc = cq["Gam"] * scale * dqg + scale * torch.einsum("tj,tjk,jk->tk", dAqk, D, kc)
        dk_pos = cq["Gam"] * dkgam + torch.einsum("tj,tjk,jk->tk", dAkk_b, D, kc)
        dk_end = dkg * cq["decay_to_end"]
        dk_neg = (dk_end + scale * torch.einsum("tj,tjk,tk->jk", dAqk, D, qc)
                  + torch.einsum("tj,tjk,tk->jk", dAkk_b, D, kc))
        dkc = dk_pos + dk_neg
        dG = qc * dqc + kc * (dk_pos - dk_neg)
        dG[-1] = dG[-1] + (kc * dk_end).sum(0) + cq["Gam"][-1] * (h * dh_next).sum(-1)
        dgc = dG.flip(0).cumsum(0).flip(0)
        n = e - s
        dq[s:e], dk[s:e], dv[s:e], dg[s:e], db[s:e] = dqc[:n], dkc[:n], dvc[:n], dgc[:n], dbc[:n]
        dh_next = dh
    return dq, dk, dv, dg, db, dh_next


def chunk_kda_chunked(q, k, v, g, beta, scale, h0=None, do=None, dht=None):
    """[B,T,H,*] front end over (batch, head); float64.  Returns dict like recurrent_kda_grads."""
    q, k, v, g, beta = (x.double() for x in (q, k, v, g, beta))
    B, T, H, K = q.shape
    V = v.shape[-1]
    o = q.new_zeros(B, T, H, V)
    ht = q.new_zeros(B, H, K, V)
    res = dict(o=o, ht=ht)
    if do is not None:
        for n, shp in (("dq", q.shape), ("dk", q.shape), ("dv", v.shape), ("dg", q.shape), ("dbeta", beta.shape),
                       ("dh0", ht.shape)):
            res[n] = q.new_zeros(shp)
    for b in range(B):
        for h in range(H):
            h0_bh = q.new_zeros(K, V) if h0 is None else h0[b, h].double()
            o_bh, ht_bh, saved = chunked_forward(q[b, :, h], k[b, :, h], v[b, :, h], g[b, :, h], beta[b, :, h],
                                                 scale, h0_bh)
            o[b, :, h], ht[b, h] = o_bh, ht_bh
            if do is not None:
                dht_bh = q.new_zeros(K, V) if dht is None else dht[b, h].double()
                r = chunked_backward(saved, do[b, :, h].double(), dht_bh, scale)
                for n, val in zip(("dq", "dk", "dv", "dg", "dbeta"), r[:5]):
                    res[n][b, :, h] = val
                res["dh0"][b, h] = r[5]
    return res
