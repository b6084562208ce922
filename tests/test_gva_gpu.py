"""Grouped value heads (HV > H, fla/ops/kda/chunk.py:194-196,379-386): value head h reads q/k head h // (HV // H) and
dq, dk are summed over each group.  Against the fp64 oracle run on q, k repeated per group (autograd sums the groups)."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import assert_bf16_parity, max_norm_err, recurrent_kda

pytestmark = pytest.mark.gpu
NAMES = ("q", "k", "v", "g", "beta", "h0")


def _inputs(T, H, HV, seed, dtype=torch.bfloat16, K=128, V=128, n_states=None, B=1):
    d = make_inputs(B, T, HV, K, V, dtype, seed=seed, h0_std=0.02, backward=True, **({"n_states": n_states} if n_states else {}))
    d["q"], d["k"] = d["q"][:, :, :H].contiguous(), d["k"][:, :, :H].contiguous()
    return d


def _oracle(d, grp, cu=None, l2=False):
    lo = {n: d[n].double().requires_grad_(True) for n in NAMES}
    o, ht = recurrent_kda(lo["q"].repeat_interleave(grp, dim=2), lo["k"].repeat_interleave(grp, dim=2), lo["v"], lo["g"], lo["beta"],
                          initial_state=lo["h0"], output_final_state=True, cu_seqlens=cu, use_qk_l2norm=l2)
    grads = torch.autograd.grad((o * d["do"].double()).sum() + (ht * d["dht"].double()).sum(), [lo[n] for n in NAMES])
    return dict(o=o.detach(), ht=ht.detach(), **{"d" + n: g for n, g in zip(NAMES, grads)})


def _gpu(d, cu=None, l2=False):
    from kda_b200 import chunk_kda
    lc = {n: d[n].cuda().requires_grad_(True) for n in NAMES}
    o, ht = chunk_kda(lc["q"], lc["k"], lc["v"], lc["g"], lc["beta"], initial_state=lc["h0"], output_final_state=True,
                      cu_seqlens=None if cu is None else cu.cuda(), use_qk_l2norm_in_kernel=l2)
    ((o.float() * d["do"].cuda().float()).sum() + (ht * d["dht"].cuda()).sum()).backward()
    return dict(o=o.detach(), ht=ht.detach(), **{"d" + n: lc[n].grad for n in NAMES})


def _check(got, ref):
    for n, r in ref.items():
        assert got[n].shape == r.shape, (n, got[n].shape, r.shape)
        assert_bf16_parity(got[n], r, n)      # max-normalised AND relative L2 <= 2e-2, cosine >= 0.9999


@pytest.mark.parametrize("H,HV,l2", [(2, 4, False), (1, 4, True), (2, 6, False)])
def test_gva_chunk_fwd_bwd(H, HV, l2):
    d = _inputs(200, H, HV, seed=60 + HV)
    _check(_gpu(d, l2=l2), _oracle(d, HV // H, l2=l2))


def test_gva_varlen():
    lens = [70, 1, 129]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    d = _inputs(sum(lens), 2, 4, seed=71, n_states=len(lens))
    _check(_gpu(d, cu=cu), _oracle(d, 2, cu=cu))


def test_gva_recurrent_and_fp32():
    from kda_b200 import chunk_kda, fused_recurrent_kda
    d = _inputs(40, 2, 4, seed=72, dtype=torch.float32, K=64, V=64, B=2)
    o_ref, ht_ref = recurrent_kda(d["q"].repeat_interleave(2, dim=2), d["k"].repeat_interleave(2, dim=2), d["v"], d["g"], d["beta"],
                                  initial_state=d["h0"], output_final_state=True)
    c = {n: d[n].cuda() for n in NAMES}
    for fn in (fused_recurrent_kda, chunk_kda):
        o, ht = fn(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
        assert max_norm_err(o, o_ref) <= 1e-4 and max_norm_err(ht, ht_ref) <= 1e-4
    o, ht = fused_recurrent_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"].transpose(-1, -2).contiguous(),
                                output_final_state=True, transpose_state_layout=True)
    assert max_norm_err(o, o_ref) <= 1e-4 and max_norm_err(ht.transpose(-1, -2), ht_ref) <= 1e-4
    with pytest.raises(AssertionError, match="evenly divisible"):
        chunk_kda(c["q"], c["k"], c["v"][:, :, :3], c["g"][:, :, :3], c["beta"][:, :, :3])
