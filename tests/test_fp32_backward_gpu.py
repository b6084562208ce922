"""GPU parity of the float32 training path (token-recurrent forward + its exact reverse-mode backward,
`kda_recurrent_bwd`) against float64 autograd through the token-by-token oracle: max-normalised error <= 1e-4 for
o, the final state and every gradient (the fp32-mode bar)."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import max_norm_err, recurrent_kda_grads

pytestmark = pytest.mark.gpu
NAMES = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")
TOL = 1e-4


def _run(d, cu=None, scale=None, l2=False, with_h0=True, transpose=False):
    from kda_b200 import chunk_kda
    lv = {n: d[n].cuda().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    h0 = None
    if with_h0 and d["h0"] is not None:
        h0 = d["h0"].cuda()
        if transpose:
            h0 = h0.transpose(-1, -2).contiguous()
        h0.requires_grad_(True)
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], scale=scale, initial_state=h0, output_final_state=True,
                      use_qk_l2norm_in_kernel=l2, cu_seqlens=None if cu is None else cu.cuda(), transpose_state_layout=transpose)
    assert o.dtype == torch.float32 and ht.dtype == torch.float32
    dht = d["dht"].cuda()
    torch.autograd.backward([o, ht], [d["do"].cuda(), dht.transpose(-1, -2).contiguous() if transpose else dht])
    un = (lambda t: t.transpose(-1, -2)) if transpose else (lambda t: t)
    return dict(o=o.detach(), ht=un(ht.detach()), dq=lv["q"].grad, dk=lv["k"].grad, dv=lv["v"].grad, dg=lv["g"].grad,
                dbeta=lv["beta"].grad, dh0=None if h0 is None else un(h0.grad))


def _check(got, ref):
    for n in NAMES:
        if ref[n] is None or got[n] is None:
            continue
        assert torch.isfinite(got[n]).all(), n
        e = max_norm_err(got[n], ref[n])
        assert e <= TOL, f"{n}: max-normalised error {e:.3e}"


@pytest.mark.parametrize("T", [1, 63, 64, 65, 200])
def test_fp32_backward_lengths(T):
    d = make_inputs(2, T, 2, 128, 128, torch.float32, seed=300 + T, h0_std=0.1, backward=True)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    _check(_run(d), ref)


@pytest.mark.parametrize("K,V", [(32, 32), (64, 64), (64, 128), (128, 32), (32, 64)])
def test_fp32_backward_head_sizes(K, V):
    d = make_inputs(1, 150, 3, K, V, torch.float32, seed=400 + K + V, h0_std=0.1, backward=True)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    _check(_run(d), ref)


def test_fp32_backward_l2norm_scale_no_h0():
    d = make_inputs(1, 130, 2, 64, 64, torch.float32, seed=41, backward=True)
    d["q"], d["k"] = d["q"] * 2.5, d["k"] * 0.4
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], scale=0.2, use_qk_l2norm=True)
    _check(_run(d, scale=0.2, l2=True, with_h0=False), ref)


def test_fp32_backward_packed_with_an_empty_sequence_and_transposed_states():
    lens = [70, 0, 1, 129]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    d = make_inputs(1, sum(lens), 2, 128, 128, torch.float32, seed=42, h0_std=0.1, n_states=len(lens), backward=True)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"],
                              cu_seqlens=cu, use_qk_l2norm=True)
    got = _run(d, cu=cu, l2=True, transpose=True)
    _check(got, ref)
    assert torch.equal(got["dh0"][1].cpu(), d["dht"][1])      # the empty sequence hands its state gradient through


def test_fp32_backward_grouped_value_heads():
    """q, k with one head shared by two value heads: dq, dk are the sums over the group."""
    d = make_inputs(1, 100, 2, 64, 64, torch.float32, seed=43, h0_std=0.1, backward=True)
    d["q"], d["k"] = d["q"][:, :, :1].contiguous(), d["k"][:, :, :1].contiguous()
    rep = lambda t: t.expand(-1, -1, 2, -1)      # noqa: E731
    lq, lk = d["q"].double().requires_grad_(True), d["k"].double().requires_grad_(True)
    from oracle.kda_oracle import recurrent_kda
    rest = [d[n].double().requires_grad_(True) for n in ("v", "g", "beta")]
    h0 = d["h0"].double().requires_grad_(True)
    o, ht = recurrent_kda(rep(lq), rep(lk), *rest, initial_state=h0, output_final_state=True)
    gr = torch.autograd.grad([o, ht], [lq, lk] + rest + [h0], [d["do"].double(), d["dht"].double()])
    ref = dict(o=o.detach(), ht=ht.detach(), dq=gr[0], dk=gr[1], dv=gr[2], dg=gr[3], dbeta=gr[4], dh0=gr[5])
    _check(_run(d), ref)


def test_fp32_backward_is_deterministic():
    d = make_inputs(2, 100, 2, 128, 128, torch.float32, seed=44, h0_std=0.1, backward=True)
    a, b = _run(d), _run(d)
    for n in NAMES:
        assert torch.equal(a[n], b[n]), n
