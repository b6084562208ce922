"""GPU parity of the bf16 chunked path for head sizes below 128 (fla allows any K <= 256,
fla/ops/kda/chunk.py:376-384): the operator pads key and value channels to the kernels' 128 with zeros, which must leave
o, the states and every gradient those of the unpadded problem -- checked against float64 autograd through the
token-by-token oracle at the real head sizes."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import assert_bf16_parity, recurrent_kda_grads

pytestmark = pytest.mark.gpu
NAMES = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")


def _run(d, cu=None, l2=False, transpose=False):
    from kda_b200 import chunk_kda
    lv = {n: d[n].cuda().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    h0 = d["h0"].cuda()
    if transpose:
        h0 = h0.transpose(-1, -2).contiguous()
    h0.requires_grad_(True)
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=h0, output_final_state=True,
                      use_qk_l2norm_in_kernel=l2, cu_seqlens=None if cu is None else cu.cuda(), transpose_state_layout=transpose)
    dht = d["dht"].cuda()
    torch.autograd.backward([o, ht], [d["do"].cuda(), dht.transpose(-1, -2).contiguous() if transpose else dht])
    un = (lambda t: t.transpose(-1, -2)) if transpose else (lambda t: t)
    return dict(o=o.detach(), ht=un(ht.detach()), dq=lv["q"].grad, dk=lv["k"].grad, dv=lv["v"].grad, dg=lv["g"].grad,
                dbeta=lv["beta"].grad, dh0=un(h0.grad))


@pytest.mark.parametrize("K,V", [(64, 64), (96, 32), (128, 64), (32, 128)])
def test_small_heads_forward_backward(K, V):
    d = make_inputs(2, 150, 2, K, V, torch.bfloat16, seed=900 + K + V, h0_std=0.02, backward=True)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    got = _run(d)
    assert got["o"].shape[-1] == V and got["ht"].shape[-2:] == (K, V) and got["dq"].shape[-1] == K
    for n in NAMES:
        assert_bf16_parity(got[n], ref[n], n)


def test_small_heads_l2norm_packed_transposed_states():
    """K = V = 64 with in-kernel L2 normalisation, packed sequences and the [V, K] state layout."""
    lens = [70, 1, 129]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    d = make_inputs(1, sum(lens), 2, 64, 64, torch.bfloat16, seed=911, h0_std=0.02, n_states=len(lens), backward=True)
    d["q"] = (d["q"].float() * 3).bfloat16()
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"],
                              use_qk_l2norm=True, cu_seqlens=cu)
    got = _run(d, cu=cu, l2=True, transpose=True)
    for n in NAMES:
        assert_bf16_parity(got[n], ref[n], n)


def test_small_heads_intermediate_states():
    from kda_b200 import chunk_kda
    d = make_inputs(1, 200, 2, 64, 32, torch.bfloat16, seed=912, h0_std=0.02)
    with torch.inference_mode():
        o, ht, h = chunk_kda(*(d[n].cuda() for n in ("q", "k", "v", "g", "beta")), initial_state=d["h0"].cuda(),
                             output_final_state=True, return_intermediate_states=True)
    assert o.shape == (1, 200, 2, 32) and ht.shape == (1, 2, 64, 32) and h.shape == (1, 4, 2, 64, 32)
    assert_bf16_parity(h[:, 0], d["h0"], "h[0]")


def test_key_size_256_runs_forward_only():
    """K = 256 (fla's upper limit): forward through the token-recurrent kernel, bf16 in and out; training raises."""
    from kda_b200 import chunk_kda
    from oracle.kda_oracle import recurrent_kda
    d = make_inputs(2, 100, 2, 256, 128, torch.bfloat16, seed=913, h0_std=0.02)
    c = {n: d[n].cuda() for n in ("q", "k", "v", "g", "beta", "h0")}
    with torch.no_grad():
        o, ht = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
    ro, rh = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    assert o.dtype == torch.bfloat16 and ht.shape == (2, 2, 256, 128)
    assert_bf16_parity(o, ro, "o")
    assert_bf16_parity(ht, rh, "ht")
    with pytest.raises(NotImplementedError):
        chunk_kda(c["q"].requires_grad_(True), c["k"], c["v"], c["g"], c["beta"])
    e = make_inputs(1, 64, 1, 192, 128, torch.bfloat16, seed=914)
    with pytest.raises(NotImplementedError):
        with torch.no_grad():
            chunk_kda(*(e[n].cuda() for n in ("q", "k", "v", "g", "beta")))
