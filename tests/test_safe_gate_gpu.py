"""GPU parity of the bounded-gate forward variant (`safe_gate=True`: every gate value is at least -5, the caller's
promise of fla/ops/kda/chunk.py:235-246).  With the promise the forward factors the diagonal 16 x 16 blocks of the
intra-chunk products around each block's middle row and runs them on tensor cores; these tests pin that variant to
the float64 token-by-token oracle at the edge of the bound, for ragged chunks, packed sequences, the in-kernel gate
and the backward that reads the tiles this forward leaves."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import assert_bf16_parity, kda_gate, recurrent_kda, recurrent_kda_grads

pytestmark = pytest.mark.gpu
NAMES = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")


def _bounded(d, seed, lower=-5.0, edge=0.0):
    """Replaces d['g'] by lower * sigmoid(x), x ~ N(0, 2); a fraction `edge` of the values sits exactly on the bound."""
    gen = torch.Generator().manual_seed(seed)
    g = lower * torch.sigmoid(2.0 * torch.randn(d["g"].shape, generator=gen))
    if edge > 0:
        g = torch.where(torch.rand(g.shape, generator=gen) < edge, torch.full_like(g, lower), g)
    d["g"] = g.float()
    return d


def _run(d, safe, cu=None, l2=False):
    from kda_b200 import chunk_kda
    lv = {n: d[n].cuda().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True,
                      use_qk_l2norm_in_kernel=l2, safe_gate=safe, cu_seqlens=None if cu is None else cu.cuda())
    torch.autograd.backward([o, ht], [d["do"].cuda(), d["dht"].cuda()])
    return dict(o=o.detach(), ht=ht.detach(), dq=lv["q"].grad, dk=lv["k"].grad, dv=lv["v"].grad, dg=lv["g"].grad,
                dbeta=lv["beta"].grad, dh0=lv["h0"].grad)


@pytest.mark.parametrize("T", [1, 15, 17, 64, 100, 257])
def test_safe_gate_lengths_forward_backward(T):
    d = _bounded(make_inputs(2, T, 2, 128, 128, torch.bfloat16, seed=700 + T, h0_std=0.02, backward=True), seed=T)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    got = _run(d, safe=True)
    for n in NAMES:
        assert_bf16_parity(got[n], ref[n], n)


def test_safe_gate_at_the_bound():
    """Half of all gate values exactly -5, the rest close to it: the largest factors the factorisation can meet
    (eight tokens of -5 either side of the middle row).  Everything finite and on the oracle."""
    d = make_inputs(1, 192, 4, 128, 128, torch.bfloat16, seed=71, h0_std=0.02, backward=True)
    d = _bounded(d, seed=72, edge=0.5)
    d["g"] = torch.minimum(d["g"], torch.tensor(-4.5))
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    got = _run(d, safe=True)
    for n in NAMES:
        assert torch.isfinite(got[n]).all(), n
        assert_bf16_parity(got[n], ref[n], n)


def test_safe_gate_agrees_with_default_variant():
    """The two variants compute the same products with different roundings: close to each other, and the outputs of
    the off-diagonal blocks' rows unchanged in kind -- both within the bar of the oracle (checked above); here the
    distance between them, which bounds what a caller sees when switching the flag."""
    d = _bounded(make_inputs(2, 320, 4, 128, 128, torch.bfloat16, seed=73, h0_std=0.02, backward=True), seed=74)
    a, b = _run(d, safe=True, l2=True), _run(d, safe=False, l2=True)
    for n in NAMES:
        assert_bf16_parity(a[n], b[n].double().cpu(), n)


def test_safe_gate_packed_sequences_bit_equal_alone():
    lens = [130, 1, 64, 77]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    d = _bounded(make_inputs(1, sum(lens), 2, 128, 128, torch.bfloat16, seed=75, h0_std=0.02, n_states=len(lens),
                             backward=True), seed=76)
    got = _run(d, safe=True, cu=cu)
    for i, (s, e) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        one = {n: d[n][:, s:e] for n in ("q", "k", "v", "g", "beta", "do")}
        one.update(h0=d["h0"][i:i + 1], dht=d["dht"][i:i + 1])
        alone = _run(one, safe=True)
        for n in ("o", "dq", "dk", "dv", "dg", "dbeta"):
            assert torch.equal(got[n][:, s:e], alone[n]), (n, i)
        for n in ("ht", "dh0"):
            assert torch.equal(got[n][i:i + 1], alone[n]), (n, i)


def test_safe_gate_with_gate_in_kernel():
    """The operator's own use: raw gate input, `use_gate_in_kernel=True`, `lower_bound=-5`, `safe_gate=True`."""
    from kda_b200 import chunk_kda
    B, T, H, K = 1, 200, 2, 128
    d = make_inputs(B, T, H, K, K, torch.bfloat16, seed=77, h0_std=0.02)
    gen = torch.Generator().manual_seed(78)
    g_raw = (torch.randn(B, T, H, K, generator=gen) * 2).bfloat16()
    A_log = torch.log(torch.empty(H).uniform_(1, 16, generator=gen))
    dt_bias = torch.randn(H * K, generator=gen)
    with torch.no_grad():
        o, ht = chunk_kda(d["q"].cuda(), d["k"].cuda(), d["v"].cuda(), g_raw.cuda(), d["beta"].cuda(),
                          initial_state=d["h0"].cuda(), output_final_state=True, use_gate_in_kernel=True, safe_gate=True,
                          lower_bound=-5.0, A_log=A_log.cuda(), dt_bias=dt_bias.cuda())
    g = kda_gate(g_raw.double(), A_log.double(), dt_bias.double(), lower_bound=-5.0)
    ro, rh = recurrent_kda(d["q"], d["k"], d["v"], g, d["beta"], initial_state=d["h0"], output_final_state=True)
    assert_bf16_parity(o, ro, "o")
    assert_bf16_parity(ht, rh, "ht")
