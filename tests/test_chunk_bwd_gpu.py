"""GPU parity of the bf16 chunked backward against float64 autograd through the token-by-token oracle
(bf16 mode: max-normalised error and relative L2 error <= 2e-2 and cosine >= 0.9999 for every gradient)."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import assert_bf16_parity, recurrent_kda_grads

pytestmark = pytest.mark.gpu
REL, COS = 2e-2, 0.9999
NAMES = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")


def run_gpu(d, cu=None, scale=None, l2=False, with_h0=True):
    from kda_b200 import chunk_kda
    leaves = {n: d[n].cuda().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    h0 = d["h0"].cuda().requires_grad_(True) if (with_h0 and d["h0"] is not None) else None
    o, ht = chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], scale=scale, initial_state=h0,
                      output_final_state=True, use_qk_l2norm_in_kernel=l2, cu_seqlens=None if cu is None else cu.cuda())
    loss = (o.float() * d["do"].cuda().float()).sum() + (ht * d["dht"].cuda()).sum()
    loss.backward()
    return dict(o=o.detach(), ht=ht.detach(), dq=leaves["q"].grad, dk=leaves["k"].grad, dv=leaves["v"].grad,
                dg=leaves["g"].grad, dbeta=leaves["beta"].grad, dh0=None if h0 is None else h0.grad)


def check(got, ref, names=NAMES):
    for n in names:
        if ref[n] is not None:
            assert_bf16_parity(got[n], ref[n], n, REL, COS)      # max-normalised AND relative L2 <= 2e-2, cosine >= 0.9999


@pytest.mark.parametrize("T", [1, 63, 64, 65, 130, 256])
def test_chunk_bwd_lengths(T):
    d = make_inputs(2, T, 2, 128, 128, torch.bfloat16, seed=100 + T, h0_std=0.02, backward=True)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    check(run_gpu(d), ref)


def test_chunk_bwd_mild_gates():
    d = make_inputs(1, 320, 2, 128, 128, torch.bfloat16, seed=31, h0_std=0.02, backward=True)
    d["g"] = d["g"] * 0.01
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    check(run_gpu(d), ref)


def test_chunk_bwd_l2norm_scale_no_h0():
    d = make_inputs(1, 150, 2, 128, 128, torch.bfloat16, seed=32, backward=True)
    d["q"] = (d["q"].float() * 2.5).bfloat16()
    d["k"] = (d["k"].float() * 0.4).bfloat16()
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], scale=0.2, use_qk_l2norm=True)
    check(run_gpu(d, scale=0.2, l2=True, with_h0=False), ref)


def test_chunk_bwd_varlen_bit_exact_segmentation():
    lens = [130, 1, 64, 77]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    d = make_inputs(1, sum(lens), 2, 128, 128, torch.bfloat16, seed=33, h0_std=0.02, n_states=len(lens), backward=True)
    got = run_gpu(d, cu=cu)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"],
                              cu_seqlens=cu)
    check(got, ref)
    for i in range(len(lens)):
        s, e = int(cu[i]), int(cu[i + 1])
        di = {n: (d[n][:, s:e] if n in ("q", "k", "v", "g", "beta", "do") else d[n][i:i + 1]) for n in d}
        gi = run_gpu(di)
        for n in ("o", "dq", "dk", "dv", "dg", "dbeta"):
            assert torch.equal(gi[n], got[n][:, s:e]), (n, i)
        for n in ("ht", "dh0"):
            assert torch.equal(gi[n], got[n][i:i + 1]), (n, i)


def test_chunk_bwd_production_slice():
    """T=2048 at the production head shape (one batch, two heads) against float64 autograd."""
    d = make_inputs(1, 2048, 2, 128, 128, torch.bfloat16, seed=34, h0_std=0.02, backward=True)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"])
    check(run_gpu(d), ref)


def test_chunk_bwd_deterministic():
    d = make_inputs(2, 200, 2, 128, 128, torch.bfloat16, seed=35, h0_std=0.02, backward=True)
    a, b = run_gpu(d), run_gpu(d)
    for n in NAMES:
        assert torch.equal(a[n], b[n]), n


@pytest.mark.parametrize("l2", [False, True])
def test_chunk_bwd_persistent_tile_walk(l2):
    """B=48 T=130 H=4: 576 (chunk, head) tiles with ragged tails, more than three per SM, so every persistent CTA of the
    per-chunk backward walks several tiles (next-tile prefetch, the alternating chunk-info slots, barrier phase flips,
    re-use of the dq / dk staging tiles).  Every batch row must equal, bit for bit, the same row run alone (fewer tiles
    than SMs: no CTA takes a second tile there), and one row must match float64 autograd; with and without the fused
    L2-normalisation epilogue."""
    B, T, H = 48, 130, 4
    d = make_inputs(B, T, H, 128, 128, torch.bfloat16, seed=36, h0_std=0.02, backward=True)
    if l2:
        d["q"], d["k"] = (d["q"].float() * 1.7).bfloat16(), (d["k"].float() * 0.6).bfloat16()
    got = run_gpu(d, l2=l2)
    for b in (0, 17, 47):
        di = {n: d[n][b:b + 1] for n in d}
        gi = run_gpu(di, l2=l2)
        for n in NAMES:
            assert torch.equal(gi[n], got[n][b:b + 1]), (n, b)
    b = 31
    ref = recurrent_kda_grads(*(d[n][b:b + 1] for n in ("q", "k", "v", "g", "beta", "do", "dht")), initial_state=d["h0"][b:b + 1],
                              use_qk_l2norm=l2)
    check({n: got[n][b:b + 1] for n in NAMES}, ref)


def test_training_after_an_inference_mode_call_of_the_same_shape():
    """The per-shape table of sequence starts is cached; the copy made by a call under torch.inference_mode() must
    still be usable by a later training call of the same shape (inference tensors cannot be saved for backward)."""
    from kda_b200 import chunk_kda
    d = make_inputs(2, 70, 1, 128, 128, torch.bfloat16, seed=35, h0_std=0.02, backward=True)
    c = {n: t.cuda() for n, t in d.items()}
    with torch.inference_mode():
        o_inf, _ = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
    got = run_gpu(d)
    assert torch.equal(got["o"], o_inf)
    assert all(torch.isfinite(got[n]).all() for n in NAMES)
