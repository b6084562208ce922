"""The two state scans run with one CTA per (sequence, head) unit or, for calls with few units, with four CTAs per unit
(one per slice of 32 value columns).  Every layout computes the same sums in the same order, so o, the
final state and every gradient are the same bits whichever is used -- which is what lets a packed sequence equal the
same sequence run alone even when the two calls pick different layouts -- and each layout matches the float64 oracle."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import assert_bf16_parity, recurrent_kda_grads

pytestmark = pytest.mark.gpu
NAMES = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")


def _run(d, cu, slices, backward=True, l2=False):
    from kda_b200 import chunk_kda, ops
    old = ops.SCAN_SLICES
    ops.SCAN_SLICES = slices
    try:
        lv = {n: d[n].cuda().requires_grad_(backward) for n in ("q", "k", "v", "g", "beta", "h0")}
        with torch.set_grad_enabled(backward):
            o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True,
                              cu_seqlens=None if cu is None else cu.cuda(), use_qk_l2norm_in_kernel=l2)
        out = dict(o=o.detach(), ht=ht.detach())
        if backward:
            torch.autograd.backward([o, ht], [d["do"].cuda(), d["dht"].cuda()])
            out.update(dq=lv["q"].grad, dk=lv["k"].grad, dv=lv["v"].grad, dg=lv["g"].grad, dbeta=lv["beta"].grad, dh0=lv["h0"].grad)
        return out
    finally:
        ops.SCAN_SLICES = old


@pytest.mark.parametrize("lens,l2", [([200], False), ([130, 1, 64, 77], False), ([65, 320], True)])
def test_every_scan_layout_gives_the_same_bits_and_matches_the_oracle(lens, l2):
    N = len(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32) if N > 1 else None
    d = make_inputs(1, sum(lens), 3, 128, 128, torch.bfloat16, seed=900 + sum(lens), h0_std=0.02, n_states=N, backward=True)
    if l2:
        d["q"], d["k"] = (d["q"].float() * 1.3).bfloat16(), (d["k"].float() * 0.8).bfloat16()
    one = _run(d, cu, 1, l2=l2)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], initial_state=d["h0"], cu_seqlens=cu,
                              use_qk_l2norm=l2)
    for n in NAMES:
        assert_bf16_parity(one[n], ref[n], n)
    for slices in (4,):
        got = _run(d, cu, slices, l2=l2)
        for n in NAMES:
            assert torch.equal(got[n], one[n]), (n, slices)


def test_forward_only_layouts_agree():
    """Inference (no tiles kept for a backward): the sliced scans skip their staging stores; same bits again."""
    d = make_inputs(2, 333, 2, 128, 128, torch.bfloat16, seed=950, h0_std=0.02, backward=True)
    one = _run(d, None, 1, backward=False)
    for slices in (4,):
        got = _run(d, None, slices, backward=False)
        assert torch.equal(got["o"], one["o"]) and torch.equal(got["ht"], one["ht"]), slices


def test_automatic_choice_and_argument_check():
    """Few units pick the sliced layout on their own; a slice count other than 0, 1, 4 is an argument error."""
    import ctypes as C
    from kda_b200 import _lib
    d = make_inputs(1, 100, 2, 128, 128, torch.bfloat16, seed=951, h0_std=0.02, backward=True)
    auto, one = _run(d, None, 0), _run(d, None, 1)
    for n in NAMES:
        assert torch.equal(auto[n], one[n]), n
    a = _lib.ChunkArgs(tokens=64, N=1, H=2, K=128, V=128, io_dtype=0, scan_slices=2)
    assert _lib.load().kda_chunk_fwd(C.byref(a), None) == -2
