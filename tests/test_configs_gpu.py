"""GPU parity at the stated shapes of the benchmark workloads (kda_b200/inputs.py:WORKLOADS).

Every test runs the FULL shape through the operator -- so the tile indexing over 32 heads, the persistent tile walk of
the per-chunk backward over tens of thousands of tiles, the packed tables of 64 sequences and the decode ring over
32,768 units are the ones the benchmark times -- and compares sampled (sequence, head) slices with the float64
token-by-token oracle.  A (sequence, head) slice is an exact sub-problem of the recurrence, so the oracle of a slice is
the oracle of the whole.  The oracle itself runs on the GPU in float64 here (same code, `oracle/kda_oracle.py`), which
turns minutes of CPU time into seconds.  Inputs are drawn on the device (`generate_on_device=True`): same
distributions as the CPU generator, seeded, without tens of GB of float32 staging on the host.

Bars: bf16 mode, max-normalised error and relative L2 error <= 2e-2 and cosine >= 0.9999 for o, the final state and
every gradient; decode states (fp32) 1e-4 max-normalised; packed sequences bit-equal to the same sequence run alone."""
import pytest
import torch

from kda_b200.inputs import WORKLOADS, make_inputs, make_workload
from oracle.kda_oracle import assert_bf16_parity, max_norm_err, recurrent_kda, recurrent_kda_grads

pytestmark = pytest.mark.gpu
GRADS = ("dq", "dk", "dv", "dg", "dbeta")


def _slice_bh(t, pairs, state=False):
    """Stacks the (b, h) slices of [B, T, H, ...] (or of a state [N, H, K, V]) as a batch with one head."""
    if state:
        return torch.stack([t[b, h] for b, h in pairs]).unsqueeze(1)
    return torch.stack([t[b, :, h] for b, h in pairs]).unsqueeze(2)


def test_prefill_shape_forward():
    """B=4 T=4096 H=32 K=V=128 forward with an initial state: o and the final state of three (batch, head) slices."""
    from kda_b200 import chunk_kda
    w = WORKLOADS["prefill_bf16"]
    d = make_workload("prefill_bf16", seed=0, device="cuda", generate_on_device=True)
    assert d["q"].shape == (w.B, w.T, w.H, w.K) == (4, 4096, 32, 128)
    with torch.no_grad():
        o, ht = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    pairs = [(0, 0), (2, 17), (3, 31)]
    ro, rh = recurrent_kda(*(_slice_bh(d[n], pairs) for n in ("q", "k", "v", "g", "beta")),
                           initial_state=_slice_bh(d["h0"], pairs, state=True), output_final_state=True)
    assert_bf16_parity(_slice_bh(o, pairs), ro, "o")
    assert_bf16_parity(_slice_bh(ht, pairs, state=True), rh, "ht")


def test_training_shape_forward_backward():
    """B=8 T=8192 H=32 K=V=128 forward + backward (the headline workload): o, the final state and every gradient of
    two (batch, head) slices, the last batch row and head among them, against float64 autograd through 8,192 steps."""
    from kda_b200 import chunk_kda
    d = make_workload("train_bf16", seed=0, device="cuda", generate_on_device=True)
    assert d["q"].shape == (8, 8192, 32, 128)
    lv = {n: d[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True)
    torch.autograd.backward([o, ht], [d["do"], d["dht"]])
    pairs = [(7, 31), (3, 12)]
    got = dict(o=_slice_bh(o.detach(), pairs), ht=_slice_bh(ht.detach(), pairs, state=True),
               dh0=_slice_bh(lv["h0"].grad, pairs, state=True))
    for gname, n in zip(GRADS, ("q", "k", "v", "g", "beta")):
        got[gname] = _slice_bh(lv[n].grad, pairs)
    sl = {n: _slice_bh(d[n].detach(), pairs) for n in ("q", "k", "v", "g", "beta", "do")}
    h0s, dhts = _slice_bh(d["h0"].detach(), pairs, state=True), _slice_bh(d["dht"], pairs, state=True)
    del o, ht, lv, d
    torch.cuda.empty_cache()
    ref = recurrent_kda_grads(sl["q"], sl["k"], sl["v"], sl["g"], sl["beta"], sl["do"], dhts, initial_state=h0s)
    for n in ("o", "ht", "dh0") + GRADS:
        assert_bf16_parity(got[n], ref[n], n)


def test_packed_varlen_shape_forward_backward():
    """64 packed sequences of 128..16,384 tokens, H=32: the shortest, the median and the longest sequence (a) are, bit
    for bit, what the same sequence gives when it is run alone (all 32 heads, forward and every gradient), and (b) match
    float64 autograd on heads 0 and 31."""
    from kda_b200 import chunk_kda
    d = make_workload("varlen_bf16", seed=0, device="cuda", generate_on_device=True)
    cu = d.pop("cu_seqlens")
    lens = (cu[1:] - cu[:-1]).tolist()
    assert len(lens) == 64 and d["q"].shape[0] == 1 and d["q"].shape[2] == 32
    order = sorted(range(64), key=lambda i: lens[i])
    picks = [order[0], order[32], order[-1]]
    lv = {n: d[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True,
                      cu_seqlens=cu)
    torch.autograd.backward([o, ht], [d["do"], d["dht"]])
    cul = cu.tolist()
    packed, alone_in = {}, {}
    for i in picks:
        s, e = cul[i], cul[i + 1]
        packed[i] = dict(o=o.detach()[:, s:e].clone(), ht=ht.detach()[i:i + 1].clone(), dh0=lv["h0"].grad[i:i + 1].clone(),
                         **{gname: lv[n].grad[:, s:e].clone() for gname, n in zip(GRADS, ("q", "k", "v", "g", "beta"))})
        alone_in[i] = {n: d[n].detach()[:, s:e].clone() for n in ("q", "k", "v", "g", "beta", "do")}
        alone_in[i].update(h0=d["h0"].detach()[i:i + 1].clone(), dht=d["dht"][i:i + 1].clone())
    del o, ht, lv, d
    torch.cuda.empty_cache()
    for i in picks:
        a = alone_in[i]
        la = {n: a[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
        o1, h1 = chunk_kda(la["q"], la["k"], la["v"], la["g"], la["beta"], initial_state=la["h0"], output_final_state=True)
        torch.autograd.backward([o1, h1], [a["do"], a["dht"]])
        alone = dict(o=o1.detach(), ht=h1.detach(), dh0=la["h0"].grad,
                     **{gname: la[n].grad for gname, n in zip(GRADS, ("q", "k", "v", "g", "beta"))})
        for n, x in alone.items():
            assert torch.equal(x, packed[i][n]), (n, i, lens[i])
        heads = [0, 31]
        ref = recurrent_kda_grads(*(a[n].detach()[:, :, heads] for n in ("q", "k", "v", "g", "beta", "do")), a["dht"][:, heads],
                                  initial_state=a["h0"].detach()[:, heads])
        for n in ("o",) + GRADS:
            assert_bf16_parity(packed[i][n][:, :, heads], ref[n], f"{n} (sequence of {lens[i]} tokens)")
        for n in ("ht", "dh0"):
            assert_bf16_parity(packed[i][n][:, heads], ref[n], f"{n} (sequence of {lens[i]} tokens)")
        del la, o1, h1, alone, ref
        torch.cuda.empty_cache()


def test_decode_shape_256_consecutive_steps():
    """1,024 sequences x 32 heads, 256 consecutive single-token steps with the fp32 states updated in place (the
    bulk-copy kernel): after step 256 the states of 8 sampled sequences (all heads) match the oracle to 1e-4
    max-normalised and their 256 outputs to the bf16 bar; the kernel's status word stays 0."""
    from kda_b200 import _lib, fused_recurrent_kda_fwd
    w = WORKLOADS["decode"]
    N, H, T = w.B, w.H, w.steps
    assert (N, H, T) == (1024, 32, 256)
    d = make_inputs(N, T, H, 128, 128, torch.bfloat16, seed=0, h0_std=0.02, device="cuda", generate_on_device=True)
    state = d["h0"].clone()
    sample = [0, 1, 255, 256, 511, 700, 1022, 1023]
    outs = []
    for t in range(T):
        o, _ = fused_recurrent_kda_fwd(d["q"][:, t:t + 1], d["k"][:, t:t + 1], d["v"][:, t:t + 1], d["g"][:, t:t + 1],
                                       d["beta"][:, t:t + 1], scale=128 ** -0.5, initial_state=state, inplace_final_state=True)
        outs.append(o[sample])
    torch.cuda.synchronize()
    assert _lib.recurrent_status() == 0
    ro, rh = recurrent_kda(*(d[n][sample] for n in ("q", "k", "v", "g", "beta")), initial_state=d["h0"][sample],
                           output_final_state=True)
    assert torch.isfinite(state).all()
    assert max_norm_err(state[sample], rh) <= 1e-4
    assert_bf16_parity(torch.cat(outs, dim=1), ro, "o")
