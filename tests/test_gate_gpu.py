"""GPU parity of the gate front end (decay activation, beta sigmoid, their backward) against the float64 oracle
and the committed fla vectors, alone and in front of chunk_kda / fused_recurrent_kda."""
import os

import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import beta_sigmoid, cosine, kda_gate, max_norm_err, recurrent_kda, rel_l2_err

pytestmark = pytest.mark.gpu


def _rel(got, ref):
    ref = ref.double()
    return (got.double().cpu() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)


def test_gate_matches_golden_fp32(golden_dir):
    """fp32 raw inputs: forward 1e-5 and gradients 1e-4 (max-normalised) against fla's naive gate functions."""
    from kda_b200 import fused_kda_gate
    z = np.load(os.path.join(golden_dir, "kda_gate.npz"))
    dy = torch.from_numpy(z["dy"]).cuda()
    for tag, use_bias, lb in (("sp", True, None), ("sp_nobias", False, None), ("lb", True, float(z["lower_bound"]))):
        g, a, b = (torch.from_numpy(z[n]).cuda().requires_grad_(True) for n in ("g_raw", "A_log", "dt_bias"))
        y = fused_kda_gate(g, a, b if use_bias else None, lower_bound=lb)
        assert y.dtype == torch.float32
        (y * dy).sum().backward()
        assert _rel(y.detach(), torch.from_numpy(z[f"y_{tag}"])) <= 1e-5, tag
        assert _rel(g.grad, torch.from_numpy(z[f"dg_{tag}"])) <= 1e-4, tag
        assert _rel(a.grad, torch.from_numpy(z[f"dA_{tag}"])) <= 1e-4, tag
        if use_bias:
            assert _rel(b.grad, torch.from_numpy(z[f"db_{tag}"])) <= 1e-4, tag
        else:
            assert b.grad is None


@pytest.mark.parametrize("lb", [None, -5.0])
@pytest.mark.parametrize("tokens", [1, 77, 4096])
def test_gate_bf16_against_oracle(tokens, lb):
    """bf16 raw gate and beta logits at the production head shape; float64 autograd on the same bf16 values.
    g and beta (fp32 outputs) 1e-5; dg_raw / dbeta_raw (bf16 outputs) 1e-2; the reduced dA_log, ddt_bias 1e-3."""
    from kda_b200.ops import KDAGateFunction
    H, K = 32, 128
    gen = torch.Generator().manual_seed(5 + tokens)
    g_raw = (torch.randn(1, tokens, H, K, generator=gen) * 2).bfloat16()
    beta_raw = torch.randn(1, tokens, H, generator=gen).bfloat16()
    A_log = torch.log(torch.empty(H).uniform_(1, 16, generator=gen))
    dt_bias = torch.randn(H * K, generator=gen)
    dg = torch.randn(1, tokens, H, K, generator=gen)
    db = torch.randn(1, tokens, H, generator=gen)
    # oracle
    lo = [t.double().requires_grad_(True) for t in (g_raw, A_log, dt_bias, beta_raw)]
    g_ref, b_ref = kda_gate(lo[0], lo[1], lo[2], lower_bound=lb), beta_sigmoid(lo[3])
    grads = torch.autograd.grad((g_ref * dg.double()).sum() + (b_ref * db.double()).sum(), lo)
    # CUDA
    lc = [t.cuda().requires_grad_(True) for t in (g_raw, A_log, dt_bias, beta_raw)]
    g, b = KDAGateFunction.apply(lc[0], lc[1], lc[2], lc[3], lb)
    ((g * dg.cuda()).sum() + (b * db.cuda()).sum()).backward()
    assert g.dtype == torch.float32 and b.dtype == torch.float32
    assert _rel(g.detach(), g_ref.detach()) <= 1e-5 and _rel(b.detach(), b_ref.detach()) <= 1e-5
    assert lc[0].grad.dtype == torch.bfloat16 and lc[3].grad.dtype == torch.bfloat16
    assert _rel(lc[0].grad, grads[0]) <= 1e-2 and _rel(lc[3].grad, grads[3]) <= 1e-2
    assert _rel(lc[1].grad, grads[1]) <= 1e-3 and _rel(lc[2].grad, grads[2]) <= 1e-3


def test_gate_backward_is_bit_reproducible():
    from kda_b200 import fused_kda_gate
    gen = torch.Generator().manual_seed(3)
    g_raw = torch.randn(2, 3000, 32, 128, generator=gen).bfloat16().cuda()
    A_log, dt_bias, dy = torch.randn(32, generator=gen).cuda(), torch.randn(4096, generator=gen).cuda(), torch.randn(2, 3000, 32, 128, generator=gen).cuda()
    outs = []
    for _ in range(2):
        leaves = [t.clone().requires_grad_(True) for t in (g_raw, A_log, dt_bias)]
        (fused_kda_gate(*leaves) * dy).sum().backward()
        outs.append([t.grad.clone() for t in leaves])
    for x, y in zip(*outs):
        assert torch.equal(x, y)


def _gated_inputs(T, seed, B=1, H=2):
    d = make_inputs(B, T, H, 128, 128, torch.bfloat16, seed=seed, h0_std=0.02, backward=True)
    gen = torch.Generator().manual_seed(seed + 1)
    d["g_raw"] = torch.randn(B, T, H, 128, generator=gen).bfloat16()
    d["beta_raw"] = torch.randn(B, T, H, generator=gen).bfloat16()
    d["A_log"] = torch.log(torch.empty(H).uniform_(0.5, 4, generator=gen))
    d["dt_bias"] = torch.randn(H * 128, generator=gen) * 0.5
    return d


@pytest.mark.parametrize("raw_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("lb", [None, -5.0])
def test_chunk_kda_with_gate_in_kernel(lb, raw_dtype):
    """bf16 and fp32 raw gate input; the gate kernels run in front of the chunk kernels and behind their backward.
    The operator as the layer calls it (raw gate, beta logits, l2norm in kernel), forward and every gradient
    including A_log and dt_bias, against float64 autograd through oracle gate + oracle recurrence (bf16 mode:
    2e-2 max-normalised and cosine 0.9999; dA_log and ddt_bias are sums over all tokens of the bf16-noisy dg with
    heavy cancellation, so the element noise of dg shows up amplified there: 5e-2 and cosine 0.999 for those)."""
    from kda_b200 import chunk_kda
    d = _gated_inputs(200, 41)
    d["g_raw"] = d["g_raw"].to(raw_dtype)
    names = ("q", "k", "v", "g_raw", "beta_raw", "A_log", "dt_bias", "h0")
    lo = {n: d[n].double().requires_grad_(True) for n in names}
    o_ref, ht_ref = recurrent_kda(lo["q"], lo["k"], lo["v"], kda_gate(lo["g_raw"], lo["A_log"], lo["dt_bias"], lower_bound=lb),
                                  beta_sigmoid(lo["beta_raw"]), initial_state=lo["h0"], output_final_state=True, use_qk_l2norm=True)
    ref = torch.autograd.grad((o_ref * d["do"].double()).sum() + (ht_ref * d["dht"].double()).sum(), [lo[n] for n in names])
    lc = {n: d[n].cuda().requires_grad_(True) for n in names}
    o, ht = chunk_kda(lc["q"], lc["k"], lc["v"], lc["g_raw"], lc["beta_raw"], initial_state=lc["h0"], output_final_state=True,
                      use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                      A_log=lc["A_log"], dt_bias=lc["dt_bias"], lower_bound=lb, safe_gate=lb is not None)
    ((o.float() * d["do"].cuda().float()).sum() + (ht * d["dht"].cuda()).sum()).backward()
    bad = []
    for n, r in [("o", o_ref.detach()), ("ht", ht_ref.detach())] + [("d" + n, r) for n, r in zip(names, ref)]:
        got = {"o": o.detach(), "ht": ht.detach()}.get(n)
        if got is None:
            got = lc[n[1:]].grad
        e, e2, c = max_norm_err(got, r), rel_l2_err(got, r), cosine(got, r)
        rel, cos = (5e-2, 0.999) if n in ("dA_log", "ddt_bias") else (2e-2, 0.9999)
        if e > rel or e2 > rel or c < cos:
            bad.append((n, e, e2, c))
    assert not bad, bad


def test_beta_sigmoid_alone_and_recurrent_gate():
    from kda_b200 import chunk_kda, fused_recurrent_kda
    d = _gated_inputs(96, 43)
    # beta sigmoid without the gate
    o_ref, _ = recurrent_kda(d["q"], d["k"], d["v"], d["g"], beta_sigmoid(d["beta_raw"]), initial_state=d["h0"])
    c = {n: d[n].cuda() for n in ("q", "k", "v", "g", "g_raw", "beta_raw", "A_log", "dt_bias", "h0")}
    o, _ = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta_raw"], initial_state=c["h0"], use_beta_sigmoid_in_kernel=True)
    assert max_norm_err(o, o_ref) <= 2e-2 and cosine(o, o_ref) >= 0.9999
    # decode-style operator with the gate options
    o_ref, ht_ref = recurrent_kda(d["q"], d["k"], d["v"], kda_gate(d["g_raw"], d["A_log"], d["dt_bias"]), beta_sigmoid(d["beta_raw"]),
                                  initial_state=d["h0"], output_final_state=True)
    o, ht = fused_recurrent_kda(c["q"], c["k"], c["v"], c["g_raw"], c["beta_raw"], A_log=c["A_log"], dt_bias=c["dt_bias"],
                                initial_state=c["h0"], output_final_state=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True)
    assert max_norm_err(o, o_ref) <= 2e-2 and max_norm_err(ht, ht_ref) <= 1e-3


def test_gate_option_errors():
    from kda_b200 import chunk_kda
    d = _gated_inputs(64, 44)
    c = {n: d[n].cuda() for n in ("q", "k", "v", "g_raw", "beta", "A_log")}
    with pytest.raises(AssertionError, match="A_log must be provided"):
        chunk_kda(c["q"], c["k"], c["v"], c["g_raw"], c["beta"], use_gate_in_kernel=True)
    with pytest.raises(ValueError, match="lower_bound` must be specified"):
        chunk_kda(c["q"], c["k"], c["v"], c["g_raw"], c["beta"], use_gate_in_kernel=True, A_log=c["A_log"], safe_gate=True)
    with pytest.raises(ValueError, match="safe range"):
        chunk_kda(c["q"], c["k"], c["v"], c["g_raw"], c["beta"], use_gate_in_kernel=True, A_log=c["A_log"], safe_gate=True, lower_bound=-7.0)
