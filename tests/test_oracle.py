"""CPU tests: the float64 oracle against the committed golden vectors, its own invariants, and the
chunked restatement (the formulas the CUDA kernels implement) against float64 autograd."""
import os

import numpy as np
import torch

from kda_b200.inputs import make_inputs, make_workload
from oracle.kda_chunked import chunk_kda_chunked
from oracle.kda_oracle import cosine, max_norm_err, recurrent_kda, recurrent_kda_grads


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_oracle_matches_golden_small(golden_dir):
    z = np.load(os.path.join(golden_dir, "kda_small.npz"))
    r = recurrent_kda_grads(_t(z["q"]), _t(z["k"]), _t(z["v"]), _t(z["g"]), _t(z["beta"]), _t(z["do"]), _t(z["dht"]),
                            scale=float(z["scale"]), initial_state=_t(z["h0"]))
    # the golden vectors are fp32 (the generating package computes in fp32): 1e-4 max-normalised
    for n in ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0"):
        assert max_norm_err(r[n], _t(z[n])) < 1e-4, n
        assert cosine(r[n], _t(z[n])) > 0.999999, n


def test_oracle_matches_golden_cfg0(golden_dir):
    z = np.load(os.path.join(golden_dir, "kda_cfg0.npz"))
    d = make_workload("fwd_fp32_small", seed=0)
    sums = np.array([d[n].double().sum().item() for n in ("q", "k", "v", "g", "beta")])
    np.testing.assert_allclose(sums, z["input_sums"], rtol=1e-9, atol=1e-9)
    o, ht = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True)
    assert max_norm_err(o, _t(z["o"])) < 1e-4
    assert max_norm_err(ht, _t(z["ht"])) < 1e-4


def test_split_and_resume():
    d = make_inputs(2, 96, 2, 16, 8, torch.float32, seed=3, h0_std=0.3)
    full_o, full_h = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                   output_final_state=True)
    cut = 41
    a = {n: d[n][:, :cut] for n in ("q", "k", "v", "g", "beta")}
    b = {n: d[n][:, cut:] for n in ("q", "k", "v", "g", "beta")}
    o1, h1 = recurrent_kda(**a, initial_state=d["h0"], output_final_state=True)
    o2, h2 = recurrent_kda(**b, initial_state=h1, output_final_state=True)
    assert torch.equal(torch.cat([o1, o2], 1), full_o)
    assert torch.equal(h2, full_h)


def test_varlen_equals_per_sequence():
    lens = [5, 64, 1, 70]
    T = sum(lens)
    d = make_inputs(1, T, 2, 16, 8, torch.float32, seed=4, h0_std=0.3, n_states=len(lens))
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    o, ht = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True,
                          cu_seqlens=torch.tensor(cu))
    for i in range(len(lens)):
        s, e = cu[i], cu[i + 1]
        oi, hi = recurrent_kda(d["q"][:, s:e], d["k"][:, s:e], d["v"][:, s:e], d["g"][:, s:e], d["beta"][:, s:e],
                               initial_state=d["h0"][i:i + 1], output_final_state=True)
        assert torch.equal(oi, o[:, s:e])
        assert torch.equal(hi, ht[i:i + 1])


def test_l2norm_flag():
    d = make_inputs(1, 20, 1, 16, 8, torch.float32, seed=5)
    q, k = d["q"] * 3.0, d["k"] * 0.5
    o1, _ = recurrent_kda(q, k, d["v"], d["g"], d["beta"], use_qk_l2norm=True)
    qn = q.double() * torch.rsqrt((q.double() ** 2).sum(-1, keepdim=True) + 1e-6)
    kn = k.double() * torch.rsqrt((k.double() ** 2).sum(-1, keepdim=True) + 1e-6)
    o2, _ = recurrent_kda(qn, kn, d["v"], d["g"], d["beta"])
    assert torch.allclose(o1, o2, atol=1e-14)


def test_chunked_restatement_matches_autograd():
    # T = 150: two full chunks and a ragged tail; strong gates (within-chunk cumulative decay << e^-88)
    d = make_inputs(2, 150, 2, 32, 16, torch.float32, seed=1, h0_std=0.5, backward=True)
    ref = recurrent_kda_grads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], scale=0.3,
                              initial_state=d["h0"])
    got = chunk_kda_chunked(d["q"], d["k"], d["v"], d["g"], d["beta"], 0.3, d["h0"], d["do"], d["dht"])
    for n in ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0"):
        assert max_norm_err(got[n], ref[n]) < 1e-12, n


def test_empty_sequence():
    d = make_inputs(1, 0, 2, 8, 8, torch.float32, seed=6, h0_std=0.1)
    o, ht = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    assert o.shape == (1, 0, 2, 8)
    assert torch.equal(ht, d["h0"].double())


def test_gate_oracle_matches_golden(golden_dir):
    """The float64 gate restatement against fla's naive_kda_gate / naive_kda_lowerbound_gate outputs and their
    autograd gradients (fp32 fixtures: 2e-6 relative)."""
    import numpy as np
    from oracle.kda_oracle import kda_gate
    z = np.load(os.path.join(golden_dir, "kda_gate.npz"))
    dy = torch.from_numpy(z["dy"]).double()
    for tag, use_bias, lb in (("sp", True, None), ("sp_nobias", False, None), ("lb", True, float(z["lower_bound"]))):
        g, a, b = (torch.from_numpy(z[n]).double().requires_grad_(True) for n in ("g_raw", "A_log", "dt_bias"))
        y = kda_gate(g, a, b if use_bias else None, lower_bound=lb)
        grads = torch.autograd.grad((y * dy).sum(), [g, a] + ([b] if use_bias else []))
        pairs = [(y, z[f"y_{tag}"]), (grads[0], z[f"dg_{tag}"]), (grads[1], z[f"dA_{tag}"])]
        if use_bias:
            pairs.append((grads[2], z[f"db_{tag}"]))
        for got, ref in pairs:
            ref = torch.from_numpy(ref).double()
            assert (got.detach() - ref).abs().max() <= 2e-6 * max(1.0, ref.abs().max().item()), tag
