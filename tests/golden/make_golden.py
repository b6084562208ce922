"""Generates the golden vectors under tests/golden/ from flash-linear-attention 0.5.1's pure-PyTorch
`naive_recurrent_kda` (fla/ops/kda/naive.py:12-66), imported from the build container's
site-packages.  That package is third-party; the NVlabs/kda repository itself holds no vectors for
this operator.  Run from the repository root:   python tests/golden/make_golden.py

Files written:
  kda_small.npz   inputs + fp32 outputs + fp32 autograd gradients, B=2 T=100 H=2 K=32 V=16, h0 != 0
  kda_cfg0.npz    outputs only for the CPU-runnable workload (B=1 T=256 H=2 K=V=64, fp32, h0 = 0);
                  its inputs come from kda_b200.inputs.make_workload("fwd_fp32_small", seed=0) and
                  the file stores their float64 sums so that a generator drift is detected.
  kda_gate.npz    gate front end: raw inputs, fla's naive_kda_gate / naive_kda_lowerbound_gate outputs
                  (fla/ops/kda/gate.py:26-69) and their fp32 autograd gradients, tokens=24 H=3 K=16.
"""
import os
import sys
import warnings

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
warnings.filterwarnings("ignore")
from fla.ops.kda.gate import naive_kda_gate, naive_kda_lowerbound_gate  # noqa: E402
from fla.ops.kda.naive import naive_recurrent_kda  # noqa: E402

from kda_b200.inputs import make_inputs, make_workload  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def small():
    d = make_inputs(2, 100, 2, 32, 16, torch.float32, seed=7, h0_std=0.5, backward=True)
    leaves = {n: d[n].clone().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = naive_recurrent_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], scale=0.25,
                                initial_state=leaves["h0"], output_final_state=True)
    loss = (o * d["do"]).sum() + (ht * d["dht"]).sum()
    grads = torch.autograd.grad(loss, [leaves[n] for n in ("q", "k", "v", "g", "beta", "h0")])
    out = {n: d[n].numpy() for n in ("q", "k", "v", "g", "beta", "h0", "do", "dht")}
    out.update(o=o.detach().numpy(), ht=ht.detach().numpy(), scale=np.float64(0.25))
    for n, gr in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), grads):
        out[n] = gr.numpy()
    np.savez_compressed(os.path.join(HERE, "kda_small.npz"), **out)


def cfg0():
    d = make_workload("fwd_fp32_small", seed=0)
    o, ht = naive_recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=None,
                                output_final_state=True)
    sums = np.array([d[n].double().sum().item() for n in ("q", "k", "v", "g", "beta")])
    np.savez_compressed(os.path.join(HERE, "kda_cfg0.npz"), o=o.numpy(), ht=ht.numpy(), input_sums=sums)


def gate():
    gen = torch.Generator().manual_seed(11)
    g_raw = (torch.randn(2, 12, 3, 16, generator=gen) * 3.0)
    g_raw[0, 0, 0, :4] = torch.tensor([25.0, 19.5, -30.0, 0.0])        # both sides of the softplus switch at 20
    A_log = torch.randn(3, generator=gen)
    dt_bias = torch.randn(3 * 16, generator=gen)
    dy = torch.randn(2, 12, 3, 16, generator=gen)
    out = dict(g_raw=g_raw.numpy(), A_log=A_log.numpy(), dt_bias=dt_bias.numpy(), dy=dy.numpy(), lower_bound=np.float64(-5.0))
    for tag, fn in (("sp", lambda g, a, b: naive_kda_gate(g, a, b)),
                    ("sp_nobias", lambda g, a, b: naive_kda_gate(g, a, None)),
                    ("lb", lambda g, a, b: naive_kda_lowerbound_gate(g, a, b, lower_bound=-5.0))):
        g, a, b = (t.clone().requires_grad_(True) for t in (g_raw, A_log, dt_bias))
        y = fn(g, a, b)
        grads = torch.autograd.grad((y * dy).sum(), [g, a, b], allow_unused=True)
        out[f"y_{tag}"] = y.detach().numpy()
        out[f"dg_{tag}"] = grads[0].numpy()
        out[f"dA_{tag}"] = grads[1].numpy()
        if grads[2] is not None:
            out[f"db_{tag}"] = grads[2].numpy()
    np.savez_compressed(os.path.join(HERE, "kda_gate.npz"), **out)


if __name__ == "__main__":
    small()
    cfg0()
    gate()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
