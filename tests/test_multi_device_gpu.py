"""One process, two devices: the opt-in to large dynamic shared memory is a per-device attribute, so the first call on a
second GPU must set it there too.  The same inputs give the same bits on both devices.  Plain independent launches: no
peer access, no collective."""
import pytest
import torch

from kda_b200.inputs import make_inputs

pytestmark = pytest.mark.gpu


def _step(d, dev):
    from kda_b200 import chunk_kda, fused_recurrent_kda_fwd
    c = {n: t.to(dev) for n, t in d.items() if t is not None}
    lv = {n: c[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True,
                      use_qk_l2norm_in_kernel=True)
    torch.autograd.backward([o, ht], [c["do"], c["dht"]])
    outs = [o.detach(), ht.detach()] + [lv[n].grad for n in ("q", "k", "v", "g", "beta", "h0")]
    # a bulk decode step: 640 (sequence, head) units, one token each
    e = {n: t.to(dev) for n, t in make_inputs(40, 1, 16, 128, 128, torch.bfloat16, seed=9, h0_std=0.05).items() if t is not None}
    state = e["h0"].clone()
    od, _ = fused_recurrent_kda_fwd(e["q"], e["k"], e["v"], e["g"], e["beta"], scale=0.1, initial_state=state, inplace_final_state=True)
    # the bounded-gate variant of the forward and the float32 training path have kernels (and attributes) of their own
    with torch.no_grad():
        gs = -5.0 * torch.sigmoid(c["g"])
        o_safe, _ = chunk_kda(c["q"], c["k"], c["v"], gs, c["beta"], initial_state=c["h0"], output_final_state=True, safe_gate=True)
    f = {n: t.to(dev) for n, t in make_inputs(1, 70, 2, 128, 128, torch.float32, seed=10, h0_std=0.1, backward=True).items()}
    lf = {n: f[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o32, ht32 = chunk_kda(lf["q"], lf["k"], lf["v"], lf["g"], lf["beta"], initial_state=lf["h0"], output_final_state=True)
    torch.autograd.backward([o32, ht32], [f["do"], f["dht"]])
    outs += [o_safe, o32.detach(), lf["q"].grad, lf["g"].grad, lf["h0"].grad]
    torch.cuda.synchronize(dev)
    return [t.cpu() for t in outs + [od, state]]


def test_same_bits_on_a_second_device():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    d = make_inputs(2, 200, 3, 128, 128, torch.bfloat16, seed=8, h0_std=0.02, backward=True)
    a = _step(d, torch.device("cuda", 0))
    b = _step(d, torch.device("cuda", 1))
    for i, (x, y) in enumerate(zip(a, b)):
        assert torch.isfinite(x.float()).all() and torch.equal(x, y), i
