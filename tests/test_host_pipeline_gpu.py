"""GPU test of the host-resident pipeline: results equal those of one whole-batch call, bit for bit."""
import pytest
import torch

from kda_b200.inputs import make_inputs

pytestmark = pytest.mark.gpu


def test_host_pipeline_matches_whole_batch():
    from kda_b200 import chunk_kda
    from kda_b200.host import chunk_kda_fwd_bwd_host
    d = make_inputs(4, 200, 2, 128, 128, torch.bfloat16, seed=50, h0_std=0.02, backward=True)
    pinned = {n: t.pin_memory() for n, t in d.items() if t is not None}
    out = chunk_kda_fwd_bwd_host(pinned)
    out2 = chunk_kda_fwd_bwd_host(pinned, out, slices=2)          # staging buffers and outputs re-used
    c = {n: t.cuda() for n, t in d.items() if t is not None}
    leaves = [c[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")]
    o, ht = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
    grads = torch.autograd.grad([o, ht], leaves, [c["do"], c["dht"]])
    ref = dict(o=o, ht=ht, dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3], dbeta=grads[4], dh0=grads[5])
    out3 = chunk_kda_fwd_bwd_host(pinned, None, slices=4, head_groups=2)      # also cut along the head axis (strided copies)
    for n, r in ref.items():
        assert out2[n].is_pinned()
        assert torch.equal(out2[n], r.detach().cpu()), n
        assert torch.equal(out3[n], r.detach().cpu()), (n, "head groups")


def test_host_pipeline_overlapped_steps():
    """wait=False: three steps queued back to back on two different inputs with alternating output buffers; after
    host_synchronize() every step's results equal those of the blocking call, bit for bit."""
    from kda_b200.host import chunk_kda_fwd_bwd_host, host_synchronize
    ins = []
    for seed in (60, 61):
        d = make_inputs(4, 130, 2, 128, 128, torch.bfloat16, seed=seed, h0_std=0.02, backward=True)
        ins.append({n: t.pin_memory() for n, t in d.items() if t is not None})
    ref = [{n: t.clone() for n, t in chunk_kda_fwd_bwd_host(x).items()} for x in ins]
    outs = [None, None]
    outs[0] = chunk_kda_fwd_bwd_host(ins[0], None, wait=False)
    outs[1] = chunk_kda_fwd_bwd_host(ins[1], None, wait=False)
    host_synchronize()
    for i in range(2):
        for n, r in ref[i].items():
            assert torch.equal(outs[i][n], r), (i, n)
    # a third step into the first buffer set while nothing else is pending, then a blocking step right behind an async one
    chunk_kda_fwd_bwd_host(ins[1], outs[0], wait=False)
    last = chunk_kda_fwd_bwd_host(ins[0], outs[1])
    host_synchronize()
    for n in ref[0]:
        assert torch.equal(outs[0][n], ref[1][n]), n
        assert torch.equal(last[n], ref[0][n]), n


def test_first_backward_on_a_worker_thread_in_a_fresh_process():
    """The backward builds TMA tensor maps with a driver call that needs a context bound to the calling thread; the very
    first backward of a process may run on an autograd worker thread that has none yet."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import torch, sys; sys.path.insert(0, %r)\n"
        "from kda_b200.inputs import make_inputs\n"
        "from kda_b200.host import chunk_kda_fwd_bwd_host\n"
        "d = make_inputs(2, 100, 2, 128, 128, torch.bfloat16, seed=1, h0_std=0.02, backward=True)\n"
        "out = chunk_kda_fwd_bwd_host({n: t.pin_memory() for n, t in d.items() if t is not None})\n"
        "assert all(torch.isfinite(t.float()).all() for t in out.values()); print('ok')\n" % root)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]
