"""Guard bands: every output, workspace and state pool is placed between sentinel-filled margins; after the kernels have
run on ragged shapes (partial chunks, one-token sequences, packed variable lengths) the margins must be untouched and
the results must equal those of the operator called the ordinary way."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from _abi import Guarded, chunk_fwd_bwd_guarded

pytestmark = pytest.mark.gpu


def _ordinary(d, cu, l2=False, backward=True):
    from kda_b200 import chunk_kda
    lv = {n: d[n].detach().clone().requires_grad_(backward) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True,
                      cu_seqlens=cu, use_qk_l2norm_in_kernel=l2)
    out = dict(o=o.detach(), ht=ht.detach())
    if backward:
        ((o.float() * d["do"].float()).sum() + (ht * d["dht"]).sum()).backward()
        out.update(dq=lv["q"].grad, dk=lv["k"].grad, dv=lv["v"].grad, dg=lv["g"].grad, dbeta=lv["beta"].grad, dh0=lv["h0"].grad)
    return out


@pytest.mark.parametrize("lens,l2", [([1], False), ([63], False), ([65], True), ([130], False), ([130, 1, 64, 77], False),
                                      ([5, 200, 64], True)])
def test_chunk_fwd_bwd_stays_inside_its_buffers(lens, l2):
    tokens, N = sum(lens), len(lens)
    d = make_inputs(1, tokens, 3, 128, 128, torch.bfloat16, seed=500 + tokens, h0_std=0.02, n_states=N, backward=True)
    d = {n: t.cuda().contiguous() for n, t in d.items()}
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    got, guards = chunk_fwd_bwd_guarded(d, cu, l2=l2)
    for name, g in guards:
        assert g.margins_intact(), name
    ref = _ordinary(d, cu, l2=l2)
    for n in ref:
        assert torch.equal(got[n].view(ref[n].shape), ref[n]), n


@pytest.mark.parametrize("lens", [[1], [65], [70, 3, 129]])
def test_noalloc_forward_stays_inside_its_buffers(lens):
    tokens, N = sum(lens), len(lens)
    d = make_inputs(1, tokens, 3, 128, 128, torch.bfloat16, seed=600 + tokens, h0_std=0.02, n_states=N, backward=True)
    d = {n: t.cuda().contiguous() for n, t in d.items()}
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    got, guards = chunk_fwd_bwd_guarded(d, cu, noalloc=True)
    for name, g in guards:
        assert g.margins_intact(), name
    ref = _ordinary(d, cu, backward=False)
    assert torch.equal(got["o"].view(ref["o"].shape), ref["o"]) and torch.equal(got["ht"], ref["ht"])


@pytest.mark.parametrize("N,H,slots", [(3, 2, False), (40, 16, False), (40, 16, True), (5, 3, True)])
def test_decode_stays_inside_its_buffers(N, H, slots):
    """One decode step with the output and the state pool between sentinel margins: the per-warp kernel (few units)
    and the bulk-copy kernel (640 units), with and without a state-slot table."""
    from kda_b200 import _lib, fused_recurrent_kda_fwd
    d = make_inputs(N, 1, H, 128, 128, torch.bfloat16, seed=700 + N, h0_std=0.05)
    c = {n: t.cuda() for n, t in d.items() if t is not None}
    extra = 4 if slots else 0
    gpool = Guarded((N + extra) * H * 128 * 128 * 4)
    pool = gpool.view(torch.float32, (N + extra, H, 128, 128))
    go = Guarded(N * H * 128 * 2)
    out = go.view(torch.bfloat16, (N, 1, H, 128))
    idx = None
    if slots:
        idx = torch.randperm(N + extra, generator=torch.Generator().manual_seed(N))[:N].to(torch.int32).cuda()
        pool.fill_(3.0)
        pool[idx.long()] = c["h0"]
    else:
        pool.copy_(c["h0"])
    ref_state = c["h0"].clone()
    o_ref, _ = fused_recurrent_kda_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], scale=0.1, initial_state=ref_state,
                                       inplace_final_state=True)
    o, _ = fused_recurrent_kda_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], scale=0.1, initial_state=pool,
                                   inplace_final_state=True, ssm_state_indices=idx, out=out)
    torch.cuda.synchronize()
    assert _lib.recurrent_status() == 0
    assert gpool.margins_intact() and go.margins_intact()
    assert torch.equal(o, o_ref)
    assert torch.equal(pool[idx.long()] if slots else pool, ref_state)
    if slots:
        rest = sorted(set(range(N + extra)) - set(idx.tolist()))
        assert all(bool((pool[i] == 3.0).all()) for i in rest)


@pytest.mark.parametrize("lens,K,V", [([1], 128, 128), ([65], 64, 32), ([70, 0, 3, 129], 128, 128)])
def test_fp32_recurrent_backward_stays_inside_its_buffers(lens, K, V):
    """kda_recurrent_bwd through the C ABI with every output and its workspace between sentinel margins; the results
    equal those of the operator's float32 autograd path."""
    import ctypes as C
    from kda_b200 import _lib, chunk_kda
    from _abi import guarded_like
    lib = _lib.load()
    tokens, N, H = sum(lens), len(lens), 2
    d = make_inputs(1, tokens, H, K, V, torch.float32, seed=800 + tokens, h0_std=0.1, n_states=N, backward=True)
    d = {n: t.cuda().contiguous() for n, t in d.items()}
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    guards, out = [], {}
    for name, ref in (("dq", d["q"]), ("dk", d["k"]), ("dv", d["v"]), ("dg", d["g"]), ("dbeta", d["beta"]), ("dh0", d["h0"])):
        g, t = guarded_like(tuple(ref.shape), torch.float32)
        guards.append((name, g))
        out[name] = t
    wsg, ws = guarded_like((lib.kda_recurrent_bwd_workspace_bytes(tokens, N, H, K, V),), torch.uint8)
    guards.append(("workspace", wsg))
    p = lambda t: C.c_void_p(t.data_ptr())      # noqa: E731
    a = _lib.RecurrentBwdArgs(q=p(d["q"]), k=p(d["k"]), v=p(d["v"]), g=p(d["g"]), beta=p(d["beta"]), h0=p(d["h0"]), cu_seqlens=p(cu),
                              d_o=p(d["do"]), d_ht=p(d["dht"]), dq=p(out["dq"]), dk=p(out["dk"]), dv=p(out["dv"]), dg=p(out["dg"]),
                              dbeta=p(out["dbeta"]), dh0=p(out["dh0"]), workspace=p(ws), workspace_bytes=ws.numel(), tokens=tokens,
                              N=N, T=0, H=H, K=K, V=V, HQ=H, io_dtype=_lib.KDA_FP32, use_qk_l2norm=0, scale=K ** -0.5)
    _lib.check(lib.kda_recurrent_bwd(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)), "kda_recurrent_bwd")
    torch.cuda.synchronize()
    for name, g in guards:
        assert g.margins_intact(), name
    lv = {n: d[n].detach().clone().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True, cu_seqlens=cu)
    torch.autograd.backward([o, ht], [d["do"], d["dht"]])
    for name, src in (("dq", "q"), ("dk", "k"), ("dv", "v"), ("dg", "g"), ("dbeta", "beta"), ("dh0", "h0")):
        assert torch.equal(out[name], lv[src].grad), name
    # argument errors launch nothing
    a.K = 48
    assert lib.kda_recurrent_bwd(C.byref(a), None) == -2
    a.K, a.workspace_bytes = K, 16
    assert lib.kda_recurrent_bwd(C.byref(a), None) == -5
