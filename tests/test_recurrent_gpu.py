"""GPU parity of the token-recurrent kernel (decode and exact fp32 scans) against the float64 oracle."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs, make_workload
from oracle.kda_oracle import cosine, max_norm_err, recurrent_kda

pytestmark = pytest.mark.gpu


def _cuda(d):
    return {n: (t.cuda() if isinstance(t, torch.Tensor) else t) for n, t in d.items()}


def test_fp32_small_workload_matches_oracle_and_golden(golden_dir):
    """The CPU-runnable workload (B=1 T=256 H=2 K=V=64 fp32): 1e-4 max-normalised vs the fp64 oracle."""
    import os
    from kda_b200 import chunk_kda
    d = make_workload("fwd_fp32_small", seed=0)
    ref_o, ref_h = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True)
    c = _cuda(d)
    o, ht = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], output_final_state=True)
    assert o.dtype == torch.float32 and ht.dtype == torch.float32
    assert max_norm_err(o, ref_o) <= 1e-4
    assert max_norm_err(ht, ref_h) <= 1e-4
    z = np.load(os.path.join(golden_dir, "kda_cfg0.npz"))
    assert max_norm_err(o, torch.from_numpy(z["o"])) <= 1e-4
    assert max_norm_err(ht, torch.from_numpy(z["ht"])) <= 1e-4


@pytest.mark.parametrize("K,V", [(32, 32), (64, 64), (128, 128), (256, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_recurrent_shapes(K, V, dtype):
    from kda_b200 import fused_recurrent_kda
    d = make_inputs(2, 37, 3, K, V, dtype, seed=K + V, h0_std=0.3)
    ref_o, ref_h = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    c = _cuda(d)
    o, ht = fused_recurrent_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
    tol = 1e-4 if dtype == torch.float32 else 2e-2     # bf16 output rounding only; the state stays fp32
    assert max_norm_err(o, ref_o) <= tol
    assert max_norm_err(ht, ref_h) <= 1e-4
    assert cosine(o, ref_o) >= 0.9999


def test_recurrent_varlen_l2norm_scale():
    from kda_b200 import fused_recurrent_kda
    lens = [5, 64, 1, 70, 3]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int64)
    d = make_inputs(1, sum(lens), 2, 64, 32, torch.float32, seed=11, h0_std=0.3, n_states=len(lens))
    q, k = d["q"] * 3.0, d["k"] * 0.7
    ref_o, ref_h = recurrent_kda(q, k, d["v"], d["g"], d["beta"], scale=0.5, initial_state=d["h0"],
                                 output_final_state=True, cu_seqlens=cu, use_qk_l2norm=True)
    c = _cuda(d)
    o, ht = fused_recurrent_kda(q.cuda(), k.cuda(), c["v"], c["g"], c["beta"], scale=0.5, initial_state=c["h0"],
                                output_final_state=True, cu_seqlens=cu.cuda(), use_qk_l2norm_in_kernel=True)
    assert max_norm_err(o, ref_o) <= 1e-4
    assert max_norm_err(ht, ref_h) <= 1e-4


def test_decode_inplace_steps_match_scan():
    """Three single-token in-place steps (with a state-slot table) equal one 3-token scan."""
    from kda_b200 import fused_recurrent_kda, fused_recurrent_kda_fwd
    d = _cuda(make_inputs(4, 3, 2, 128, 128, torch.bfloat16, seed=5, h0_std=0.02))
    scale = 128 ** -0.5
    o_ref, h_ref = fused_recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                       output_final_state=True)
    pool = torch.zeros(6, 2, 128, 128, device="cuda")
    slots = torch.tensor([4, 0, 5, 2], device="cuda", dtype=torch.int32)
    pool[slots.long()] = d["h0"]
    outs = []
    for t in range(3):
        o_t, _ = fused_recurrent_kda_fwd(d["q"][:, t:t + 1], d["k"][:, t:t + 1], d["v"][:, t:t + 1], d["g"][:, t:t + 1],
                                         d["beta"][:, t:t + 1], scale=scale, initial_state=pool, inplace_final_state=True,
                                         ssm_state_indices=slots)
        outs.append(o_t)
    assert torch.equal(torch.cat(outs, 1), o_ref)
    assert torch.equal(pool[slots.long()], h_ref)
    assert torch.count_nonzero(pool[1]) == 0 and torch.count_nonzero(pool[3]) == 0


@pytest.mark.parametrize("case", ["plain", "l2norm_slots_gva", "fp32", "transposed", "transposed_l2norm_slots_gva"])
def test_large_decode_batch_bulk_copy_kernel(case):
    """640 (sequence, head) units with one token each: the step runs on the kernel that moves whole state tiles with the
    bulk-copy engine (at least four units per SM).  o and the new states against the float64 oracle: bf16 o 2e-2,
    fp32 o and the fp32 states 1e-4 (max-normalised); untouched slots stay untouched; the status word stays 0."""
    from kda_b200 import _lib, fused_recurrent_kda_fwd
    N, H = 40, 16
    dtype = torch.float32 if case == "fp32" else torch.bfloat16
    d = make_inputs(N, 1, H, 128, 128, dtype, seed=21, h0_std=0.05)
    l2 = case.endswith("l2norm_slots_gva")
    tr = case.startswith("transposed")          # states [.., V, K]
    HQ = 4 if l2 else H
    q, k = d["q"][:, :, :HQ].contiguous(), d["k"][:, :, :HQ].contiguous()
    if l2:
        q, k = q * 3, k * 0.5                      # not normalised on entry
    rep = H // HQ
    o_ref, h_ref = recurrent_kda(q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2), d["v"], d["g"], d["beta"],
                                 scale=0.11, initial_state=d["h0"], output_final_state=True, use_qk_l2norm=l2)
    c = _cuda(d)
    if tr:
        c["h0"] = c["h0"].transpose(-1, -2).contiguous()
    if l2:
        perm = torch.randperm(N + 8, generator=torch.Generator().manual_seed(1))[:N].to(torch.int32).cuda()
        pool = torch.full((N + 8, H, 128, 128), 7.0, device="cuda")
        pool[perm.long()] = c["h0"]
        o, ret = fused_recurrent_kda_fwd(q.cuda(), k.cuda(), c["v"], c["g"], c["beta"], scale=0.11, initial_state=pool,
                                         inplace_final_state=True, ssm_state_indices=perm, use_qk_l2norm_in_kernel=True,
                                         transpose_state_layout=tr)
        assert ret.data_ptr() == pool.data_ptr()
        ht = pool[perm.long()]
        rest = sorted(set(range(N + 8)) - set(perm.tolist()))
        assert all(bool((pool[i] == 7.0).all()) for i in rest)
    else:
        h0_before = c["h0"].clone()
        o, ht = fused_recurrent_kda_fwd(q.cuda(), k.cuda(), c["v"], c["g"], c["beta"], scale=0.11, initial_state=c["h0"],
                                        inplace_final_state=False, output_final_state=True, transpose_state_layout=tr)
        assert torch.equal(c["h0"], h0_before)
    if tr:
        ht = ht.transpose(-1, -2)
    assert _lib.recurrent_status() == 0
    assert max_norm_err(o, o_ref) <= (1e-4 if case == "fp32" else 2e-2) and cosine(o, o_ref) >= 0.9999
    assert max_norm_err(ht, h_ref) <= 1e-4


@pytest.mark.captures_graph
@pytest.mark.parametrize("N", [4, 40])
def test_decode_step_replays_from_a_cuda_graph(N):
    """Serving loops capture the decode step in a CUDA graph: the C entry point makes no synchronising call and takes the
    capturing stream, so a captured in-place step (per-warp kernel for N = 4, bulk-copy kernel for N = 40) replays to the
    same states and outputs as eager calls, bit for bit."""
    from kda_b200 import fused_recurrent_kda_fwd
    H = 16
    c = _cuda(make_inputs(N, 1, H, 128, 128, torch.bfloat16, seed=31, h0_std=0.05))
    args = (c["q"], c["k"], c["v"], c["g"], c["beta"])
    eager_state, graph_state, scratch = c["h0"].clone(), c["h0"].clone(), c["h0"].clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):           # first call outside the capture (one-time attribute setting)
        fused_recurrent_kda_fwd(*args, initial_state=scratch, inplace_final_state=True, use_qk_l2norm_in_kernel=True)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_graph, _ = fused_recurrent_kda_fwd(*args, initial_state=graph_state, inplace_final_state=True, use_qk_l2norm_in_kernel=True)
    for step in range(3):
        graph.replay()
        o_eager, _ = fused_recurrent_kda_fwd(*args, initial_state=eager_state, inplace_final_state=True, use_qk_l2norm_in_kernel=True)
        torch.cuda.synchronize()
        assert torch.equal(o_graph, o_eager), step
        assert torch.equal(graph_state, eager_state), step


@pytest.mark.parametrize("N,tr,lb", [(3, False, None), (3, True, -5.0), (40, False, -5.0), (40, True, None)])
def test_decode_with_the_gate_front_end_in_kernel(N, tr, lb):
    """The layer's decode call (fla/layers/kda.py:282-296): raw bf16 gate input with A_log, dt_bias (optionally the
    lower-bound form), beta logits, l2norm -- all inside the recurrent kernel, no pass over g and beta in front of it.
    Per-warp kernels (N = 3) and bulk-copy kernel (N = 40), both state layouts; o 2e-2, states 1e-4 against the oracle."""
    from kda_b200 import fused_recurrent_kda
    from oracle.kda_oracle import beta_sigmoid, kda_gate
    H = 16
    d = make_inputs(N, 1, H, 128, 128, torch.bfloat16, seed=33, h0_std=0.05)
    gen = torch.Generator().manual_seed(34)
    g_raw = torch.randn(N, 1, H, 128, generator=gen).bfloat16()
    beta_raw = torch.randn(N, 1, H, generator=gen).bfloat16()
    A_log = torch.log(torch.empty(H).uniform_(1, 16, generator=gen))
    dt_bias = torch.randn(H * 128, generator=gen) * 0.5
    o_ref, h_ref = recurrent_kda(d["q"], d["k"], d["v"], kda_gate(g_raw, A_log, dt_bias, lower_bound=lb), beta_sigmoid(beta_raw),
                                 initial_state=d["h0"], output_final_state=True, use_qk_l2norm=True)
    h0 = d["h0"].cuda()
    o, ht = fused_recurrent_kda(d["q"].cuda(), d["k"].cuda(), d["v"].cuda(), g_raw.cuda(), beta_raw.cuda(), A_log=A_log.cuda(),
                                dt_bias=dt_bias.cuda(), initial_state=h0.transpose(-1, -2).contiguous() if tr else h0,
                                output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                use_beta_sigmoid_in_kernel=True, lower_bound=lb, transpose_state_layout=tr)
    if tr:
        ht = ht.transpose(-1, -2)
    assert max_norm_err(o, o_ref) <= 2e-2 and cosine(o, o_ref) >= 0.9999
    assert max_norm_err(ht, h_ref) <= 1e-4


def test_speculative_decoding_state_slots():
    """Continuous batching with per-token state slots (fla/ops/kda/fused_recurrent.py:122-144,195-210): a sequence
    starts from the slot of its last accepted token and the state after draft token t lands in slot [n, t]."""
    from kda_b200 import fused_recurrent_kda, fused_recurrent_kda_fwd
    N, T = 3, 4
    d = _cuda(make_inputs(N, T, 2, 128, 128, torch.bfloat16, seed=9, h0_std=0.02))
    slots = torch.tensor([[7, 1, 12, 3], [0, 9, 4, 14], [5, 2, 11, 8]], device="cuda", dtype=torch.int32)
    accepted = torch.tensor([1, 3, 2], device="cuda", dtype=torch.int32)
    pool = torch.zeros(16, 2, 128, 128, device="cuda")
    for n in range(N):
        pool[int(slots[n, int(accepted[n]) - 1])] = d["h0"][n]
    o, ret = fused_recurrent_kda_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=pool, inplace_final_state=True,
                                     ssm_state_indices=slots, num_accepted_tokens=accepted)
    assert ret.data_ptr() == pool.data_ptr()
    for t in range(T):
        o_ref, h_ref = fused_recurrent_kda(d["q"][:, :t + 1], d["k"][:, :t + 1], d["v"][:, :t + 1], d["g"][:, :t + 1],
                                           d["beta"][:, :t + 1], initial_state=d["h0"], output_final_state=True)
        assert torch.equal(o[:, :t + 1], o_ref)
        assert torch.equal(pool[slots[:, t].long()], h_ref), t
    untouched = sorted(set(range(16)) - set(slots.flatten().tolist()))
    assert all(torch.count_nonzero(pool[i]) == 0 for i in untouched)
    with pytest.raises(ValueError, match="requires ssm_state_indices"):
        fused_recurrent_kda_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=pool, num_accepted_tokens=accepted)


def test_transposed_state_layout():
    """transpose_state_layout (states [N, H, V, K]): the dedicated decode kernel against the default layout, with slots;
    chunk_kda with transposed states in and out (fp32 1e-5 for decode: another summation order; bf16 mode for the chunk path)."""
    from kda_b200 import chunk_kda, fused_recurrent_kda, fused_recurrent_kda_fwd
    d = _cuda(make_inputs(3, 5, 2, 128, 128, torch.bfloat16, seed=21, h0_std=0.02))
    o_ref, h_ref = fused_recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True,
                                       use_qk_l2norm_in_kernel=True)
    o_t, h_t = fused_recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"].transpose(-1, -2).contiguous(),
                                   output_final_state=True, use_qk_l2norm_in_kernel=True, transpose_state_layout=True)
    assert h_t.shape == (3, 2, 128, 128)
    assert (o_t.float() - o_ref.float()).abs().max() <= 1e-2 * o_ref.float().abs().max()          # bf16 outputs: one ulp
    assert (h_t.transpose(-1, -2) - h_ref).abs().max() <= 1e-5 * h_ref.abs().max()
    # in-place pool with per-token slots, K = 64 fp32
    d64 = _cuda(make_inputs(2, 3, 2, 64, 64, torch.float32, seed=22, h0_std=0.1))
    slots = torch.tensor([[3, 0, 5], [1, 4, 2]], device="cuda", dtype=torch.int32)
    pool, pool_t = torch.zeros(6, 2, 64, 64, device="cuda"), torch.zeros(6, 2, 64, 64, device="cuda")
    pool[slots[:, 0].long()] = d64["h0"]
    pool_t[slots[:, 0].long()] = d64["h0"].transpose(-1, -2)
    o_a, _ = fused_recurrent_kda_fwd(d64["q"], d64["k"], d64["v"], d64["g"], d64["beta"], initial_state=pool, ssm_state_indices=slots)
    o_b, _ = fused_recurrent_kda_fwd(d64["q"], d64["k"], d64["v"], d64["g"], d64["beta"], initial_state=pool_t, ssm_state_indices=slots,
                                     transpose_state_layout=True)
    assert (o_a - o_b).abs().max() <= 1e-5 * o_a.abs().max()
    assert (pool_t.transpose(-1, -2) - pool).abs().max() <= 1e-5 * pool.abs().max()
    # chunk path
    dc = _cuda(make_inputs(2, 130, 2, 128, 128, torch.bfloat16, seed=23, h0_std=0.02))
    o1, h1 = chunk_kda(dc["q"], dc["k"], dc["v"], dc["g"], dc["beta"], initial_state=dc["h0"], output_final_state=True)
    o2, h2 = chunk_kda(dc["q"], dc["k"], dc["v"], dc["g"], dc["beta"], initial_state=dc["h0"].transpose(-1, -2).contiguous(),
                       output_final_state=True, transpose_state_layout=True)
    assert torch.equal(o1, o2) and torch.equal(h1, h2.transpose(-1, -2))


def test_empty_and_errors():
    from kda_b200 import chunk_kda, fused_recurrent_kda
    d = _cuda(make_inputs(1, 8, 2, 64, 64, torch.float32, seed=1, h0_std=0.1))
    with pytest.raises(ValueError):
        fused_recurrent_kda(d["q"].repeat(2, 1, 1, 1), d["k"].repeat(2, 1, 1, 1), d["v"].repeat(2, 1, 1, 1),
                            d["g"].repeat(2, 1, 1, 1), d["beta"].repeat(2, 1, 1), cu_seqlens=torch.tensor([0, 8]).cuda())
    with pytest.raises(AssertionError, match="A_log must be provided"):
        chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], use_gate_in_kernel=True)
    with pytest.raises(NotImplementedError):
        chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], cp_context=object())
    with pytest.raises(RuntimeError):
        chunk_kda(d["q"].cpu(), d["k"].cpu(), d["v"].cpu(), d["g"].cpu(), d["beta"].cpu())
    e = _cuda(make_inputs(2, 0, 2, 64, 64, torch.float32, seed=1, h0_std=0.1))
    o, ht = fused_recurrent_kda(e["q"], e["k"], e["v"], e["g"], e["beta"], initial_state=e["h0"], output_final_state=True)
    assert o.shape == (2, 0, 2, 64) and torch.equal(ht, e["h0"])
