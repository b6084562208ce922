"""GPU parity of the bf16 chunked forward against the float64 oracle (bf16 mode: max-normalised error and
relative L2 error <= 2e-2 and cosine >= 0.9999 for o and the final state)."""
import numpy as np
import pytest
import torch

from kda_b200.inputs import make_inputs
from oracle.kda_oracle import assert_bf16_parity, max_norm_err, recurrent_kda

pytestmark = pytest.mark.gpu
REL, COS = 2e-2, 0.9999


def _cuda(d):
    return {n: (t.cuda() if isinstance(t, torch.Tensor) else t) for n, t in d.items()}


def _check(o, ht, ref_o, ref_h):
    assert_bf16_parity(o, ref_o, "o", REL, COS)          # max-normalised AND relative L2 <= 2e-2, cosine >= 0.9999
    assert_bf16_parity(ht, ref_h, "ht", REL, COS)


@pytest.mark.parametrize("T", [1, 63, 64, 65, 130, 256])
def test_chunk_fwd_lengths(T):
    from kda_b200 import chunk_kda
    d = make_inputs(2, T, 3, 128, 128, torch.bfloat16, seed=T, h0_std=0.02)
    ref_o, ref_h = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    c = _cuda(d)
    with torch.no_grad():
        o, ht = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
    assert o.dtype == torch.bfloat16 and ht.dtype == torch.float32
    _check(o, ht, ref_o, ref_h)


def test_chunk_fwd_no_state_l2norm_scale():
    from kda_b200 import chunk_kda
    d = make_inputs(1, 200, 2, 128, 128, torch.bfloat16, seed=3)
    q, k = (d["q"].float() * 2.5).bfloat16(), (d["k"].float() * 0.4).bfloat16()
    ref_o, ref_h = recurrent_kda(q, k, d["v"], d["g"], d["beta"], scale=0.2, output_final_state=True, use_qk_l2norm=True)
    c = _cuda(d)
    with torch.no_grad():
        o, ht = chunk_kda(q.cuda(), k.cuda(), c["v"], c["g"], c["beta"], scale=0.2, output_final_state=True,
                          use_qk_l2norm_in_kernel=True)
        o2, none = chunk_kda(q.cuda(), k.cuda(), c["v"], c["g"], c["beta"], scale=0.2, use_qk_l2norm=True)
    _check(o, ht, ref_o, ref_h)
    assert none is None and torch.equal(o, o2)


def test_chunk_fwd_mild_gates():
    """Weak decay (|g| ~ 0.02 per step): long memory, the inter-chunk state dominates."""
    from kda_b200 import chunk_kda
    d = make_inputs(1, 512, 2, 128, 128, torch.bfloat16, seed=9, h0_std=0.02)
    g = d["g"] * 0.01
    ref_o, ref_h = recurrent_kda(d["q"], d["k"], d["v"], g, d["beta"], initial_state=d["h0"], output_final_state=True)
    c = _cuda(d)
    with torch.no_grad():
        o, ht = chunk_kda(c["q"], c["k"], c["v"], g.cuda(), c["beta"], initial_state=c["h0"], output_final_state=True)
    _check(o, ht, ref_o, ref_h)


def test_chunk_fwd_varlen_bit_exact_segmentation():
    """Packed variable-length result == each sequence run alone, bit for bit; and both match the oracle."""
    from kda_b200 import chunk_kda
    lens = [130, 1, 64, 77, 300]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    d = make_inputs(1, sum(lens), 4, 128, 128, torch.bfloat16, seed=21, h0_std=0.02, n_states=len(lens))
    c = _cuda(d)
    with torch.no_grad():
        o, ht = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True,
                          cu_seqlens=cu.cuda())
        for i in range(len(lens)):
            s, e = int(cu[i]), int(cu[i + 1])
            oi, hi = chunk_kda(c["q"][:, s:e], c["k"][:, s:e], c["v"][:, s:e], c["g"][:, s:e], c["beta"][:, s:e],
                               initial_state=c["h0"][i:i + 1], output_final_state=True)
            assert torch.equal(oi, o[:, s:e]), i
            assert torch.equal(hi, ht[i:i + 1]), i
    ref_o, ref_h = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                 output_final_state=True, cu_seqlens=cu)
    _check(o, ht, ref_o, ref_h)


def test_chunk_fwd_deterministic():
    """Same call twice -> identical bits."""
    from kda_b200 import chunk_kda
    d = _cuda(make_inputs(2, 100, 2, 128, 128, torch.bfloat16, seed=2, h0_std=0.02))
    with torch.no_grad():
        o1, h1 = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
        o2, h2 = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    assert torch.equal(o1, o2) and torch.equal(h1, h2)


def test_chunk_matches_recurrent_kernel_at_production_slice():
    """T=4096 at the production head shape, one batch x 4 heads: chunked bf16 vs the fp32 recurrent kernel
    (itself pinned to the oracle at small sizes)."""
    from kda_b200 import chunk_kda, fused_recurrent_kda
    d = _cuda(make_inputs(1, 4096, 4, 128, 128, torch.bfloat16, seed=4, h0_std=0.02))
    with torch.no_grad():
        o, ht = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
        ro, rh = fused_recurrent_kda(d["q"].float(), d["k"].float(), d["v"].float(), d["g"], d["beta"],
                                     initial_state=d["h0"], output_final_state=True)
    _check(o, ht, ro, rh)


def test_return_intermediate_states():
    """h[b, i] = the state at the start of chunk i (fla/ops/kda/chunk.py:95-98), against the fp64 oracle run on the
    prefix of the sequence; equal-length batch and packed varlen."""
    from kda_b200 import chunk_kda
    from oracle.kda_oracle import recurrent_kda
    d = make_inputs(2, 150, 2, 128, 128, torch.bfloat16, seed=77, h0_std=0.02)
    c = {n: (t.cuda() if t is not None else None) for n, t in d.items()}
    with torch.inference_mode():
        o, ht, h = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True,
                             return_intermediate_states=True)
    assert h.shape == (2, 3, 2, 128, 128) and h.dtype == torch.bfloat16
    o_ref, ht_ref = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    assert max_norm_err(o, o_ref) <= 2e-2 and max_norm_err(ht, ht_ref) <= 2e-2
    for i in range(3):
        if i == 0:
            ref = d["h0"].double()
        else:
            _, ref = recurrent_kda(d["q"][:, :64 * i], d["k"][:, :64 * i], d["v"][:, :64 * i], d["g"][:, :64 * i], d["beta"][:, :64 * i],
                                   initial_state=d["h0"], output_final_state=True)
        assert max_norm_err(h[:, i], ref) <= 2e-2, i
    # packed: 70 + 130 tokens -> 2 + 3 chunks
    cu = torch.tensor([0, 70, 200], dtype=torch.int32)
    dv = make_inputs(1, 200, 2, 128, 128, torch.bfloat16, seed=78, h0_std=0.02, n_states=2)
    cv = {n: (t.cuda() if t is not None else None) for n, t in dv.items()}
    with torch.inference_mode():
        _, _, hv = chunk_kda(cv["q"], cv["k"], cv["v"], cv["g"], cv["beta"], initial_state=cv["h0"], cu_seqlens=cu.cuda(),
                             return_intermediate_states=True)
    assert hv.shape == (1, 5, 2, 128, 128)
    _, ref = recurrent_kda(dv["q"][:, 70:134], dv["k"][:, 70:134], dv["v"][:, 70:134], dv["g"][:, 70:134], dv["beta"][:, 70:134],
                           initial_state=dv["h0"][1:2], output_final_state=True)
    assert max_norm_err(hv[0, 3], ref[0]) <= 2e-2
    assert max_norm_err(hv[0, 2], dv["h0"][1].double()) <= 2e-2
    with pytest.raises(AssertionError, match="inference mode"):
        chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], return_intermediate_states=True)


def test_chunk_size_32_is_the_same_function():
    """fla allows chunk_size 32 or 64 (fla/ops/kda/chunk.py:365-367); it only selects the tiling, so o, the final state
    and the gradients are those of the 64-token tiles, bit for bit here, and within tolerance of the oracle."""
    from kda_b200 import chunk_kda
    from oracle.kda_oracle import recurrent_kda
    d = make_inputs(1, 150, 2, 128, 128, torch.bfloat16, seed=79, h0_std=0.02)
    outs = []
    for cs in (32, 64):
        c = {n: t.cuda().requires_grad_(True) for n, t in d.items() if n in ("q", "k", "v", "g", "beta", "h0")}
        o, ht = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True, chunk_size=cs)
        (o.float().sum() + ht.sum()).backward()
        outs.append([o.detach(), ht.detach()] + [c[n].grad for n in ("q", "k", "v", "g", "beta", "h0")])
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    o_ref, ht_ref = recurrent_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    assert max_norm_err(outs[0][0], o_ref) <= 2e-2 and max_norm_err(outs[0][1], ht_ref) <= 2e-2
    with pytest.raises(ValueError, match="32 or 64"):
        chunk_kda(*(d[n].cuda() for n in ("q", "k", "v", "g", "beta")), chunk_size=16)


def test_intermediate_states_every_32_tokens():
    """chunk_size=32 with return_intermediate_states: one state per 32 tokens (fla/ops/kda/chunk.py:95-98 with
    chunk_size=32), each against the fp64 oracle run on the prefix; equal-length batch with a ragged tail and packed varlen."""
    from kda_b200 import chunk_kda
    from oracle.kda_oracle import recurrent_kda
    d = make_inputs(2, 150, 2, 128, 128, torch.bfloat16, seed=81, h0_std=0.02)
    c = {n: (t.cuda() if t is not None else None) for n, t in d.items()}
    with torch.inference_mode():
        o, ht, h = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True,
                             return_intermediate_states=True, chunk_size=32, use_qk_l2norm_in_kernel=True)
        o64, ht64, h64 = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True,
                                   return_intermediate_states=True, use_qk_l2norm_in_kernel=True)
    assert h.shape == (2, 5, 2, 128, 128) and h.dtype == torch.bfloat16          # ceil(150 / 32) = 5
    assert torch.equal(o, o64) and torch.equal(ht, ht64) and torch.equal(h[:, 0::2], h64)
    for i in range(5):
        if i == 0:
            ref = d["h0"].double()
        else:
            _, ref = recurrent_kda(d["q"][:, :32 * i], d["k"][:, :32 * i], d["v"][:, :32 * i], d["g"][:, :32 * i], d["beta"][:, :32 * i],
                                   initial_state=d["h0"], output_final_state=True, use_qk_l2norm=True)
        assert max_norm_err(h[:, i], ref) <= 2e-2, i
    # packed: 70 + 20 + 130 tokens -> 3 + 1 + 5 states
    cu = torch.tensor([0, 70, 90, 220], dtype=torch.int32)
    dv = make_inputs(1, 220, 2, 128, 128, torch.bfloat16, seed=82, h0_std=0.02, n_states=3)
    cv = {n: (t.cuda() if t is not None else None) for n, t in dv.items()}
    with torch.inference_mode():
        _, _, hv = chunk_kda(cv["q"], cv["k"], cv["v"], cv["g"], cv["beta"], initial_state=cv["h0"], cu_seqlens=cu.cuda(),
                             return_intermediate_states=True, chunk_size=32)
    assert hv.shape == (1, 9, 2, 128, 128)
    for pos, (seq, ntok) in {1: (0, 32), 2: (0, 64), 3: (1, 0), 5: (2, 32), 8: (2, 128)}.items():
        s0 = int(cu[seq])
        if ntok == 0:
            ref = dv["h0"][seq].double()
        else:
            _, ref = recurrent_kda(*(dv[n][:, s0:s0 + ntok] for n in ("q", "k", "v", "g", "beta")), initial_state=dv["h0"][seq:seq + 1],
                                   output_final_state=True)
            ref = ref[0]
        assert max_norm_err(hv[0, pos], ref) <= 2e-2, pos


@pytest.mark.captures_graph
def test_prefill_forward_replays_from_a_cuda_graph():
    """The forward entry point neither synchronises nor allocates: a captured prefill (packed variable-length batch, final
    states kept) replays to the eager result, bit for bit, also after the inputs have been overwritten in place."""
    from kda_b200 import chunk_kda
    cu = torch.tensor([0, 70, 200], dtype=torch.int32).cuda()
    d = make_inputs(1, 200, 2, 128, 128, torch.bfloat16, seed=90, h0_std=0.02, n_states=2)
    d2 = make_inputs(1, 200, 2, 128, 128, torch.bfloat16, seed=91, h0_std=0.02, n_states=2)
    c = {n: t.cuda() for n, t in d.items() if t is not None}

    def run():
        with torch.no_grad():
            return chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True, cu_seqlens=cu)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()                                   # one-time attribute setting outside the capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_g, ht_g = run()
    for src in (d, d2):
        for n in c:
            c[n].copy_(src[n])
        graph.replay()
        o_e, ht_e = run()
        torch.cuda.synchronize()
        assert torch.equal(o_g, o_e) and torch.equal(ht_g, ht_e)
