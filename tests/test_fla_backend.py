"""The opt-in shim that registers kda_b200 in flash-linear-attention's backend registry."""
import pytest
import torch

fla = pytest.importorskip("fla")


def _unregister():
    from fla.ops.kda.backends import kda_registry
    kda_registry._backends.pop("kda_b200", None)
    kda_registry._update_active_backend()


def test_register_and_verifier_rejects_what_the_kernels_do_not_cover():
    import kda_b200.fla_backend as shim
    from fla.ops.kda.backends import kda_registry
    be = shim.register(priority=1)
    try:
        assert kda_registry._backends["kda_b200"] is be and be.priority == 1
        q = torch.zeros(1, 64, 2, 128, dtype=torch.bfloat16)
        g, beta = torch.zeros(1, 64, 2, 128), torch.zeros(1, 64, 2)
        ok, why = be.verify("chunk_kda", q, q, q, g, beta)
        assert not ok and "sm_100" in why                      # CPU tensors stay on fla's own path
    finally:
        _unregister()


@pytest.mark.gpu
def test_fla_chunk_kda_routes_to_kda_b200():
    import kda_b200.fla_backend as shim
    from fla.ops.kda import chunk_kda as fla_chunk_kda
    from fla.ops.kda.backends import kda_registry
    from kda_b200 import chunk_kda
    from kda_b200.inputs import make_inputs
    d = make_inputs(1, 200, 2, 128, 128, torch.bfloat16, seed=3, h0_std=0.02)
    c = {n: (t.cuda() if t is not None else None) for n, t in d.items()}
    shim.register(priority=1)
    try:
        with torch.no_grad():
            o1, h1 = fla_chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
            o2, h2 = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"], output_final_state=True)
        assert "kda:chunk_kda:kda_b200" in kda_registry._logged
        assert torch.equal(o1, o2) and torch.equal(h1, h2)
        # what the kernels do not cover is handed back
        ok, why = shim._accepts(c["q"], c["k"], c["v"], c["g"], c["beta"], chunk_size=16)
        assert not ok and "chunk_size" in why
        assert shim._accepts(c["q"], c["k"], c["v"], c["g"], c["beta"], chunk_size=32, return_intermediate_states=True)[0]
        ok, why = shim._accepts(c["q"], c["k"], c["v"], c["g"], c["beta"], cp_context=object())
        assert not ok and "context parallelism" in why
        assert shim._accepts(c["q"], c["k"], c["v"], c["g"], c["beta"], chunk_size=32)[0]
    finally:
        _unregister()
