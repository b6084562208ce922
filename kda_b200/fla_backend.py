"""Opt-in registration of the kda_b200 kernels in flash-linear-attention's backend registry.

fla routes `fla.ops.kda.chunk_kda` through a per-operation registry (fla/ops/backends/__init__.py:30-204; the KDA
registry lives in fla/ops/kda/backends/__init__.py:14-16): every registered backend gets a `<function>_verifier`
call and the first one that accepts handles the call.  `register()` adds a backend that accepts what the sm_100a
kernels implement and forwards to `kda_b200.chunk_kda`, so existing fla users (e.g. `fla.layers.kda`) reach these
kernels without touching their code:

    import kda_b200.fla_backend as shim
    shim.register()            # once, after importing fla; FLA_KDA_B200=0 switches it off again

Nothing here runs unless `register()` is called; kda_b200 itself never dispatches between implementations.
"""
from __future__ import annotations

import torch


def _accepts(q, k, v, g, beta, initial_state=None, cp_context=None, **kwargs):
    """(ok, reason) for a chunk_kda call: the shapes, dtypes and options the CUDA kernels cover."""
    if not (q.is_cuda and torch.cuda.get_device_capability(q.device)[0] == 10):
        return False, "kda_b200 needs an sm_100 CUDA device"
    if cp_context is not None:
        return False, "kda_b200 does not implement context parallelism"
    if kwargs.get("chunk_size", 64) not in (32, 64):
        return False, "kda_b200 takes chunk_size 32 or 64"
    if v.shape[2] % q.shape[2]:
        return False, f"HV={v.shape[2]} is not a multiple of H={q.shape[2]}"
    if q.dtype == torch.bfloat16:
        if q.shape[-1] != 128 or v.shape[-1] != 128:
            # kda_b200.chunk_kda itself also serves smaller heads (zero-padded to 128 channels); as a registered backend
            # it only takes over the shape it is faster on
            return False, f"kda_b200 bf16 kernels are built for K = V = 128, got K={q.shape[-1]}, V={v.shape[-1]}"
        return True, None
    if q.dtype == torch.float32:
        needs_grad = torch.is_grad_enabled() and any(
            t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state))
        if needs_grad:
            return False, "kda_b200 trains float32 tensors token by token (exact, slow); left to fla as a backend"
        if q.shape[-1] not in (32, 64, 128, 256) or v.shape[-1] % 32:
            return False, "kda_b200 float32 path needs K in {32,64,128,256} and V a multiple of 32"
        return True, None
    return False, f"kda_b200 needs bfloat16 or float32, got {q.dtype}"


def make_backend(priority: int = 1):
    """Builds the backend object (fla must be importable)."""
    from fla.ops.backends import BaseBackend

    class KdaB200Backend(BaseBackend):
        backend_type = "kda_b200"
        package_name = "kda_b200"
        env_var = "FLA_KDA_B200"
        default_enable = True

        def chunk_kda_verifier(self, q, k, v, g, beta, *args, **kwargs):
            names = ("scale", "initial_state", "output_final_state", "use_qk_l2norm_in_kernel", "use_gate_in_kernel",
                     "use_beta_sigmoid_in_kernel", "cu_seqlens", "cu_seqlens_cpu", "safe_gate", "lower_bound",
                     "disable_recompute", "return_intermediate_states", "cp_context", "transpose_state_layout")
            kwargs.update(dict(zip(names, args)))
            return _accepts(q, k, v, g, beta, **kwargs)

        def chunk_kda(self, *args, **kwargs):
            from kda_b200 import chunk_kda
            return chunk_kda(*args, **kwargs)

    KdaB200Backend.priority = priority
    return KdaB200Backend()


def register(priority: int = 1):
    """Registers the backend in fla's KDA registry and returns it.  Lower priority numbers are tried first
    (fla's own optional backends use 3 and 5)."""
    from fla.ops.kda.backends import kda_registry
    backend = make_backend(priority)
    kda_registry.register(backend)
    return backend
