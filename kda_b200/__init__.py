"""kda_b200 — Kimi Delta Attention for NVIDIA B200 (sm_100a).

`chunk_kda` and `fused_recurrent_kda` keep the operator API of flash-linear-attention's KDA ops and run
hand-written CUDA kernels through the C ABI in include/kda_b200.h (libkda_b200.so, built in-tree by
`python -m kda_b200.build`).  No Triton, no backend dispatch, no CPU fallback."""
from .ops import chunk_kda, fused_kda_gate, fused_recurrent_kda, fused_recurrent_kda_fwd  # noqa: F401

__all__ = ["chunk_kda", "fused_kda_gate", "fused_recurrent_kda", "fused_recurrent_kda_fwd"]
__version__ = "0.1.0"
