"""Operator front end: `chunk_kda` (prefill / training, autograd) and `fused_recurrent_kda` (decode).

Signatures, argument meaning and error behaviour mirror flash-linear-attention 0.5.1
(`fla/ops/kda/chunk.py:167-411`, `fla/ops/kda/fused_recurrent.py:229-452`); everything below the
Python signature runs in hand-written sm_100a CUDA kernels reached through the C ABI of
`include/kda_b200.h`.  PyTorch only owns device memory and streams here.  There is no fallback:
CPU tensors, a missing shared library or an unsupported option raise.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import torch

from . import _lib

_DT = {torch.bfloat16: _lib.KDA_BF16, torch.float32: _lib.KDA_FP32}
CHUNK = 64
SCAN_SLICES = 0      # CTAs per (sequence, head) of the state scans: 0 = automatic; 1 or 4 force a layout (tests, measurements)


def _checked() -> bool:
    """KDA_B200_CHECK=1: after every operator call read the kernels' device status words (bounded waits that gave
    up, an inconsistent cu_seqlens) and raise if one is set.  Each read waits for the device, so this is a
    debugging / validation mode; without it a serving loop reads `_lib.chunk_status` / `_lib.recurrent_status`
    itself at a point where it synchronises anyway."""
    return os.environ.get("KDA_B200_CHECK", "0") not in ("", "0")


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _unsupported(name, value, default):
    if value is not default and value != default:
        raise NotImplementedError(f"kda_b200: `{name}` is not supported by this implementation")


def _check_common(q, k, v, g, beta, initial_state, cu_seqlens):
    if not q.is_cuda:
        raise RuntimeError("kda_b200 runs on CUDA (sm_100a) tensors only; there is no CPU path")
    B, T, H, K = q.shape
    assert q.shape == k.shape, f"q and k must have the same shape, got q={q.shape} vs k={k.shape}"
    HV, V = v.shape[2], v.shape[3]
    assert HV % H == 0, (
        f"For GVA, num_v_heads (HV={HV}) must be evenly divisible by num_qk_heads (H={H}), "
        f"but got HV % H = {HV % H}")
    assert K <= 256, f"Currently we only support key headdim <=256 for KDA, got {K}."
    assert g.shape == (B, T, HV, K), f"g must have shape [B, T, HV, K]={[B, T, HV, K]}, got {list(g.shape)}"
    assert beta.shape == (B, T, HV), f"beta must have shape [B, T, HV]={[B, T, HV]}, got {list(beta.shape)}"
    if cu_seqlens is not None:
        if B != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    if initial_state is not None:
        assert initial_state.dtype == torch.float32, "initial_state must be in float32."
    if q.dtype not in _DT or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError(f"kda_b200: q, k, v must share dtype bfloat16 or float32, got {q.dtype}")
    return B, T, HV, K, V      # H below always counts value heads; q and k may have fewer (grouped value heads)


_cu_cache: dict = {}


def _fixed_cu_seqlens(B: int, T: int, device) -> torch.Tensor:
    key = (B, T, str(device))
    cu = _cu_cache.get(key)
    if cu is None:
        # a tensor made inside torch.inference_mode() cannot be saved for a later backward: the cached table must be an
        # ordinary tensor whichever mode the first caller was in
        with torch.inference_mode(False):
            cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=device) if T > 0 else \
                torch.zeros(B + 1, dtype=torch.int32, device=device)
        if len(_cu_cache) > 64:
            _cu_cache.clear()
        _cu_cache[key] = cu
    return cu


def _as_i32(cu: torch.Tensor, device) -> torch.Tensor:
    if cu.dtype != torch.int32 or cu.device != device:
        cu = cu.to(device=device, dtype=torch.int32)
    return cu.contiguous()


# =================================================================================================
# gate front end: decay activation and beta sigmoid
# =================================================================================================

class KDAGateFunction(torch.autograd.Function):
    """g = -exp(A_log) * softplus(g_raw + dt_bias)  (or lower_bound * sigmoid(exp(A_log) * (g_raw + dt_bias))) and,
    when `beta_raw` is given, beta = sigmoid(beta_raw); both come out in float32.  Mirrors KDAGateFunction and the
    beta sigmoid of fla (fla/ops/kda/gate.py:282-318, fla/ops/kda/chunk.py:58-61,158-160)."""

    @staticmethod
    def forward(ctx, g_raw, A_log, dt_bias, beta_raw, lower_bound):
        if not g_raw.is_cuda:
            raise RuntimeError("kda_b200 runs on CUDA (sm_100a) tensors only; there is no CPU path")
        H, K = g_raw.shape[-2:]
        if K % 8:
            raise NotImplementedError(f"kda_b200: the gate kernels need K to be a multiple of 8, got {K}")
        if g_raw.dtype not in _DT or (beta_raw is not None and beta_raw.dtype not in _DT):
            raise NotImplementedError("kda_b200: raw gate / beta inputs must be bfloat16 or float32")
        assert A_log.numel() == H, f"A_log must have H={H} elements, got {A_log.numel()}"
        assert dt_bias is None or dt_bias.numel() == H * K, f"dt_bias must have H*K={H * K} elements"
        dev = g_raw.device
        g_raw = g_raw.contiguous()
        A32 = A_log.detach().contiguous().float()
        b32 = dt_bias.detach().contiguous().float() if dt_bias is not None else None
        beta_raw = beta_raw.contiguous() if beta_raw is not None else None
        tokens = g_raw.numel() // (H * K)
        g = torch.empty(g_raw.shape, dtype=torch.float32, device=dev)
        beta = torch.empty(beta_raw.shape, dtype=torch.float32, device=dev) if beta_raw is not None else None
        a = _lib.GateArgs(g_raw=_ptr(g_raw), A_log=_ptr(A32), dt_bias=_ptr(b32), beta_raw=_ptr(beta_raw), g=_ptr(g),
                          beta=_ptr(beta), tokens=tokens, H=H, K=K, g_dtype=_DT[g_raw.dtype],
                          beta_dtype=_DT[beta_raw.dtype] if beta_raw is not None else _lib.KDA_FP32,
                          use_lower_bound=int(lower_bound is not None), lower_bound=float(lower_bound or 0.0))
        with torch.cuda.device(dev):
            _lib.check(_lib.load().kda_gate_fwd(C.byref(a), _stream(dev)), "kda_gate_fwd")
        ctx.save_for_backward(g_raw, A32, b32, beta_raw)
        ctx.meta = (tokens, H, K, lower_bound, A_log.dtype, A_log.shape, dt_bias.dtype if dt_bias is not None else None,
                    dt_bias.shape if dt_bias is not None else None)
        return g, beta

    @staticmethod
    def backward(ctx, dg, dbeta):
        g_raw, A32, b32, beta_raw = ctx.saved_tensors
        tokens, H, K, lower_bound, A_dtype, A_shape, b_dtype, b_shape = ctx.meta
        dev = g_raw.device
        lib = _lib.load()
        if dg is None:
            dg = torch.zeros(g_raw.shape, dtype=torch.float32, device=dev)
        dg = dg.contiguous().float()
        dg_raw = torch.empty_like(g_raw)
        dA = torch.empty(H, dtype=torch.float32, device=dev)
        db = torch.empty(H * K, dtype=torch.float32, device=dev) if b32 is not None else None
        dbeta_raw = None
        if beta_raw is not None:
            dbeta = dbeta.contiguous().float() if dbeta is not None else torch.zeros(beta_raw.shape, dtype=torch.float32, device=dev)
            dbeta_raw = torch.empty_like(beta_raw)
        ws = torch.empty(lib.kda_gate_bwd_workspace_bytes(tokens, H, K), dtype=torch.uint8, device=dev)
        a = _lib.GateArgs(g_raw=_ptr(g_raw), A_log=_ptr(A32), dt_bias=_ptr(b32), beta_raw=_ptr(beta_raw), dg=_ptr(dg),
                          dbeta=_ptr(dbeta if beta_raw is not None else None), dg_raw=_ptr(dg_raw), dbeta_raw=_ptr(dbeta_raw),
                          dA_log=_ptr(dA), ddt_bias=_ptr(db), workspace=_ptr(ws), workspace_bytes=ws.numel(), tokens=tokens,
                          H=H, K=K, g_dtype=_DT[g_raw.dtype],
                          beta_dtype=_DT[beta_raw.dtype] if beta_raw is not None else _lib.KDA_FP32,
                          use_lower_bound=int(lower_bound is not None), lower_bound=float(lower_bound or 0.0))
        with torch.cuda.device(dev):
            _lib.check(lib.kda_gate_bwd(C.byref(a), _stream(dev)), "kda_gate_bwd")
        return (dg_raw, dA.view(A_shape).to(A_dtype), db.view(b_shape).to(b_dtype) if db is not None else None,
                dbeta_raw, None)


@torch.compiler.disable
def fused_kda_gate(g, A_log, dt_bias=None, lower_bound=None, output_dtype=torch.float32):
    """Drop-in for fla.ops.kda.gate.fused_kda_gate (fla/ops/kda/gate.py:321-344): the decay activation with
    autograd.  g [..., H, K] raw gate input, A_log [H], dt_bias [H*K] or None."""
    out, _ = KDAGateFunction.apply(g, A_log, dt_bias, None, lower_bound)
    return out if output_dtype == torch.float32 else out.to(output_dtype)


def _gate_front_end(g, beta, use_gate_in_kernel, use_beta_sigmoid_in_kernel, safe_gate, lower_bound, kwargs):
    """Applies the options of the operator that activate g and beta before the recurrence
    (fla/ops/kda/chunk.py:365-378): returns (g, beta) as the chunked / recurrent kernels want them."""
    A_log, dt_bias = None, None
    if use_gate_in_kernel:
        assert "A_log" in kwargs, "A_log must be provided when use_gate_in_kernel=True."
        A_log, dt_bias = kwargs["A_log"], kwargs.get("dt_bias")
        if safe_gate:
            if lower_bound is None:
                raise ValueError("`lower_bound` must be specified when `safe_gate=True` and `use_gate_in_kernel=True`.")
            if not (-5 <= lower_bound < 0):
                raise ValueError(f"`lower_bound` must be in the safe range [-5, 0), got {lower_bound}.")
    if use_gate_in_kernel:
        g, b = KDAGateFunction.apply(g, A_log, dt_bias, beta if use_beta_sigmoid_in_kernel else None, lower_bound)
        if use_beta_sigmoid_in_kernel:
            beta = b
    elif use_beta_sigmoid_in_kernel:
        beta = BetaSigmoidFunction.apply(beta)
    return g, beta


class BetaSigmoidFunction(torch.autograd.Function):
    """beta = sigmoid(beta_raw) in float32 without the gate (use_beta_sigmoid_in_kernel alone;
    fla/ops/kda/chunk.py:58-61,158-160)."""

    @staticmethod
    def _args(beta_raw, **kw):
        H = beta_raw.shape[-1]
        return _lib.GateArgs(beta_raw=_ptr(beta_raw), tokens=beta_raw.numel() // H, H=H, K=8, g_dtype=_lib.KDA_FP32,
                             beta_dtype=_DT[beta_raw.dtype], **{n: _ptr(t) for n, t in kw.items()})

    @staticmethod
    def forward(ctx, beta_raw):
        if not beta_raw.is_cuda:
            raise RuntimeError("kda_b200 runs on CUDA (sm_100a) tensors only; there is no CPU path")
        if beta_raw.dtype not in _DT:
            raise NotImplementedError("kda_b200: raw beta must be bfloat16 or float32")
        beta_raw = beta_raw.contiguous()
        beta = torch.empty(beta_raw.shape, dtype=torch.float32, device=beta_raw.device)
        with torch.cuda.device(beta_raw.device):
            _lib.check(_lib.load().kda_gate_fwd(C.byref(BetaSigmoidFunction._args(beta_raw, beta=beta)), _stream(beta_raw.device)),
                       "kda_gate_fwd")
        ctx.save_for_backward(beta_raw)
        return beta

    @staticmethod
    def backward(ctx, dbeta):
        (beta_raw,) = ctx.saved_tensors
        dbeta = dbeta.contiguous().float()
        dbeta_raw = torch.empty_like(beta_raw)
        with torch.cuda.device(beta_raw.device):
            _lib.check(_lib.load().kda_gate_bwd(C.byref(BetaSigmoidFunction._args(beta_raw, dbeta=dbeta, dbeta_raw=dbeta_raw)),
                                                _stream(beta_raw.device)), "kda_gate_bwd")
        return dbeta_raw


# =================================================================================================
# decode / token-recurrent forward
# =================================================================================================

def fused_recurrent_kda_fwd(q, k, v, g, beta, A_log=None, dt_bias=None, initial_state=None, scale=None,
                            output_final_state=False, inplace_final_state=True, cu_seqlens=None, ssm_state_indices=None,
                            num_accepted_tokens=None, use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False,
                            use_beta_sigmoid_in_kernel=False, lower_bound=None, out=None, transpose_state_layout=False,
                            **kwargs):
    """Lower-level decode entry with fla's signature (fla/ops/kda/fused_recurrent.py:229-325), forward only.

    With `inplace_final_state` the kernel writes states over `initial_state` and returns that tensor.
    Continuous batching: `ssm_state_indices` [N] or [N, T] names the state slot of every token; a sequence starts
    from the slot of its first token -- with `num_accepted_tokens` [N] (speculative decoding) from the slot of its
    last accepted token -- and the state after token t lands in slot `ssm_state_indices[n, t]`.
    `transpose_state_layout`: states are [N, H, V, K] instead of [N, H, K, V] (K = 64 or 128)."""
    B, T, H, K, V = _check_common(q, k, v, g, beta, None, cu_seqlens)
    if transpose_state_layout and K not in (64, 128):
        raise NotImplementedError(f"kda_b200: transpose_state_layout needs K = 64 or 128, got {K}")
    if scale is None:
        scale = K ** -0.5
    dev = q.device
    # the gate activation and the beta sigmoid run inside the recurrent kernels (no separate pass over g and beta)
    gate_kw = {}
    if use_gate_in_kernel:
        assert A_log is not None, "A_log must be provided when use_gate_in_kernel=True."
        if g.dtype not in _DT:
            g = g.float()
        a_log = A_log.detach().to(device=dev, dtype=torch.float32).contiguous()
        bias = dt_bias.detach().to(device=dev, dtype=torch.float32).contiguous() if dt_bias is not None else None
        if a_log.numel() != H or (bias is not None and bias.numel() != H * K):
            raise ValueError(f"A_log must have {H} elements and dt_bias {H * K}")
        gate_kw.update(A_log=_ptr(a_log), dt_bias=_ptr(bias), g_raw_dtype=_DT[g.dtype],
                       lower_bound=float(lower_bound) if lower_bound is not None else 0.0,
                       use_lower_bound=int(lower_bound is not None))
        g = g.detach().contiguous()
    else:
        g = g.contiguous().float()
    if use_beta_sigmoid_in_kernel:
        if beta.dtype not in _DT:
            beta = beta.float()
        gate_kw.update(beta_sigmoid=1, beta_raw_dtype=_DT[beta.dtype])
        beta = beta.detach().contiguous()
    else:
        beta = beta.contiguous().float()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    N = B if cu_seqlens is None else len(cu_seqlens) - 1
    cu = _as_i32(cu_seqlens, dev) if cu_seqlens is not None else None
    h0 = initial_state.contiguous() if initial_state is not None else None
    if inplace_final_state:
        assert initial_state is not None
        if h0.data_ptr() != initial_state.data_ptr() or h0.dtype != torch.float32:
            raise ValueError("inplace_final_state needs a contiguous fp32 initial_state")
        ht = h0
    elif output_final_state:
        ht = torch.empty((N, H, V, K) if transpose_state_layout else (N, H, K, V), dtype=torch.float32, device=dev)
    else:
        ht = None
    idx, acc, stride = None, None, 0
    if ssm_state_indices is not None:
        if not inplace_final_state:
            raise ValueError("ssm_state_indices requires inplace_final_state=True")
        idx = ssm_state_indices.to(device=dev, dtype=torch.int32).contiguous()
        stride = 1 if idx.ndim == 1 else idx.stride(0)
        if idx.ndim == 1 and cu_seqlens is None and T > 1:
            raise ValueError("ssm_state_indices must be [N, T] when a sequence has more than one token")
        if num_accepted_tokens is not None:
            acc = num_accepted_tokens.to(device=dev, dtype=torch.int32).contiguous()
    elif num_accepted_tokens is not None:
        raise ValueError("num_accepted_tokens requires ssm_state_indices")
    if out is None:
        o = torch.empty_like(v)
    else:
        assert out.shape == v.shape
        if not out.is_contiguous() or out.dtype != v.dtype:
            raise ValueError("`out` must be contiguous and of v's dtype")
        o = out
    args = _lib.RecurrentArgs(
        q=_ptr(q), k=_ptr(k), v=_ptr(v), g=_ptr(g), beta=_ptr(beta), h0=_ptr(h0), ht=_ptr(ht), o=_ptr(o),
        cu_seqlens=_ptr(cu), state_indices=_ptr(idx), tokens=B * T, N=N, T=T, H=H, K=K, V=V,
        io_dtype=_DT[q.dtype], use_qk_l2norm=int(bool(use_qk_l2norm_in_kernel)), scale=float(scale),
        num_accepted_tokens=_ptr(acc), state_indices_stride=stride, transpose_state=int(bool(transpose_state_layout)),
        HQ=q.shape[2], **gate_kw)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().kda_recurrent_fwd(C.byref(args), _stream(dev)), "kda_recurrent_fwd")
        if _checked():
            st = _lib.recurrent_status()
            if st:
                raise _lib.KdaError(f"kda_recurrent_fwd: device status 0x{st:x} (a bounded wait gave up); the outputs are incomplete")
    return o, ht


@torch.no_grad()
def fused_recurrent_kda(q, k, v, g, beta, A_log=None, dt_bias=None, scale=None, initial_state=None,
                        output_final_state=False, use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False,
                        use_beta_sigmoid_in_kernel=False, lower_bound=None, cu_seqlens=None,
                        transpose_state_layout=False, **kwargs):
    """Drop-in for fla.ops.kda.fused_recurrent_kda (fla/ops/kda/fused_recurrent.py:329-452): forward only.
    q,k [B,T,H,K]; v [B,T,H,V]; g [B,T,H,K] log-decay (raw gate input with `use_gate_in_kernel`, activated with
    `A_log`, `dt_bias`, `lower_bound` as in chunk_kda); beta [B,T,H] (logits with `use_beta_sigmoid_in_kernel`);
    initial_state [N,H,K,V] fp32 ([N,H,V,K] with `transpose_state_layout`).  Returns (o, final_state or None)."""
    if "use_qk_l2norm" in kwargs:
        use_qk_l2norm_in_kernel = kwargs.pop("use_qk_l2norm")
    _check_common(q, k, v, g, beta, initial_state, cu_seqlens)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    return fused_recurrent_kda_fwd(q, k, v, g, beta, A_log=A_log, dt_bias=dt_bias, initial_state=initial_state, scale=scale,
                                   output_final_state=output_final_state, inplace_final_state=False, cu_seqlens=cu_seqlens,
                                   use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, use_gate_in_kernel=use_gate_in_kernel,
                                   use_beta_sigmoid_in_kernel=use_beta_sigmoid_in_kernel, lower_bound=lower_bound,
                                   transpose_state_layout=transpose_state_layout)


class RecurrentKDAFunction(torch.autograd.Function):
    """float32 path of chunk_kda with gradients: forward by the token-recurrent fp32 kernel, backward by its exact
    reverse-mode counterpart (`kda_recurrent_bwd`, fla/ops/kda/naive.py:12-66 differentiated).  K, V in {32, 64, 128}."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, use_l2norm, cu_seqlens):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        g32, beta32 = g.contiguous().float(), beta.contiguous().float()
        h0 = initial_state.contiguous().float() if initial_state is not None else None
        o, ht = fused_recurrent_kda_fwd(q, k, v, g32, beta32, initial_state=h0, scale=scale,
                                        output_final_state=output_final_state, inplace_final_state=False,
                                        use_qk_l2norm_in_kernel=use_l2norm, cu_seqlens=cu_seqlens)
        cu = _as_i32(cu_seqlens, q.device) if cu_seqlens is not None else None
        ctx.save_for_backward(q, k, v, g32, beta32, h0, cu)
        ctx.meta = (float(scale), bool(use_l2norm), g.dtype, beta.dtype)
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, g32, beta32, h0, cu = ctx.saved_tensors
        scale, use_l2norm, g_dtype, beta_dtype = ctx.meta
        B, T, HQ, K = q.shape
        H, V = v.shape[-2], v.shape[-1]
        N = B if cu is None else cu.numel() - 1
        dev = q.device
        lib = _lib.load()
        do = do.contiguous().float()
        dht = dht.contiguous().float() if dht is not None else None
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dg, dbeta = torch.empty_like(g32), torch.empty_like(beta32)
        dh0 = torch.empty(N, H, K, V, dtype=torch.float32, device=dev) if h0 is not None else None
        ws = torch.empty(lib.kda_recurrent_bwd_workspace_bytes(B * T, N, H, K, V), dtype=torch.uint8, device=dev)
        args = _lib.RecurrentBwdArgs(
            q=_ptr(q), k=_ptr(k), v=_ptr(v), g=_ptr(g32), beta=_ptr(beta32), h0=_ptr(h0), cu_seqlens=_ptr(cu),
            d_o=_ptr(do), d_ht=_ptr(dht), dq=_ptr(dq), dk=_ptr(dk), dv=_ptr(dv), dg=_ptr(dg), dbeta=_ptr(dbeta), dh0=_ptr(dh0),
            workspace=_ptr(ws), workspace_bytes=ws.numel(), tokens=B * T, N=N, T=T, H=H, K=K, V=V, HQ=HQ,
            io_dtype=_lib.KDA_FP32, use_qk_l2norm=int(use_l2norm), scale=scale)
        with torch.cuda.device(dev):
            _lib.check(lib.kda_recurrent_bwd(C.byref(args), _stream(dev)), "kda_recurrent_bwd")
        return dq, dk, dv, dg.to(g_dtype), dbeta.to(beta_dtype), None, dh0, None, None, None


# =================================================================================================
# chunked forward / backward
# =================================================================================================

def _chunk_args(q, k, v, g, beta, h0, cu, o, ht, ws, N, H, K, V, tokens, l2, save, scale, **extra):
    a = _lib.ChunkArgs(
        q=_ptr(q), k=_ptr(k), v=_ptr(v), g=_ptr(g), beta=_ptr(beta), h0=_ptr(h0), cu_seqlens=_ptr(cu),
        o=_ptr(o), ht=_ptr(ht), workspace=_ptr(ws), workspace_bytes=ws.numel() if ws is not None else 0,
        tokens=tokens, N=N, H=H, K=K, V=V, io_dtype=_lib.KDA_BF16, use_qk_l2norm=int(l2),
        save_for_backward=int(save), scale=float(scale), HQ=q.shape[-2], scan_slices=int(SCAN_SLICES),
        safe_gate=int(bool(extra.pop("safe_gate", False))))
    for name, t in extra.items():
        if name == "bwd_ws":
            a.bwd_workspace = _ptr(t)
            a.bwd_workspace_bytes = t.numel()
        else:
            setattr(a, name, _ptr(t))
    return a


class ChunkKDAFunction(torch.autograd.Function):
    """bf16 chunked path.  Saved for backward: the inputs plus one workspace buffer in which the forward
    kernels left the per-chunk tiles the backward kernels read (fla/ops/kda/chunk.py:22-162 keeps the
    inputs and recomputes; with 180 GB of HBM the tiles are kept instead)."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, use_l2norm, cu_seqlens, safe_gate=False):
        B, T, HQ, K = q.shape
        H, V = v.shape[-2], v.shape[-1]          # H counts value heads; q and k may have fewer (grouped value heads)
        dev = q.device
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        g32 = g.contiguous().float()
        beta32 = beta.contiguous().float()
        h0 = initial_state.contiguous() if initial_state is not None else None
        if cu_seqlens is None:
            N, cu = B, _fixed_cu_seqlens(B, T, dev)
        else:
            cu = _as_i32(cu_seqlens, dev)
            N = cu.numel() - 1
        tokens = B * T
        need_grad = any(ctx.needs_input_grad)
        save = (1 | (2 if use_l2norm else 0)) if need_grad else 0      # bit 1: the forward keeps the normalised q, k
        lib = _lib.load()
        ws = torch.empty(lib.kda_chunk_workspace_bytes(tokens, N, H, K, V, save), dtype=torch.uint8, device=dev)
        o = torch.empty_like(v)
        ht = torch.empty(N, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
        args = _chunk_args(q, k, v, g32, beta32, h0, cu, o, ht, ws, N, H, K, V, tokens, use_l2norm, save, scale, safe_gate=safe_gate)
        with torch.cuda.device(dev):
            _lib.check(lib.kda_chunk_fwd(C.byref(args), _stream(dev)), "kda_chunk_fwd")
            if _checked():
                _lib.check_chunk_status(ws.data_ptr(), "kda_chunk_fwd")
        if need_grad:
            ctx.save_for_backward(q, k, v, g32, beta32, h0, cu, ws)
            ctx.meta = (N, H, K, V, tokens, use_l2norm, scale, g.dtype, beta.dtype, initial_state is not None, HQ)
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, g32, beta32, h0, cu, ws = ctx.saved_tensors
        N, H, K, V, tokens, use_l2norm, scale, g_dtype, beta_dtype, has_h0, HQ = ctx.meta
        dev = q.device
        lib = _lib.load()
        do = do.contiguous()
        dht = dht.contiguous().float() if dht is not None else None
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dg = torch.empty_like(g32)
        dbeta = torch.empty_like(beta32)
        dh0 = torch.empty(N, H, K, V, dtype=torch.float32, device=dev) if has_h0 else None
        flags = int(use_l2norm) | (2 if HQ != H else 0) | (4 if use_l2norm else 0)
        bws = torch.empty(lib.kda_chunk_bwd_workspace_bytes(tokens, N, H, K, V, flags), dtype=torch.uint8, device=dev)
        args = _chunk_args(q, k, v, g32, beta32, h0, cu, None, None, ws, N, H, K, V, tokens, use_l2norm, 1 | (2 if use_l2norm else 0), scale,
                           d_o=do, d_ht=dht, dq=dq, dk=dk, dv=dv, dg=dg, dbeta=dbeta, dh0=dh0, bwd_ws=bws)
        with torch.cuda.device(dev):
            _lib.check(lib.kda_chunk_bwd(C.byref(args), _stream(dev)), "kda_chunk_bwd")
            if _checked():
                _lib.check_chunk_status(ws.data_ptr(), "kda_chunk_bwd")
        return dq, dk, dv, dg.to(g_dtype), dbeta.to(beta_dtype), None, dh0, None, None, None, None


def _chunk_fwd_with_states(q, k, v, g, beta, scale, initial_state, output_final_state, use_l2norm, cu_seqlens, chunk_size=CHUNK,
                           safe_gate=False):
    """Forward for inference engines (fla/ops/kda/chunk.py:95-98): also returns h, the state at the start of every
    chunk of `chunk_size` tokens, [B, NT, H, K, V] bf16 (NT chunks per sequence; with cu_seqlens B = 1 and NT counts all
    chunks).  The kernels tile by 64 tokens and keep the state at the start of every 64-token chunk; for chunk_size = 32
    the state in the middle of a chunk is that chunk's start state advanced over its first 32 tokens by the
    token-recurrent kernel (one short sequence per chunk)."""
    B, T, _, K = q.shape
    H, V = v.shape[-2], v.shape[-1]
    dev = q.device
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    g32, beta32 = g.contiguous().float(), beta.contiguous().float()
    h0 = initial_state.contiguous() if initial_state is not None else None
    if cu_seqlens is None:
        N, cu = B, _fixed_cu_seqlens(B, T, dev)
        starts, lens = [b * T for b in range(B)], [T] * B
    else:
        cu = _as_i32(cu_seqlens, dev)
        N = cu.numel() - 1
        cul = cu.cpu().tolist()                               # the output shape depends on the lengths: one host read
        starts, lens = cul[:-1], [cul[i + 1] - cul[i] for i in range(N)]
    tokens = B * T
    lib = _lib.load()
    ws = torch.empty(lib.kda_chunk_workspace_bytes(tokens, N, H, K, V, 1), dtype=torch.uint8, device=dev)
    o = torch.empty_like(v)
    ht = torch.empty(N, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
    hbuf = torch.empty(lib.kda_chunk_max_chunks(tokens, N), H, K, V, dtype=torch.bfloat16, device=dev)
    args = _chunk_args(q, k, v, g32, beta32, h0, cu, o, ht, ws, N, H, K, V, tokens, use_l2norm, True, scale, safe_gate=safe_gate)
    with torch.cuda.device(dev):
        _lib.check(lib.kda_chunk_fwd(C.byref(args), _stream(dev)), "kda_chunk_fwd")
        _lib.check(lib.kda_chunk_export_states(_ptr(ws), ws.numel(), tokens, N, H, _ptr(hbuf), _stream(dev)), "kda_chunk_export_states")
        if _checked():
            _lib.check_chunk_status(ws.data_ptr(), "kda_chunk_fwd")
    nt64 = [(n + CHUNK - 1) // CHUNK for n in lens]
    h64 = hbuf[:sum(nt64)]
    if chunk_size == CHUNK:
        h = h64
        nt = nt64
    else:
        # states every 32 tokens: even positions are the 64-token chunks' start states; an odd position exists where the
        # chunk has more than 32 tokens and is that chunk's state after its first 32 tokens
        half = CHUNK // 2
        nt = [(n + half - 1) // half for n in lens]
        h = torch.empty(sum(nt), H, K, V, dtype=torch.bfloat16, device=dev)
        even_dst, odd_dst, odd_src, tok = [], [], [], []
        base32 = base64 = 0
        for s0, n, c64, c32 in zip(starts, lens, nt64, nt):
            for c in range(c64):
                even_dst.append(base32 + 2 * c)
                if n - c * CHUNK > half:
                    odd_dst.append(base32 + 2 * c + 1)
                    odd_src.append(base64 + c)
                    tok.append(s0 + c * CHUNK)
            base32, base64 = base32 + c32, base64 + c64
        h[torch.tensor(even_dst, device=dev, dtype=torch.long)] = h64
        if odd_dst:
            idx = (torch.tensor(tok, device=dev, dtype=torch.long).unsqueeze(1) + torch.arange(half, device=dev)).reshape(-1)
            flat = lambda t: t.reshape(tokens, *t.shape[2:]).index_select(0, idx).unsqueeze(0)      # noqa: E731
            seg_cu = torch.arange(0, len(tok) * half + 1, half, dtype=torch.int32, device=dev)
            start_state = h64.index_select(0, torch.tensor(odd_src, device=dev, dtype=torch.long)).float()
            _, mid = fused_recurrent_kda_fwd(flat(q), flat(k), flat(v), flat(g32), flat(beta32), initial_state=start_state, scale=scale,
                                             output_final_state=True, inplace_final_state=False, cu_seqlens=seg_cu,
                                             use_qk_l2norm_in_kernel=use_l2norm)
            h[torch.tensor(odd_dst, device=dev, dtype=torch.long)] = mid.to(torch.bfloat16)
    if cu_seqlens is None:
        return o, ht, h.view(B, nt[0], H, K, V)
    return o, ht, h.view(1, sum(nt), H, K, V)


@torch.compiler.disable
def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
              cu_seqlens=None, cu_seqlens_cpu=None, safe_gate=False, lower_bound=None, disable_recompute=False,
              return_intermediate_states=False, cp_context=None, transpose_state_layout=False, **kwargs):
    """Drop-in for fla.ops.kda.chunk_kda (fla/ops/kda/chunk.py:167-411).

    q, k [B,T,H,K]; v [B,T,HV,V]; g [B,T,HV,K] log-space decay; beta [B,T,HV]; initial_state [N,HV,K,V] fp32;
    cu_seqlens [N+1] with B == 1.  HV is a multiple of H (grouped value heads: value head h reads q/k head
    h // (HV // H); dq, dk are summed over each group).  With `use_gate_in_kernel=True` g is the raw gate input and `A_log` [H]
    (and optionally `dt_bias` [H*K]) are keyword arguments: g = -exp(A_log) softplus(g + dt_bias), or, with
    `lower_bound`, lower_bound * sigmoid(exp(A_log) (g + dt_bias)); with `use_beta_sigmoid_in_kernel=True` beta
    holds logits.  Returns (o, final_state or None); differentiable w.r.t. q, k, v, g, beta, initial_state,
    A_log and dt_bias.  With `return_intermediate_states=True` (inference mode only) a third value h
    [B, NT, H, K, V] bf16 holds the state at the start of every chunk.  `transpose_state_layout`: every state
    tensor is [.., V, K] instead of [.., K, V].

    bf16 inputs with K, V <= 128 take the chunked tensor-core kernels (built for K = V = 128; smaller heads are
    zero-padded to 128 channels, which leaves every result unchanged; K = 256 runs forward-only through the
    token-recurrent kernel).  float32 inputs take the exact
    token-recurrent fp32 kernels: forward for K in {32, 64, 128, 256}, with gradients for K, V in {32, 64, 128}.  `safe_gate=True` is the caller's promise that every gate value is at least
    -5 (fla/ops/kda/chunk.py:235-246); the forward then computes the diagonal 16 x 16 blocks of the intra-chunk products on
    tensor cores as well (factored around each block's middle row) instead of pairwise, which is faster and only safe under
    that bound; without it the kernels are range-safe for any gate.  `disable_recompute` only selects a variant of the
    same computation upstream and is accepted as a no-op; `chunk_size` (32 or
    64) changes nothing but the spacing of the intermediate states (the kernels always tile by 64 tokens); options
    that change results and are not built raise.
    """
    _unsupported("cp_context", cp_context, None)
    if "use_qk_l2norm" in kwargs:
        use_qk_l2norm_in_kernel = kwargs.pop("use_qk_l2norm")
    chunk_size = kwargs.pop("chunk_size", 64)
    if chunk_size not in (32, 64):
        raise ValueError(f"`chunk_size` must be either 32 or 64 for KDA, got {chunk_size}.")
    # chunk_size only selects how the same recurrence is tiled: o, the final state and every gradient are the same
    # function of the inputs for 32 and 64, so both run on the 64-token tiles.  Only the intermediate states depend on
    # it (one state per chunk of that size, see _chunk_fwd_with_states).
    B, T, H, K, V = _check_common(q, k, v, g, beta, initial_state, cu_seqlens)
    if scale is None:
        scale = K ** -0.5
    g, beta = _gate_front_end(g, beta, use_gate_in_kernel, use_beta_sigmoid_in_kernel, safe_gate, lower_bound, kwargs)
    if q.dtype == torch.float32:
        if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state)):
            if K not in (32, 64, 128) or V not in (32, 64, 128) or return_intermediate_states:
                raise NotImplementedError(f"kda_b200: float32 gradients need K, V in {{32, 64, 128}}, got K={K}, V={V}")
            tr = (lambda t: t.transpose(-1, -2)) if transpose_state_layout else (lambda t: t)
            o, ht = RecurrentKDAFunction.apply(q, k, v, g, beta, float(scale), tr(initial_state) if initial_state is not None else None,
                                               bool(output_final_state), bool(use_qk_l2norm_in_kernel), cu_seqlens)
            return o, (tr(ht).contiguous() if (transpose_state_layout and ht is not None) else ht)
        return fused_recurrent_kda_fwd(q, k, v, g, beta, initial_state=initial_state, scale=scale,
                                       output_final_state=output_final_state, inplace_final_state=False,
                                       use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, cu_seqlens=cu_seqlens,
                                       transpose_state_layout=transpose_state_layout)
    if K > 128 or V > 128:
        # larger heads (fla allows K <= 256): forward through the token-recurrent kernel (bf16 in and out, fp32 state),
        # which serves K = 256; there is no backward for them
        needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state))
        if needs_grad or return_intermediate_states or K != 256 or V % 32 != 0 or (transpose_state_layout and K not in (64, 128)):
            raise NotImplementedError(f"kda_b200: the bf16 chunked kernels are built for head sizes up to 128, got K={K}, V={V} "
                                      "(K = 256 runs forward-only)")
        return fused_recurrent_kda_fwd(q, k, v, g, beta, initial_state=initial_state, scale=scale,
                                       output_final_state=output_final_state, inplace_final_state=False,
                                       use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, cu_seqlens=cu_seqlens)
    # transposed state layout ([N, H, V, K]): the chunk kernels keep [N, H, K, V]; states cross the boundary once per
    # sequence, so they are transposed there (differentiably)
    tr = (lambda t: t.transpose(-1, -2)) if transpose_state_layout else (lambda t: t)
    if initial_state is not None:
        initial_state = tr(initial_state)
    # Smaller heads ride on the 128-wide kernels: key channels padded with k = q = 0 and g = 0 (decay 1) and value
    # channels padded with v = 0 never touch the real ones -- the padded state rows and columns stay zero, the row norms
    # of q and k are unchanged -- so o, the states and (through autograd of the padding) every gradient are those of
    # the unpadded problem.  `scale` was fixed from the real K above.
    pad_k, pad_v = 128 - K, 128 - V
    if pad_k or pad_v:
        padk = lambda t: torch.nn.functional.pad(t, (0, pad_k))      # noqa: E731
        q, k, g, v = padk(q), padk(k), padk(g), torch.nn.functional.pad(v, (0, pad_v))
        if initial_state is not None:
            initial_state = torch.nn.functional.pad(initial_state, (0, pad_v, 0, pad_k))
    if return_intermediate_states:
        assert torch.is_inference_mode_enabled(), "return_intermediate_states is only allowed in inference mode"
        assert disable_recompute is False, "return_intermediate_states must be used with disable_recompute=False"
        o, ht, h = _chunk_fwd_with_states(q, k, v, g, beta, float(scale), initial_state, bool(output_final_state),
                                          bool(use_qk_l2norm_in_kernel), cu_seqlens, chunk_size, bool(safe_gate))
        if pad_k or pad_v:
            o, ht, h = o[..., :V], (ht[..., :K, :V] if ht is not None else None), h[..., :K, :V]
        if transpose_state_layout:
            ht, h = (tr(ht).contiguous() if ht is not None else None), tr(h).contiguous()
        return o, ht, h
    o, ht = ChunkKDAFunction.apply(q, k, v, g, beta, float(scale), initial_state, bool(output_final_state),
                                   bool(use_qk_l2norm_in_kernel), cu_seqlens, bool(safe_gate))
    if pad_k or pad_v:
        o, ht = o[..., :V], (ht[..., :K, :V] if ht is not None else None)
    if transpose_state_layout and ht is not None:
        ht = tr(ht).contiguous()
    return o, ht


def default_scale(K: int) -> float:
    return 1.0 / math.sqrt(K)
