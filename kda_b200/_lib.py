"""ctypes binding of libkda_b200.so (the C ABI declared in include/kda_b200.h).

There is no fallback: if the shared library is missing or does not load, importing an operator raises."""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libkda_b200.so")

KDA_BF16, KDA_FP32 = 0, 1
NOALLOC_SCRATCH_BYTES = 32 << 20
ABI_VERSION = 9


class RecurrentArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
        ("h0", C.c_void_p), ("ht", C.c_void_p), ("o", C.c_void_p), ("cu_seqlens", C.c_void_p),
        ("state_indices", C.c_void_p),
        ("tokens", C.c_int64), ("N", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("K", C.c_int32),
        ("V", C.c_int32), ("io_dtype", C.c_int32), ("use_qk_l2norm", C.c_int32), ("scale", C.c_float),
        ("num_accepted_tokens", C.c_void_p), ("state_indices_stride", C.c_int32), ("transpose_state", C.c_int32),
        ("HQ", C.c_int32),
        ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("lower_bound", C.c_float), ("use_lower_bound", C.c_int32),
        ("g_raw_dtype", C.c_int32), ("beta_sigmoid", C.c_int32), ("beta_raw_dtype", C.c_int32),
    ]


class ChunkArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
        ("h0", C.c_void_p), ("cu_seqlens", C.c_void_p),
        ("o", C.c_void_p), ("ht", C.c_void_p),
        ("d_o", C.c_void_p), ("d_ht", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dg", C.c_void_p), ("dbeta", C.c_void_p),
        ("dh0", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("bwd_workspace", C.c_void_p), ("bwd_workspace_bytes", C.c_size_t),
        ("tokens", C.c_int64), ("N", C.c_int32), ("H", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("io_dtype", C.c_int32), ("use_qk_l2norm", C.c_int32), ("save_for_backward", C.c_int32),
        ("scale", C.c_float), ("HQ", C.c_int32), ("scan_slices", C.c_int32), ("safe_gate", C.c_int32),
    ]


class RecurrentBwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
        ("h0", C.c_void_p), ("cu_seqlens", C.c_void_p), ("d_o", C.c_void_p), ("d_ht", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dg", C.c_void_p), ("dbeta", C.c_void_p),
        ("dh0", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("tokens", C.c_int64), ("N", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("HQ", C.c_int32), ("io_dtype", C.c_int32), ("use_qk_l2norm", C.c_int32), ("scale", C.c_float),
    ]


class GateArgs(C.Structure):
    _fields_ = [
        ("g_raw", C.c_void_p), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("beta_raw", C.c_void_p),
        ("g", C.c_void_p), ("beta", C.c_void_p), ("dg", C.c_void_p), ("dbeta", C.c_void_p),
        ("dg_raw", C.c_void_p), ("dbeta_raw", C.c_void_p), ("dA_log", C.c_void_p), ("ddt_bias", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("tokens", C.c_int64), ("H", C.c_int32), ("K", C.c_int32), ("g_dtype", C.c_int32), ("beta_dtype", C.c_int32),
        ("use_lower_bound", C.c_int32), ("lower_bound", C.c_float),
    ]


EXPORTS = (
    "kda_b200_abi_version", "kda_b200_strerror", "kda_recurrent_fwd", "kda_recurrent_status",
    "kda_recurrent_bwd_workspace_bytes", "kda_recurrent_bwd",
    "kda_chunk_max_chunks", "kda_chunk_workspace_bytes", "kda_chunk_bwd_workspace_bytes",
    "kda_chunk_fwd", "kda_chunk_bwd", "kda_chunk_status", "kda_chunk_fwd_noalloc", "kda_chunk_export_states",
    "kda_gate_bwd_workspace_bytes", "kda_gate_fwd", "kda_gate_bwd",
    "kda_copy_rows_async", "kda_b200_profile_enable", "kda_b200_profile_read",
)

_lib = None


def load() -> C.CDLL:
    """Loads the library once; raises RuntimeError with a build hint if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m kda_b200.build` (nvcc, sm_100a). "
            "kda_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    lib.kda_b200_abi_version.restype = C.c_int
    lib.kda_b200_strerror.restype = C.c_char_p
    lib.kda_b200_strerror.argtypes = [C.c_int]
    lib.kda_recurrent_fwd.restype = C.c_int
    lib.kda_recurrent_fwd.argtypes = [C.POINTER(RecurrentArgs), C.c_void_p]
    lib.kda_recurrent_status.restype = C.c_int
    lib.kda_recurrent_status.argtypes = [C.POINTER(C.c_uint32)]
    lib.kda_recurrent_bwd_workspace_bytes.restype = C.c_size_t
    lib.kda_recurrent_bwd_workspace_bytes.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    lib.kda_recurrent_bwd.restype = C.c_int
    lib.kda_recurrent_bwd.argtypes = [C.POINTER(RecurrentBwdArgs), C.c_void_p]
    lib.kda_chunk_max_chunks.restype = C.c_int64
    lib.kda_chunk_max_chunks.argtypes = [C.c_int64, C.c_int32]
    lib.kda_chunk_workspace_bytes.restype = C.c_size_t
    lib.kda_chunk_workspace_bytes.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    lib.kda_chunk_bwd_workspace_bytes.restype = C.c_size_t
    lib.kda_chunk_bwd_workspace_bytes.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    for name in ("kda_chunk_fwd", "kda_chunk_bwd", "kda_chunk_fwd_noalloc"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(ChunkArgs), C.c_void_p]
    lib.kda_chunk_status.restype = C.c_int
    lib.kda_chunk_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
    lib.kda_chunk_export_states.restype = C.c_int
    lib.kda_chunk_export_states.argtypes = [C.c_void_p, C.c_size_t, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.kda_gate_bwd_workspace_bytes.restype = C.c_size_t
    lib.kda_gate_bwd_workspace_bytes.argtypes = [C.c_int64, C.c_int32, C.c_int32]
    for name in ("kda_gate_fwd", "kda_gate_bwd"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(GateArgs), C.c_void_p]
    lib.kda_copy_rows_async.restype = C.c_int
    lib.kda_copy_rows_async.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]
    lib.kda_b200_profile_enable.restype = C.c_int
    lib.kda_b200_profile_enable.argtypes = [C.c_int]
    lib.kda_b200_profile_read.restype = C.c_int
    lib.kda_b200_profile_read.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_int]
    if lib.kda_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libkda_b200.so was built from a different ABI version; rebuild it")
    _lib = lib
    return lib


class KdaError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().kda_b200_strerror(code).decode()
        raise KdaError(f"{what} failed with code {code}: {msg}")


STAGES = ("tables", "prepare", "scan", "bwd_scan", "bwd_main", "l2norm", "gate_fwd", "gate_bwd")


def profile_enable(on: bool) -> None:
    check(load().kda_b200_profile_enable(int(on)), "kda_b200_profile_enable")


def recurrent_status() -> int:
    """Status word of the bulk-copy decode kernel since the last call (0 = every bounded wait completed); synchronises."""
    v = C.c_uint32(0)
    check(load().kda_recurrent_status(C.byref(v)), "kda_recurrent_status")
    return int(v.value)


STATUS_BITS = {0x1: "forward scan: operand tiles did not arrive", 0x2: "forward scan: a product did not complete",
               0x4: "reverse scan: operand tiles did not arrive", 0x8: "reverse scan: a product did not complete",
               0x20: "per-chunk backward: a tile's loads did not arrive", 0x40: "per-chunk backward: a product did not complete",
               0x100: "cu_seqlens is inconsistent with the number of tokens: nothing was computed"}


def chunk_status(workspace_ptr=None) -> int:
    """Status word of the chunked kernels for the workspace at `workspace_ptr` (None: the fixed array of
    kda_chunk_fwd_noalloc on the current device); 0 = nothing to report.  Synchronises with the device."""
    v = C.c_uint32(0)
    check(load().kda_chunk_status(C.c_void_p(workspace_ptr or 0), C.byref(v)), "kda_chunk_status")
    return int(v.value)


def check_chunk_status(workspace_ptr, what: str) -> None:
    """Raises KdaError when the chunked kernels reported a problem for this workspace."""
    v = chunk_status(workspace_ptr)
    if v:
        why = "; ".join(t for b, t in STATUS_BITS.items() if v & b) or "unknown bits"
        raise KdaError(f"{what}: device status 0x{v:x} ({why}); the outputs of this call are incomplete")


def profile_read(reset: bool = True) -> dict:
    """{stage: (total_ms, launches)} of the chunk kernels since the last reset (waits for the events)."""
    ms = (C.c_float * len(STAGES))()
    n = (C.c_int * len(STAGES))()
    check(load().kda_b200_profile_read(ms, n, int(reset)), "kda_b200_profile_read")
    return {s: (float(ms[i]), int(n[i])) for i, s in enumerate(STAGES)}
