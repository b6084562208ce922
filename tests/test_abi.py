"""CPU tests of the C-ABI boundary: the library loads, exports every declared symbol, and rejects bad
arguments on the host without touching a GPU."""
import ctypes as C
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    ge.build()
    from kda_b200 import _lib
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    import __graft_entry__ as ge
    names = ge.declared_symbols()
    assert {"kda_recurrent_fwd", "kda_chunk_fwd", "kda_chunk_bwd", "kda_b200_strerror"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n


def test_exports_nothing_but_the_declared_symbols(lib):
    """The header says its entries are the library's only exports: development checks live in libkda_b200_debug.so."""
    import subprocess
    import __graft_entry__ as ge
    from kda_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    assert exported == set(ge.declared_symbols()) == set(_lib.EXPORTS)


def test_version_and_error_text(lib):
    import re
    from kda_b200 import _lib
    header = open(os.path.join(ROOT, "include", "kda_b200.h")).read()
    assert lib.kda_b200_abi_version() == int(re.search(r"#define KDA_B200_ABI_VERSION (\d+)", header).group(1)) == _lib.ABI_VERSION
    assert lib.kda_b200_strerror(0) == b"ok"
    assert b"NULL" in lib.kda_b200_strerror(-1)
    assert b"workspace" in lib.kda_b200_strerror(-5)
    assert b"tensor map" in lib.kda_b200_strerror(-8)
    assert lib.kda_chunk_status(None, None) == -1


def test_workspace_sizes_are_monotone(lib):
    a = lib.kda_chunk_workspace_bytes(4096, 1, 2, 128, 128, 0)
    b = lib.kda_chunk_workspace_bytes(4096, 1, 2, 128, 128, 1)
    c = lib.kda_chunk_workspace_bytes(8192, 1, 2, 128, 128, 1)
    assert 0 < a < b < c
    assert lib.kda_chunk_max_chunks(130, 2) == 4
    assert lib.kda_chunk_bwd_workspace_bytes(4096, 1, 2, 128, 128, 0) > 0


def test_argument_errors_without_gpu(lib):
    from kda_b200 import _lib
    assert lib.kda_recurrent_fwd(None, None) == -1
    assert lib.kda_chunk_fwd(None, None) == -1
    r = _lib.RecurrentArgs(N=1, T=4, tokens=4, H=2, K=48, V=64, io_dtype=0)
    r.q = r.k = r.v = r.g = r.beta = r.o = C.c_void_p(256)
    assert lib.kda_recurrent_fwd(C.byref(r), None) == -2          # K = 48 unsupported
    r.K = 64
    r.io_dtype = 7
    assert lib.kda_recurrent_fwd(C.byref(r), None) == -3          # dtype
    r.io_dtype = 0
    r.q = C.c_void_p(260)
    assert lib.kda_recurrent_fwd(C.byref(r), None) == -4          # alignment
    r.q = C.c_void_p(0)
    assert lib.kda_recurrent_fwd(C.byref(r), None) == -1          # NULL
    a = _lib.ChunkArgs(tokens=64, N=1, H=2, K=64, V=64, io_dtype=0)
    assert lib.kda_chunk_fwd(C.byref(a), None) == -2              # K, V must be 128
    a.K = a.V = 128
    assert lib.kda_chunk_fwd(C.byref(a), None) == -1              # NULL pointers
    a.q = a.k = a.v = a.g = a.beta = a.o = a.cu_seqlens = a.workspace = C.c_void_p(512)
    a.workspace_bytes = 16
    assert lib.kda_chunk_fwd(C.byref(a), None) == -5              # workspace too small


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from kda_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
