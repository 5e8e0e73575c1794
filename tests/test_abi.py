"""CPU tier: the C-ABI library builds, loads and exports every symbol the header declares.
No compute call is made here (there is no GPU in this tier)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib_path():
    import dl4s_b200.build as b
    return b.build()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "dl4s_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dl4s_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path():
    syms = header_symbols()
    for must in ("dl4s_cuda_sdpa_forward", "dl4s_cuda_sdpa_decode", "dl4s_cuda_mha_forward", "dl4s_cuda_ffn_forward",
                 "dl4s_cuda_encoder_forward", "dl4s_cuda_layernorm", "dl4s_cuda_gemm", "dl4s_cuda_malloc"):
        assert must in syms


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    missing = [s for s in header_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in include/dl4s_cuda.h but not exported: {missing}"


def test_python_bindings_cover_the_header(lib_path):
    from dl4s_b200 import _lib
    assert sorted(_lib.EXPORTS) == header_symbols()
    _lib.load()
    assert _lib.load().dl4s_cuda_version() >= 100


def test_no_fallback_without_a_device(lib_path):
    """Without a GPU the library must refuse to initialise; with one it must be a B200-class device."""
    from dl4s_b200 import _lib
    lib = _lib.load()
    n = ctypes.c_int32(-1)
    st = lib.dl4s_cuda_device_count(ctypes.byref(n))
    if st != 0 or n.value == 0:
        assert lib.dl4s_cuda_init(None, 0) != 0
        assert lib.dl4s_cuda_last_error()
        # compute entry points fail as well instead of computing on the host
        assert lib.dl4s_cuda_vadd(None, None, None, 4) != 0


def test_product_does_not_import_the_oracle():
    """The oracle is test infrastructure: nothing in the package may import, load or call it."""
    pkg = os.path.join(ROOT, "dl4s_b200")
    pat = re.compile(r"^\s*(from|import)\s+oracle\b|libdl4s_ref|dl4s_ref_|oracle[./]oracle", re.M)
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".swift")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert not pat.search(text), f"{f} reaches into the oracle"


def test_injected_failures_travel_through_status_and_last_error(lib_path):
    """Host-side failure injection (dl4s_cuda_inject_failure): allocation, a host-to-device copy and communicator
    creation fail with the status a real failure would carry and a message on this thread's last error; the
    injection is consumed by the call it fails. Needs no device."""
    from dl4s_b200 import _lib
    lib = _lib.load()
    OOM, CUDA, NCCL = -2, -3, -7
    p = ctypes.c_void_p(123)
    assert lib.dl4s_cuda_inject_failure(1, 1) == 0
    assert lib.dl4s_cuda_malloc(1 << 20, ctypes.byref(p)) == OOM
    assert b"injected failure" in lib.dl4s_cuda_last_error() and not p.value
    # consumed: the next call fails for the ordinary reason here (no device) or succeeds (on a GPU box)
    st = lib.dl4s_cuda_malloc(16, ctypes.byref(p))
    assert st != OOM or b"injected" not in lib.dl4s_cuda_last_error()
    if st == 0:
        assert lib.dl4s_cuda_free(p) == 0
    buf = (ctypes.c_float * 4)()
    assert lib.dl4s_cuda_inject_failure(2, 2) == 0
    assert lib.dl4s_cuda_memcpy_h2d(ctypes.c_void_p(16), buf, 16) == CUDA
    assert lib.dl4s_cuda_memcpy_h2d_async(ctypes.c_void_p(16), buf, 16) == CUDA
    assert b"host-to-device" in lib.dl4s_cuda_last_error()
    assert lib.dl4s_cuda_inject_failure(3, 1) == 0
    ident = (ctypes.c_uint8 * 128)()
    assert lib.dl4s_cuda_comm_init(0, 2, ident) == NCCL
    assert b"communicator creation refused" in lib.dl4s_cuda_last_error()
    assert lib.dl4s_cuda_inject_failure(99, 1) != 0
    for kind in (1, 2, 3, 4):
        assert lib.dl4s_cuda_inject_failure(kind, 0) == 0
    raised = None
    try:
        lib.dl4s_cuda_inject_failure(1, 1)
        _lib.call("dl4s_cuda_malloc", 64, ctypes.byref(p))
    except _lib.DL4SCudaError as e:      # what the Python mirror (and the Swift glue's fatalError) surface
        raised = e
    assert raised is not None and raised.status == OOM and "injected failure" in str(raised)
