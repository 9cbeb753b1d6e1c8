"""The C-ABI library loads without a GPU and exports every symbol include/eps_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "eps_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(epsb_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_all_symbols():
    from eps_b200 import build
    from eps_b200._lib import SIGNATURES

    path = build.build()
    lib = ctypes.CDLL(path)
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/eps_b200.h but not exported"
    # the Python binding covers every compute entry point of the header
    assert set(SIGNATURES) == set(names) - {"epsb_last_error", "epsb_version"}
    lib.epsb_version.restype = ctypes.c_int
    assert lib.epsb_version() >= 1


def test_argument_validation_needs_no_gpu():
    """Shape errors are raised on the host before any CUDA call (reference: std::runtime_error)."""
    import pytest

    from eps_b200._lib import EpsError, call

    with pytest.raises(EpsError, match="not divisible by group_size"):
        call("epsb_quant_1x128", None, 4, 100, None, None, 0, None)
    with pytest.raises(EpsError, match="Invalid num_stages"):
        call("epsb_source_plans", None, None, 8, 2, 12, 2, 4, None, None, None, None, None, 0, None)
    with pytest.raises(EpsError, match="K: 100 is not divisible by 128"):
        call("epsb_grouped_gemm_fp8", 0, None, None, None, None, None, 4, 16, 128, 100, None, None, None, None, 0, None)


def test_missing_library_fails_loudly(monkeypatch):
    import pytest

    from eps_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libeps_b200.so")
    with pytest.raises(_lib.EpsError, match="no CPU or PyTorch fallback"):
        _lib.lib()
