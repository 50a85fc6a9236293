"""The C-ABI library on a machine without a GPU: it loads, exports every declared symbol, and
refuses to create a device instead of crashing.  No compute call is made here."""
import ctypes as C
import os
import re

import pytest

from ferrum_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from ferrum_b200 import build
        build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ferrum_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fq_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    names = declared_symbols()
    assert len(names) >= 30
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_status_names(lib):
    assert lib.fq_status_name(0) == b"ok"
    assert lib.fq_status_name(_lib.ERR_SHAPE) == b"shape"
    assert lib.fq_status_name(_lib.ERR_ALIAS) == b"alias"
    assert lib.fq_status_name(99) == b"unknown"


def test_device_create_without_a_gpu_reports_an_error(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.fq_device_create(0, C.byref(h))
    assert rc == _lib.ERR_DEVICE and not h.value
    assert lib.fq_last_error(None) == b"null device handle"
    assert lib.fq_synchronize(None) == _lib.ERR_PARAM


def test_surface_has_no_cpu_fallback():
    """The product path must not import the oracle or compute with torch/numpy."""
    for name in ("surface.py", "_lib.py", "__init__.py"):
        src = open(os.path.join(ROOT, "ferrum_b200", name)).read()
        assert "oracle" not in src.replace("no CPU or PyTorch fallback", ""), name
        assert "torch.matmul" not in src and "@ " not in src and "np.dot" not in src
