"""The C-ABI library: loads, exports every symbol the header declares, and rejects bad
arguments before touching the device (none of these tests needs a GPU)."""
import ctypes
import os
import re

import pytest

from sparse_ads_baselines_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tbe_b200.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tbe_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from sparse_ads_baselines_b200 import build
        build.build()
    return _lib.lib()


def test_header_and_binding_agree(lib):
    declared = _declared_functions()
    assert len(declared) >= 15
    assert sorted(_lib.SIGNATURES) == declared


def test_every_declared_symbol_is_exported(lib):
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared_functions():
        assert hasattr(raw, name), "libtbe_b200.so does not export %s" % name


def test_abi_version_and_error_string(lib):
    assert lib.tbe_abi_version() >= 1
    assert isinstance(lib.tbe_last_error_string(), bytes)


def test_invalid_arguments_are_rejected_without_a_device(lib):
    rc = lib.tbe_forward(None, None, None, None, None, None, 1, 1, 4, _lib.TBE_F32, _lib.TBE_POOL_SUM, None)
    assert rc == -1 and b"null" in lib.tbe_last_error_string()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    # D not a multiple of 4 (the reference asserts D % 4 == 0, table_batched_embeddings_cuda.cu:273)
    rc = lib.tbe_forward(p, p, p, p, None, p, 1, 1, 6, _lib.TBE_F32, _lib.TBE_POOL_SUM, None)
    assert rc == -1 and b"multiple of 4" in lib.tbe_last_error_string()
    rc = lib.tbe_forward(p, p, p, p, None, p, 0, 1, 4, _lib.TBE_F32, _lib.TBE_POOL_SUM, None)
    assert rc == -1 and b"T must be" in lib.tbe_last_error_string()
    rc = lib.tbe_forward(p, p, p, p, p, p, 1, 1, 4, _lib.TBE_F32, _lib.TBE_POOL_MEAN, None)
    assert rc == -1 and b"per-sample" in lib.tbe_last_error_string()
    rc = lib.tbe_backward_sgd(p, 4, 4, p, p, p, p, 1, 1, 4, 1, 1, _lib.TBE_F32, 0, 0.1, 0, 0, None, 0, None)
    assert rc == -1 and b"workspace" in lib.tbe_last_error_string()
    assert lib.tbe_set_tuning(b"no_such_knob", 1) == -1
    assert lib.tbe_set_tuning(b"fwd_unroll", 0) == 0


def test_python_layer_has_no_cpu_path(lib):
    import torch
    from sparse_ads_baselines_b200 import table_batched_embeddings as tbe
    w = torch.zeros(8, 4)
    to = torch.zeros(1, dtype=torch.int32)
    idx = torch.zeros(2, dtype=torch.int32)
    off = torch.tensor([0, 2], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        tbe.forward(w, to, idx, off, None, 200, 1, False)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        tbe.backward_sgd(torch.zeros(1, 1, 4), w, to, idx, off, 0.1, 200, 1, False)
