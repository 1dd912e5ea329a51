"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, and
refuses to work without a device (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

from gufo_npu_b200 import _capi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _capi.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "gufo_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gufo_cuda_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/gufo_cuda.h but not exported"
        assert name in _capi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_capi.SIGNATURES) == names


def test_null_arguments_are_rejected_without_a_device(lib):
    assert lib.gufo_cuda_ctx_create(0, None, None) == 1
    assert b"null" in lib.gufo_cuda_last_error(None)
    assert lib.gufo_cuda_ctx_synchronize(None) == 1
    assert lib.gufo_cuda_matmul(None, None, 0, None, 0, None) == 1
    assert lib.gufo_cuda_launch_count(None) == 0


def test_no_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    handle = C.c_void_p()
    status = lib.gufo_cuda_ctx_create(0, None, C.byref(handle))
    assert status == 4 and not handle.value
    assert b"no CUDA device" in lib.gufo_cuda_last_error(None)
    from gufo_npu_b200.backend import Context
    with pytest.raises(_capi.GufoCudaError):
        Context(0)
