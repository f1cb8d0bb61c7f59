"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/vlb.h declares; the ctypes table covers exactly the same set.  No compute call
is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vlb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vlb_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from matconvnet_b200 import build, capi
    build.build()
    return ctypes.CDLL(capi.LIB_PATH)


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), "libvlb.so does not export %s" % n


def test_ctypes_table_matches_header():
    from matconvnet_b200 import capi
    assert sorted(capi.SIGNATURES) == declared_symbols()


def test_error_messages(lib):
    lib.vlb_error_message.restype = ctypes.c_char_p
    assert lib.vlb_error_message(0) == b"success"
    assert lib.vlb_error_message(7) == b"illegal argument"
    assert lib.vlb_error_message(9) == b"timeout"
    assert lib.vlb_error_message(99) == b"unknown error"
    assert lib.vlb_version() >= 100


def test_output_shape_helpers(lib):
    from matconvnet_b200 import capi
    d = capi.ConvDesc(224, 224, 3, 64, 3, 3, 3, 64, 1, 1, 1, 1, 1, 1, 1, 1)
    ho, wo = ctypes.c_int(), ctypes.c_int()
    assert lib.vlb_conv_output_shape(ctypes.byref(d), ctypes.byref(ho), ctypes.byref(wo)) == 0
    assert (ho.value, wo.value) == (224, 224)
    d = capi.ConvDesc(11, 10, 3, 2, 3, 2, 3, 5, 2, 3, 1, 2, 0, 1, 1, 1)
    lib.vlb_conv_output_shape(ctypes.byref(d), ctypes.byref(ho), ctypes.byref(wo))
    assert (ho.value, wo.value) == ((11 + 3 - 3) // 2 + 1, (10 + 1 - 2) // 3 + 1)
    p = capi.PoolDesc(32, 32, 32, 100, 3, 3, 2, 2, 0, 1, 0, 1, 0)
    lib.vlb_pool_output_shape(ctypes.byref(p), ctypes.byref(ho), ctypes.byref(wo))
    assert (ho.value, wo.value) == (16, 16)


def test_no_context_without_gpu(lib):
    """Without a CUDA device the context cannot be created: there is nothing to fall back to."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    lib.vlb_ctx_create.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    assert lib.vlb_ctx_create(ctypes.byref(h)) != 0
