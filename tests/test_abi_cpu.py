"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and
fails loudly instead of falling back."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "plb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(plb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(plb):
    handle = C.CDLL(plb.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(handle, name), "%s is declared in include/plb200.h but not exported" % name
    assert set(names) == set(plb.SYMBOLS), "python binding table and header disagree"


def test_no_cpu_fallback(plb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    handle = plb.lib()
    out = C.c_void_p()
    rc = handle.plb_ctx_create(0, None, C.byref(out))
    assert rc == plb.E_CUDA and not out.value
    assert b"failed" in handle.plb_last_error()


def test_null_arguments_are_rejected(plb):
    handle = plb.lib()
    assert handle.plb_ctx_create(0, None, None) == plb.E_INVALID
    assert handle.plb_conv_prepare(None, None, None, None, 0, None, None) == plb.E_INVALID
    out = C.c_void_p()
    assert handle.plb_conv_prepare(None, None, None, None, 0, None, C.byref(out)) == plb.E_INVALID
    assert handle.plb_fc_prepare(None, 4, 4, 0, 0.0, 1.0, 1.0, 0, None, None, 1, None, C.byref(out)) == plb.E_INVALID
    assert handle.plb_conv_run(None, None, None, 1) == plb.E_INVALID
    assert handle.plb_sparse_run(None, None, None, 1) == plb.E_INVALID
    assert handle.plb_ctx_launch_count(None) == 0
