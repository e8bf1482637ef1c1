"""CPU-side checks of the C-ABI library: it builds for sm_100a, loads, exports every symbol the
header declares, and fails loudly (no fallback) when there is no device."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_are_exported():
    from weightstream_b200 import _lib
    L = _lib.load()
    hdr = open(os.path.join(ROOT, "include", "ws_tp.h")).read()
    declared = set(re.findall(r"\b(ws_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in ws_tp.h but not exported"
    assert b"sm_100a" in L.ws_version()


def test_no_device_is_an_error_not_a_fallback():
    import ctypes as C
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from weightstream_b200 import _lib
    L = _lib.load()
    cfg = _lib.TpConfig(max_m=1, max_n=256)
    h = C.c_void_p()
    st = L.ws_tp_create(1, 0, 0, C.byref(cfg), C.byref(h))
    assert st == _lib.WS_ERR_CUDA and not h.value
    # argument validation happens before any device work
    assert L.ws_tp_create(3, 0, 0, C.byref(cfg), C.byref(h)) == _lib.WS_ERR_INVALID
    assert L.ws_tp_create(2, 2, 0, C.byref(cfg), C.byref(h)) == _lib.WS_ERR_INVALID


def test_product_code_never_touches_the_oracle():
    """The oracle is a checker: nothing in the package may import, load or link it."""
    pkg = os.path.join(ROOT, "weightstream_b200")
    pat = re.compile(r"(import\s+oracle|from\s+oracle|from\s+\.\.?oracle|libws_oracle|ws_oracle\.h|wso_)")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not pat.search(src), f"{f} reaches into oracle/"
