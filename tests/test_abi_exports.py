"""The C-ABI library loads on a machine without a GPU and exports every symbol that
``include/jabas_b200.h`` declares.  No compute call is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "jabas_b200.h")).read()
    return sorted(set(re.findall(r"JABAS_API\s+[\w\s\*]+?\b(jabas_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    from jabas_b200 import _lib
    assert _declared_symbols() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol():
    from jabas_b200 import _lib
    from jabas_b200.build import build_library
    build_library()
    lib = _lib.load()
    for name in _declared_symbols():
        assert getattr(lib, name) is not None
    assert lib.jabas_version() == 1


def test_struct_sizes_match_header():
    from jabas_b200 import _lib
    assert ctypes.sizeof(_lib.Seg) == 24
    assert ctypes.sizeof(_lib.Group) == 32
    assert ctypes.sizeof(_lib.SgdHp) == 48
    assert ctypes.sizeof(_lib.AdamHp) == 56


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from jabas_b200 import ops, JabasError
    with pytest.raises(JabasError):
        ops.Context()
    lib = __import__("jabas_b200")._lib.load()
    h = ctypes.c_void_p()
    assert lib.jabas_ctx_create(0, ctypes.byref(h)) < 0
    assert lib.jabas_last_error()
