"""The C ABI without a GPU: the library builds, loads, and exports every symbol include/niti_b200.h declares."""
import ctypes
import os
import re

from tests.conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "niti_b200.h")).read()
    return sorted(set(re.findall(r"NITI_API\s+[\w\s\*]+?\b(niti_\w+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from niti_b200 import build
    lib = ctypes.CDLL(build.build())
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/niti_b200.h but not exported"


def test_ctypes_table_matches_header():
    from niti_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_error_strings_and_argument_checks_need_no_gpu():
    from niti_b200 import _lib
    L = _lib.lib
    assert L.niti_version() >= 100
    assert L.niti_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4):
        assert len(L.niti_strerror(code)) > 5
    # null pointers / bad sizes are rejected before any CUDA call
    assert L.niti_requant_i8(None, None, None, 16, 0, 7, 0, None, 0, 0, 0, None, None, None, None, None) == -1
    assert L.niti_conv_fprop_i8(None, None, None, None, None, 0, 1, 8, 8, 128, 128, 3, 3, 1, 1, None, None) == -1
    assert L.niti_conv_wgrad_scratch_bytes(0, 8, 8, 128, 128, 3, 3) == 0
    assert L.niti_conv_fprop_requant_supported(128, 128, 3, 3, 1) == 1
    assert L.niti_conv_fprop_requant_supported(100, 128, 3, 3, 1) == 0
