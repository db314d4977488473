"""CPU-side checks of the boundary: the shared library loads without a GPU and exports every
symbol include/frame_b200.h declares; the ctypes table covers them all."""
import os
import re

from frame_public_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "frame_b200.h")).read()
    return sorted(set(re.findall(r"FB200_API[^;(]*?\b(fb200_\w+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = capi.load()
    names = declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/frame_b200.h but not exported"


def test_ctypes_table_covers_the_header():
    assert sorted(capi.SIGNATURES) == declared_symbols()


def test_no_compute_without_a_gpu_is_an_error_not_a_fallback():
    lib = capi.load()
    assert lib.fb200_version().startswith(b"frame_b200")
    if capi.device_count() == 0:
        p = capi.c_void_p()
        rc = lib.fb200_malloc(0, 64, 64, capi.byref(p))
        assert rc != 0 and lib.fb200_last_error() != b""
