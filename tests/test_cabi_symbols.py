"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "parpy_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^[A-Za-z_][A-Za-z0-9_ \*]*?\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", text, flags=re.M)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("parpy_init", "parpy_sync", "parpy_alloc_buffer", "parpy_memcpy", "parpy_memset",
                     "parpy_free_buffer", "parpy_get_error_message", "forward_kernel",
                     "parpy_b200_forward"):
        assert required in names


def test_library_exports_every_declared_symbol(native):
    handle = ctypes.CDLL(native.LIB_PATH)
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} declared in include/parpy_b200.h but not exported"


def test_python_binding_covers_every_declared_symbol(native):
    assert sorted(native.SIGNATURES) == declared_functions()


def test_error_message_getter_works_without_gpu(native):
    msg = native.lib().parpy_get_error_message()
    assert isinstance(msg, bytes) and len(msg) > 0
