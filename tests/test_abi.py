"""The C-ABI library loads and exports every symbol include/ns_b200.h declares (no compute calls, no GPU)."""
import ctypes
import os
import re

from nn_b200 import native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ns_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"NS_API\s+(?:const\s+)?\w+\*?\s+(ns_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    names = _declared()
    assert len(names) > 40
    lib = ctypes.CDLL(N.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in ns_b200.h but not exported: {missing}"


def test_binding_covers_the_header():
    assert set(_declared()) == set(N.exported_names())


def test_error_convention_without_a_device():
    lib = N.load()
    assert lib.ns_version() >= 100
    assert lib.ns_error_name(0) == b"NS_OK" and lib.ns_error_name(2) == b"NS_ERR_ARGUMENT"
    # a null out-pointer is an argument error with a message, not a crash
    rc = lib.ns_device_count(None)
    assert rc == 2 and b"null" in lib.ns_last_error()
