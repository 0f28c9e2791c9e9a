"""The C-ABI library loads without a GPU and exports every entry point the headers declare."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for header in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        text = open(header).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(wrk_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    path = os.path.join(ROOT, "web-rwkv_b200", "libwrk.so")
    assert os.path.exists(path), "libwrk.so missing: run python web-rwkv_b200/build.py"
    lib = ctypes.CDLL(path)
    declared = _declared()
    assert len(declared) > 40
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_error_reporting_without_device():
    lib = ctypes.CDLL(os.path.join(ROOT, "web-rwkv_b200", "libwrk.so"))
    lib.wrk_last_error_message.restype = ctypes.c_char_p
    lib.wrk_build_arch.restype = ctypes.c_char_p
    assert lib.wrk_build_arch() == b"sm_100a"
    # null arguments are reported as values, never crash
    assert lib.wrk_context_create(0, None) == -103
    assert b"null" in lib.wrk_last_error_message()
    table = (ctypes.c_float * 16)()
    assert lib.wrk_nf4_table(table) == 0
    assert table[0] == -1.0 and table[15] == 1.0 and table[7] == 0.0
