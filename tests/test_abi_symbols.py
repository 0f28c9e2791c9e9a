"""The C-ABI library loads without a GPU and exports every entry point the headers declare."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for header in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        with open(header) as f:
            text = f.read()
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


def test_sf4_table_matches_student_quantiles():
    # Float4Quant::new_student(5.0), src/tensor/matrix.rs:29-44 and 72-77: the library's own quantile (incomplete beta
    # function + bisection) against scipy's, which the oracle uses; no device is touched.
    import numpy as np
    from oracle import oracle
    lib = ctypes.CDLL(os.path.join(ROOT, "web-rwkv_b200", "libwrk.so"))
    for nu in (1.0, 2.5, 5.0, 30.0):
        table = (ctypes.c_float * 16)()
        assert lib.wrk_sf4_table(ctypes.c_double(nu), table) == 0
        got = np.array(list(table), dtype=np.float32)
        assert np.array_equal(got, oracle.sf4_table(nu)), nu
        assert got[0] == -1.0 and got[7] == 0.0 and got[15] == 1.0 and (np.diff(got) > 0).all()
    assert lib.wrk_sf4_table(ctypes.c_double(0.0), table) != 0
    assert lib.wrk_sf4_table(ctypes.c_double(5.0), None) != 0
