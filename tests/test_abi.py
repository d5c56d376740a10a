"""The C-ABI library: it loads, exports every symbol that include/brute_b200.h
declares, and rejects bad arguments with status codes before touching a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib(lib_built):
    from brute_b200 import _lib as L
    return L.load()


def declared_symbols():
    text = (ROOT / "include" / "brute_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(brute_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 19
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/brute_b200.h but not exported"


def test_python_signature_table_matches_header(lib):
    from brute_b200 import _lib as L
    assert sorted(L.SIGNATURES) == declared_symbols()


def test_strerror_and_caps(lib):
    from brute_b200 import _lib as L
    assert L.strerror(0) == "ok"
    for code in range(-7, 0):
        assert L.strerror(code) != "unknown error"
    assert L.strerror(-99) == "unknown error"
    caps = lib.brute_b200_query_caps()
    assert caps & 1 and caps & 8 and caps & 16


def test_argument_validation_needs_no_gpu(lib):
    # negative sizes, bad enums and misaligned pointers are refused before any CUDA call
    buf = (ctypes.c_uint64 * 8)()
    p = ctypes.addressof(buf)
    assert lib.brute_b200_pack_bool(p, p, -1, 8, None) == -1
    assert lib.brute_b200_pack_bool(None, None, 0, 8, None) == 0          # empty: nothing to do
    assert lib.brute_b200_pack_bool(p, p + 4, 1, 8, None) == -2
    assert lib.brute_b200_pack_sign(p, 9, p, 1, 8, 0, None) == -3
    assert lib.brute_b200_pack_sign(p, 0, p, 1, 8, 5, None) == -1
    assert lib.brute_b200_popcount_elems(p, p, 4, 3, None) == -3
    assert lib.brute_b200_bitwise(17, p, p, p, 1, 1, 64, None) == -1
    assert lib.brute_b200_xnor_gemm(p, p, p, 1, 1, 1, 65, 1, 0, None) == -1     # K > 64*Kp
    assert lib.brute_b200_xnor_gemm(p, p, p, 0, 4, 1, 64, 4, 0, None) == 0      # M == 0
    assert lib.brute_b200_xnor_gemm(p, p, p, 1, 1, 1, 64, 1, 9, None) == -1     # bad impl
    assert lib.brute_b200_binary_attention_fwd(p, p, p, p, 1, 1, 4, 96, 1, 0.1, None) == -3


def test_product_does_not_import_the_oracle():
    # the package must not route through the CPU oracle in any way
    for path in (ROOT / "brute_b200").rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in text.replace("the oracle", ""), f"{path} mentions the oracle"
    for path in (ROOT / "brute_b200" / "csrc").glob("*"):
        assert "oracle" not in path.read_text()
