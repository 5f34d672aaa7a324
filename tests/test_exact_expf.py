"""The library's restated expf (lumen_b200/csrc/exact_expf.h, compiled here for
the host) must equal the C library's expf on EVERY float bit pattern: the router
selects experts by comparing softmax probabilities, so the last bit matters."""
import ctypes
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def chk(tmp_path_factory):
    out = tmp_path_factory.mktemp("expf") / "expfchk.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-pthread", "-o", str(out),
                    str(ROOT / "tests" / "native" / "exact_expf_check.cpp")], check=True)
    l = ctypes.CDLL(str(out))
    l.lumen_expf_count_mismatches.restype = ctypes.c_uint64
    l.lumen_expf_count_mismatches.argtypes = [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int,
                                              ctypes.POINTER(ctypes.c_uint32)]
    return l


@pytest.mark.parametrize("lo,hi", [(0x80000000, 0xFF800001), (0x00000000, 0x7F800001)])
def test_expf_matches_libm_exhaustively(chk, lo, hi):
    bad = ctypes.c_uint32(0)
    n = chk.lumen_expf_count_mismatches(lo, hi, max(2, os.cpu_count() or 2), ctypes.byref(bad))
    assert n == 0, f"{n} mismatches, first at bits {bad.value:#010x}"
