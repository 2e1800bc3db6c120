"""CPU checks against fixtures made from cutorch's own code (tests/golden/make_golden.py):
the product's host-side layout functions and the CPU oracle both have to reproduce them."""
import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest

from cutorch_b200 import _lib
from cutorch_b200._lib import OP
from common import assert_bit_equal, assert_ulp

GOLDEN = Path(__file__).resolve().parent / "golden"
COLLAPSE = json.loads((GOLDEN / "collapse_dims.json").read_text())
FUNCTORS = json.loads((GOLDEN / "functors.json").read_text())

EXACT = {"SIGN", "ADD", "CADD", "SUB", "MUL", "DIV", "CREMAINDER", "CFMOD", "CLAMP", "LERP", "CMAX", "CMIN", "MAX_S",
         "MIN_S", "ADDCMUL", "ADDCDIV", "SQRT", "RSQRT", "CEIL", "FLOOR", "TRUNC", "ROUND", "FRAC", "CINV", "NEG", "ABS",
         "CLSHIFT", "CRSHIFT", "CBITAND", "CBITOR", "CBITXOR"}


def product_collapse(lib, sizes, strides, exclude):
    n = len(sizes)
    sz = (C.c_int64 * _lib.MAX_DIMS)(*sizes)
    st = (C.c_int64 * _lib.MAX_DIMS)(*strides)
    nd = C.c_int(n)
    ret = lib.thcb200_collapse_dims(sz, st, C.byref(nd), exclude)
    return list(sz[:nd.value]), list(st[:nd.value]), ret


def test_collapse_dims_matches_reference_fixtures():
    lib = _lib.load_library()
    for case in COLLAPSE:
        got = product_collapse(lib, case["sizes"], case["strides"], case["exclude"])
        assert got == (case["out_sizes"], case["out_strides"], case["ret"]), case


def test_index_to_offset_matches_reference_fixtures():
    lib = _lib.load_library()
    for case in COLLAPSE:
        d = _lib.make_desc(0, _lib.F32, case["sizes"], case["strides"])
        for linear, off in case["offsets"]:
            assert lib.thcb200_index_to_offset(C.byref(d), linear) == off, case
        # collapsing must not change where a logical index lands
        cs, ct, _ = product_collapse(lib, case["sizes"], case["strides"], -1)
        dc = _lib.make_desc(0, _lib.F32, cs, ct)
        for linear, off in case["offsets"]:
            assert lib.thcb200_index_to_offset(C.byref(dc), linear) == off, case


def test_baseline_config_views_collapse_as_surveyed():
    lib = _lib.load_library()
    assert product_collapse(lib, [64, 256, 56, 56], [802816, 3136, 56, 1], -1) == ([51380224], [1], -1)
    assert product_collapse(lib, [64, 256, 56, 56], [1605632, 6272, 112, 2], -1) == ([51380224], [2], -1)
    assert product_collapse(lib, [64, 256, 56, 56], [802816, 1, 256, 14336], -1)[0] == [64, 256, 56, 56]
    assert product_collapse(lib, [4, 1, 3, 5], [30, 15, 5, 1], 2) == ([4, 1, 3, 5], [30, 15, 5, 1], 2)


@pytest.mark.parametrize("key", sorted(FUNCTORS))
def test_oracle_reproduces_reference_functors(oracle, key):
    dtname, name = key.split(".")
    dt = np.dtype(dtname)
    vec = FUNCTORS[key]
    ins = [np.frombuffer(bytes.fromhex(h), dtype=dt).copy() for h in vec["inputs"]]
    want = np.frombuffer(bytes.fromhex(vec["out"]), dtype=dt)
    if name == "ADDCDIV" and dt.kind != "f":
        # TH divides after scaling ((v*a)/b), cutorch's functor before (v*(a/b)): the oracle follows
        # TH, so for integers the two differ by design.  Check TH's form instead.
        a, b, c = (x.astype(np.int64) for x in ins)
        q = np.trunc((vec["s0"] * b) / c).astype(np.int64)
        want = (a + q).astype(dt)
    got = oracle.pointwise(OP[name], np.zeros(len(want), dt), ins, vec["s0"], vec["s1"])
    if dt.kind != "f" or name in EXACT:
        assert_bit_equal(got, want, key)
    else:
        # the fixture holds the host libm result in the element type, the oracle the
        # double-precision value rounded once
        assert_ulp(got, want, 2, key)
