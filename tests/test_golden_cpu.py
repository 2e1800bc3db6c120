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


def test_baseline_config_views_collapse_to_the_golden_views():
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


# ---- comparisons and masks: the numpy oracle against cutorch's own functors --------------------
COMPARE_MASKED = json.loads((GOLDEN / "compare_masked.json").read_text())


@pytest.mark.parametrize("dtname", sorted(COMPARE_MASKED))
def test_mixed_oracle_reproduces_reference_compare_and_mask_functors(dtname):
    """oracle/mixed_oracle.py (numpy) against vectors made by compiling THCTensorMathCompare.cuh,
    THCTensorMathCompareT.cuh and THCTensorMasked.cuh from the cutorch tree (make_golden.py)."""
    from oracle import mixed_oracle as mo
    dt = np.dtype(dtname)
    e = COMPARE_MASKED[dtname]
    arr = lambda key, t=dt: np.frombuffer(bytes.fromhex(e[key]), dtype=t).copy()
    a, b, mask, packed = arr("a"), arr("b"), arr("mask", np.uint8), arr("packed")
    for name in ("lt", "gt", "le", "ge", "eq", "ne"):
        assert_bit_equal(mo.compare(name, a, b), arr(name + "Tensor", np.uint8), f"{dtname} {name}Tensor")
        assert_bit_equal(mo.compare(name, a, e["scalar"]), arr(name + "Value", np.uint8), f"{dtname} {name}Value")
        assert_bit_equal(mo.compare(name, a, b).astype(dt), arr(name + "TensorT"), f"{dtname} {name}TensorT")
        assert_bit_equal(mo.compare(name, a, e["scalar"]).astype(dt), arr(name + "ValueT"), f"{dtname} {name}ValueT")
    assert_bit_equal(mo.masked_fill(a, mask, e["fill"]), arr("maskedFill"), f"{dtname} maskedFill")
    assert_bit_equal(mo.masked_copy(a, mask, packed), arr("maskedCopy"), f"{dtname} maskedCopy")
    assert_bit_equal(mo.masked_select(a, mask), arr("maskedSelect"), f"{dtname} maskedSelect")


# ---- the C prototypes of cutorch's generic headers against include/THC/THCTypeAPI.h ------------
def _strip_parameter_names(proto: str) -> str:
    """`void f(THCState*state,real value)` -> `void f(THCState*,real)`: the contract is the types and
    their order; parameter names are free."""
    import re
    head, _, rest = proto.partition(")(")            # THCTensor_(name) ( params )
    if not rest:
        return proto
    params, _, tail = rest.rpartition(")")
    out = []
    for p in params.split(","):
        # `struct THCudaLongTensor *` and `THCudaLongTensor *` name the same type (the typedefs carry the tags)
        toks = [t for t in re.findall(r"[A-Za-z_][A-Za-z_0-9]*|\*", p) if t != "struct"]
        if len(toks) >= 2 and toks[-1] != "*" and toks[-2] not in ("unsigned", "const"):
            toks = toks[:-1]
        out.append(" ".join(toks).replace(" *", "*").replace("* ", "*"))
    return head + ")(" + ",".join(out) + ")" + tail


def test_thc_type_api_declares_every_prototype_of_cutorchs_generic_headers():
    """include/THC/THCTypeAPI.h is expanded once per tensor type exactly like cutorch's generic headers,
    so the drop-in claim is that every prototype of those headers appears in it with the same return
    type, argument types and order.  The fixture was read from the cutorch tree by make_golden.py."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    ours_text = (GOLDEN.parent.parent / "include" / "THC" / "THCTypeAPI.h").read_text()
    ours = {_strip_parameter_names(p) for p in mg.prototypes_of(ours_text)}
    fixture = json.loads((GOLDEN / "thc_prototypes.json").read_text())
    # outside this library's scope: needs sort (median), thrust tabulate with TH's evaluation order (linspace ...),
    # and cutorch's internal helper for advanced indexing
    out_of_scope = ("median", "medianall", "linspace", "logspace", "range", "arange", "calculateAdvancedIndexingOffsets")
    missing = []
    total = 0
    for header, protos in fixture.items():
        for p in protos:
            if any(f"_({name})" in p for name in out_of_scope):
                continue
            total += 1
            if _strip_parameter_names(p) not in ours:
                missing.append(f"{header}: {p}")
    assert total > 150
    assert not missing, "prototypes of cutorch's generic headers that include/THC/THCTypeAPI.h lacks:\n" + "\n".join(missing)
