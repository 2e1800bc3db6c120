"""Parity of the pointwise THC entry points with the CPU oracle, through the C ABI.

Mirrors cutorch's own pointwise tests (test/test.lua:985-1237, 1735-1761): every op runs on the
CPU path and on an exact device clone of the same (possibly non-contiguous) tensors, and every
output is compared.  Bars: bit-exact for integer types and single-IEEE-op float ops, <= 2 ulp for
transcendentals (<= 1 half ulp for Half, whose math runs in float)."""
import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import OP
from common import (ALL_KINDS, FP_KINDS, INT_KINDS, LAYOUTS, NP_OF_KIND, assert_bit_equal, assert_ulp, make_view,
                    random_array, rng, to_device)

pytestmark = pytest.mark.gpu

# name -> (oracle op, domain lo, hi, exact)
UNARY_FP = {
    "log": ("LOG", 0.1, 4, False), "lgamma": ("LGAMMA", 0.1, 4, False), "log1p": ("LOG1P", -0.5, 4, False),
    "exp": ("EXP", -4, 4, False), "cos": ("COS", -4, 4, False), "sin": ("SIN", -4, 4, False),
    "sqrt": ("SQRT", 0, 4, True), "rsqrt": ("RSQRT", 0.1, 4, True), "ceil": ("CEIL", -4, 4, True),
    "floor": ("FLOOR", -4, 4, True), "trunc": ("TRUNC", -4, 4, True), "acos": ("ACOS", -1, 1, False),
    "cosh": ("COSH", -4, 4, False), "asin": ("ASIN", -1, 1, False), "sinh": ("SINH", -4, 4, False),
    "tan": ("TAN", -1.5, 1.5, False), "atan": ("ATAN", -4, 4, False), "tanh": ("TANH", -4, 4, False),
    "round": ("ROUND", -4, 4, True), "frac": ("FRAC", -4, 4, True), "cinv": ("CINV", 0.1, 4, True),
    "sigmoid": ("SIGMOID", -2, 2, False),
}


def as_real(kind, v):
    """The value a `real` argument of this tensor type actually carries (a half scalar is rounded
    to half before the call, exactly as cutorch's Lua layer converts it)."""
    if kind in INT_KINDS:
        return int(v)
    return float(NP_OF_KIND[kind].type(v))


# Double-precision CUDA math functions documented at up to 2 ulp (tanh) / 4 ulp (lgamma) from the
# true value, against a libm that is itself up to 1 ulp off: the distance between the two exceeds
# the 2-ulp bar for these two functions only.
ULP_EXCEPTIONS = {("Double", "lgamma"): 5, ("Double", "tanh"): 3}


def check(kind, got, want, exact, what, ulp=2):
    if NP_OF_KIND[kind].kind != "f" or exact:
        assert_bit_equal(got, want, what)
    else:
        assert_ulp(got, want, 1 if kind == "Half" else ulp, what)


@pytest.mark.parametrize("kind", FP_KINDS)
@pytest.mark.parametrize("name", sorted(UNARY_FP))
def test_unary_math(state, oracle, kind, name):
    op, lo, hi, exact = UNARY_FP[name]
    r = rng(kind, name)
    for shape, layout in [((10007,), "contiguous"), ((5, 7, 6), "transposed"), ((9, 33), "strided")]:
        x = make_view(r, kind, shape, layout)
        x[...] = r.uniform(lo, hi, size=shape).astype(x.dtype)
        want = oracle.pointwise(OP[op], np.zeros(shape, x.dtype), [x])
        dx = to_device(state, x)
        out = thc.Tensor.new(state, kind)
        out.call(name, out, dx)
        ulp = ULP_EXCEPTIONS.get((kind, name), 2)
        check(kind, out.numpy(), want, exact, f"{kind}.{name} {layout}", ulp)
        # in place
        dx.call(name, dx, dx)
        check(kind, dx.numpy(), want, exact, f"{kind}.{name} in place {layout}", ulp)


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("name,op", [("abs", "ABS"), ("sign", "SIGN"), ("neg", "NEG")])
def test_abs_sign_neg(state, oracle, kind, name, op):
    if name == "neg" and kind in ("Byte", "Char"):
        pytest.skip("neg is not declared for Byte/Char (lib/THC/generic/THCTensorMathPointwise.h:37-42)")
    r = rng(11)
    for layout in LAYOUTS:
        x = make_view(r, kind, (6, 5, 8), layout)
        want = oracle.pointwise(OP[op], np.zeros(x.shape, x.dtype), [x])
        out = thc.Tensor.new(state, kind)
        out.call(name, out, to_device(state, x))
        assert_bit_equal(out.numpy(), want, f"{kind}.{name} {layout}")


BINARY = {  # name -> (op, exact for float, needs nonzero divisor, int ok)
    "cmul": ("MUL", True, False), "cdiv": ("DIV", True, True), "cmax": ("CMAX", True, False),
    "cmin": ("CMIN", True, False), "cfmod": ("CFMOD", True, True), "cremainder": ("CREMAINDER", True, True),
    "cpow": ("CPOW", False, False),
}


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("name", sorted(BINARY))
def test_binary(state, oracle, kind, name):
    op, exact, nonzero = BINARY[name]
    r = rng(kind, name)
    for la, lb in [("contiguous", "contiguous"), ("transposed", "contiguous"), ("strided", "permuted"), ("holes", "offset")]:
        shape = (7, 6, 9)
        a = make_view(r, kind, shape, la)
        b = make_view(r, kind, shape, lb)
        if nonzero:
            b[b == 0] = 1
        if name == "cpow":
            a[...] = np.abs(a) % 5 + 1 if a.dtype.kind != "f" else np.abs(a) + 0.5
            b[...] = np.abs(b) % 3 if b.dtype.kind != "f" else b
        want = oracle.pointwise(OP[op], np.zeros(shape, a.dtype), [a, b])
        da, db = to_device(state, a), to_device(state, b)
        out = thc.Tensor.new(state, kind)
        out.call(name, out, da, db)
        check(kind, out.numpy(), want, exact, f"{kind}.{name} {la}/{lb}")
        da.call(name, da, da, db)  # in place: self == src1
        check(kind, da.numpy(), want, exact, f"{kind}.{name} in place {la}/{lb}")


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("value", [1, 2.5, -3])
def test_cadd_csub(state, oracle, kind, value):
    """cadd(self, src1, v, src2) = src1 + v*src2 without FMA contraction; v == 1 is a plain add;
    csub negates the scalar (lib/THC/generic/THCTensorMathPointwise.cu:264-342)."""
    if kind == "Byte" and value < 0:
        value = 3
    v = as_real(kind, value)
    r = rng(5)
    for la, lb, shape in [("contiguous", "contiguous", (20011,)), ("transposed", "strided", (8, 5, 12))]:
        a, b = make_view(r, kind, shape, la), make_view(r, kind, shape, lb)
        for name, sv in (("cadd", v), ("csub", -v)):
            if v == 1:
                want = oracle.pointwise(OP["ADD" if name == "cadd" else "SUB"], np.zeros(shape, a.dtype), [a, b])
            else:
                if kind == "Byte":
                    sv = sv & 0xFF
                want = oracle.pointwise(OP["CADD"], np.zeros(shape, a.dtype), [a, b], sv)
            out = thc.Tensor.new(state, kind)
            out.call(name, out, to_device(state, a), v, to_device(state, b))
            assert_bit_equal(out.numpy(), want, f"{kind}.{name}({v}) {la}/{lb}")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_scalar_ops(state, oracle, kind):
    r = rng(6)
    isint = kind in INT_KINDS
    cases = [("add", "ADD_S", 3), ("sub", "SUB_S", 2), ("mul", "MUL_S", 3), ("div", "DIV_S", 3),
             ("fmod", "FMOD_S", 3), ("remainder", "REMAINDER_S", 3), ("cmaxValue", "MAX_S", 1), ("cminValue", "MIN_S", 1)]
    if not isint:
        cases += [("add", "ADD_S", 0.3), ("mul", "MUL_S", -1.7), ("div", "DIV_S", 0.7), ("remainder", "REMAINDER_S", -1.3)]
    if kind != "Half":
        cases += [("lshift", "LSHIFT_S", 2), ("rshift", "RSHIFT_S", 1)]
    if isint:
        cases += [("bitand", "BITAND_S", 5), ("bitor", "BITOR_S", 9), ("bitxor", "BITXOR_S", 6)]
    for name, op, v in cases:
        v = as_real(kind, v)
        for layout in ("contiguous", "transposed", "strided"):
            x = make_view(r, kind, (6, 10, 7), layout)
            if name in ("lshift", "rshift") and isint:
                x[...] = np.abs(x) % 16
            want = oracle.pointwise(OP[op], np.zeros(x.shape, x.dtype), [x], v)
            out = thc.Tensor.new(state, kind)
            out.call(name, out, to_device(state, x), v)
            assert_bit_equal(out.numpy(), want, f"{kind}.{name}({v}) {layout}")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_clamp(state, oracle, kind):
    r = rng(7)
    x = make_view(r, kind, (9, 11), "transposed")
    lo, hi = (2, 17) if kind == "Byte" else (-7, 9)
    want = oracle.pointwise(OP["CLAMP"], np.zeros(x.shape, x.dtype), [x], lo, hi)
    out = thc.Tensor.new(state, kind)
    out.call("clamp", out, to_device(state, x), lo, hi)
    assert_bit_equal(out.numpy(), want, f"{kind}.clamp")


@pytest.mark.parametrize("kind", FP_KINDS)
def test_pow_family(state, oracle, kind):
    r = rng(8)
    x = make_view(r, kind, (12, 9), "strided")
    x[...] = r.uniform(0.2, 3, size=x.shape).astype(x.dtype)
    for v in (1, 2, 3, -1, -2, 0.5, 2.7):
        v = as_real(kind, v)
        want = oracle.pointwise(OP["POW"], np.zeros(x.shape, x.dtype), [x], v)
        out = thc.Tensor.new(state, kind)
        out.call("pow", out, to_device(state, x), v)
        check(kind, out.numpy(), want, v in (1, 2, 3, -1, -2), f"{kind}.pow({v})")
    want = oracle.pointwise(OP["TPOW"], np.zeros(x.shape, x.dtype), [x], 1.5)
    out = thc.Tensor.new(state, kind)
    out.call("tpow", out, 1.5, to_device(state, x))
    check(kind, out.numpy(), want, False, f"{kind}.tpow")
    y = make_view(r, kind, x.shape, "contiguous")
    want = oracle.pointwise(OP["ATAN2"], np.zeros(x.shape, x.dtype), [x, y])
    out = thc.Tensor.new(state, kind)
    out.call("atan2", out, to_device(state, x), to_device(state, y))
    check(kind, out.numpy(), want, False, f"{kind}.atan2")
    w = as_real(kind, 0.3)
    want = oracle.pointwise(OP["LERP"], np.zeros(x.shape, x.dtype), [x, y], w)
    out = thc.Tensor.new(state, kind)
    out.call("lerp", out, to_device(state, x), to_device(state, y), w)
    assert_bit_equal(out.numpy(), want, f"{kind}.lerp")


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("name,op", [("addcmul", "ADDCMUL"), ("addcdiv", "ADDCDIV")])
def test_addc(state, oracle, kind, name, op):
    """addcmul(self, t, v, s1, s2): self = t + v*s1*s2.  Out of place (self != t: cutorch copies t
    into self first) and in place (self == t) must agree with the oracle bit for bit."""
    r = rng(9)
    v = 2 if kind in INT_KINDS else 0.5
    shape = (4, 6, 5, 7)
    t = make_view(r, kind, shape, "contiguous")
    s1 = make_view(r, kind, shape, "permuted")
    s2 = make_view(r, kind, shape, "strided")
    if name == "addcdiv":
        s2[s2 == 0] = 1
    want = oracle.pointwise(OP[op], np.zeros(shape, t.dtype), [t, s1, s2], v)
    dt_, d1, d2 = to_device(state, t), to_device(state, s1), to_device(state, s2)
    out = thc.Tensor.new(state, kind)
    out.call(name, out, dt_, v, d1, d2)
    assert_bit_equal(out.numpy(), want, f"{kind}.{name} out of place")
    dt_.call(name, dt_, dt_, v, d1, d2)
    assert_bit_equal(dt_.numpy(), want, f"{kind}.{name} in place")
    # self aliases src1: the reference semantics (copy t into self first, then update in place)
    t2 = to_device(state, t)
    a1 = to_device(state, s1.copy())
    a1.call(name, a1, t2, v, a1, d2)
    want_alias = oracle.pointwise(OP[op], np.zeros(shape, t.dtype), [t, t, s2], v)
    assert_bit_equal(a1.numpy(), want_alias, f"{kind}.{name} self aliases src1")


@pytest.mark.parametrize("kind", INT_KINDS)
def test_bit_and_shift_ops(state, oracle, kind):
    r = rng(10)
    a = make_view(r, kind, (8, 9), "transposed")
    b = make_view(r, kind, (8, 9), "contiguous")
    for name, op in (("cbitand", "CBITAND"), ("cbitor", "CBITOR"), ("cbitxor", "CBITXOR")):
        want = oracle.pointwise(OP[op], np.zeros(a.shape, a.dtype), [a, b])
        out = thc.Tensor.new(state, kind)
        out.call(name, out, to_device(state, a), to_device(state, b))
        assert_bit_equal(out.numpy(), want, f"{kind}.{name}")
    a[...] = np.abs(a) % 16
    s = (np.abs(b) % 3).astype(b.dtype)
    for name, op in (("clshift", "CLSHIFT"), ("crshift", "CRSHIFT")):
        want = oracle.pointwise(OP[op], np.zeros(a.shape, a.dtype), [a, s])
        out = thc.Tensor.new(state, kind)
        out.call(name, out, to_device(state, a), to_device(state, s))
        assert_bit_equal(out.numpy(), want, f"{kind}.{name}")


def test_float_shift_ops(state, oracle):
    r = rng(12)
    for kind in ("Float", "Double"):
        a = make_view(r, kind, (8, 9), "contiguous")
        s = r.integers(-3, 4, size=(8, 9)).astype(a.dtype)
        for name, op in (("clshift", "CLSHIFT"), ("crshift", "CRSHIFT")):
            want = oracle.pointwise(OP[op], np.zeros(a.shape, a.dtype), [a, s])
            out = thc.Tensor.new(state, kind)
            out.call(name, out, to_device(state, a), to_device(state, s))
            assert_bit_equal(out.numpy(), want, f"{kind}.{name}")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_fill_zero_copy(state, oracle, kind):
    r = rng(13)
    for layout in LAYOUTS:
        x = make_view(r, kind, (5, 6, 7), layout)
        dx = to_device(state, x)
        dx.call("fill", dx, 3)
        assert_bit_equal(dx.numpy(), np.full(x.shape, 3, x.dtype), f"{kind}.fill {layout}")
        dx.call("zero", dx)
        assert_bit_equal(dx.numpy(), np.zeros(x.shape, x.dtype), f"{kind}.zero {layout}")
        src = make_view(r, kind, (5, 6, 7), "permuted")
        dx.call("copy", dx, to_device(state, src))
        assert_bit_equal(dx.numpy(), np.ascontiguousarray(src), f"{kind}.copy {layout}")


def test_copy_different_shapes_same_count(state):
    """Operands need equal element counts, not equal shapes; each is walked in its own logical
    order (lib/THC/THCApply.cuh:256-260)."""
    r = rng(14)
    a = make_view(r, "Float", (6, 4, 5), "transposed")
    da = to_device(state, a)
    out = thc.Tensor.new(state, "Float", 120)
    out.call("copy", out, da)
    assert_bit_equal(out.numpy(), np.ascontiguousarray(a).reshape(120), "copy 3-D transposed -> 1-D")
    b = make_view(r, "Float", (10, 12), "strided")
    db = to_device(state, b)
    res = thc.Tensor.new(state, "Float")
    res.call("cmul", res, da, db)
    want = (np.ascontiguousarray(a).reshape(-1) * np.ascontiguousarray(b).reshape(-1)).reshape(6, 4, 5)
    assert_bit_equal(res.numpy(), want, "cmul with differently shaped operands")


@pytest.mark.parametrize("src_kind", ALL_KINDS)
@pytest.mark.parametrize("dst_kind", ALL_KINDS)
def test_copy_convert(state, oracle, src_kind, dst_kind):
    r = rng(15)
    src = make_view(r, src_kind, (7, 9), "transposed")
    if NP_OF_KIND[src_kind].kind == "f" and NP_OF_KIND[dst_kind].kind != "f":
        src[...] = np.abs(src) if dst_kind == "Byte" else src  # negative float -> unsigned is undefined in C
    if dst_kind == "Byte" and NP_OF_KIND[src_kind].kind != "f":
        src[...] = np.abs(src) % 100
    want = oracle.convert(np.zeros((7, 9), NP_OF_KIND[dst_kind]), src)
    dst = thc.Tensor.new(state, dst_kind, 7, 9)
    dst.copy_from(to_device(state, src))
    assert_bit_equal(dst.numpy(), want, f"copy {src_kind} -> {dst_kind}")


def test_cross(state, oracle):
    r = rng(16)
    for kind in ("Float", "Double", "Int"):
        x = make_view(r, kind, (5, 3, 4), "contiguous")
        y = make_view(r, kind, (5, 3, 4), "permuted")
        xs, ys = np.ascontiguousarray(x), np.ascontiguousarray(y)
        want = np.zeros_like(xs)
        for i in range(3):
            j, k = (i + 1) % 3, (i + 2) % 3
            want[:, i, :] = xs[:, j, :] * ys[:, k, :] - xs[:, k, :] * ys[:, j, :]
        out = thc.Tensor.new(state, kind)
        out.call("cross", out, to_device(state, x), to_device(state, y), 1)
        assert_bit_equal(out.numpy(), want, f"{kind}.cross")


def test_equal(state):
    r = rng(17)
    a = make_view(r, "Float", (33, 65), "contiguous")
    da, db = to_device(state, a), to_device(state, a.copy())
    assert da.call("equal", da, db) == 1
    b = a.copy()
    b[20, 40] += 1
    assert da.call("equal", da, to_device(state, b)) == 0
    assert da.call("equal", da, to_device(state, a[:, :64].copy())) == 0


def test_overlapping_output_goes_through_a_temporary(state):
    """An expanded (stride-0) receiver has aliasing index tuples: cutorch computes into a
    contiguous copy and writes back (lib/THC/THCApply.cuh:288-302).  Every element of the
    result must be one of the values some logical index produced."""
    base = np.arange(4, dtype=np.float32)
    d = to_device(state, base.reshape(1, 4))
    t = thc.Tensor.wrap(state, "Float", d.data_ptr, (3, 4), (0, 1), storage_elems=4)
    t.call("add", t, t, 1.0)
    got = d.numpy().reshape(4)
    assert np.array_equal(got, base + 1)


def test_large_contiguous_matches_numpy(state):
    """Vector path sanity at a size with full tiles and a ragged tail, all eight types."""
    r = rng(18)
    for kind in ALL_KINDS:
        n = 1_000_003
        a = random_array(r, kind, (n,))
        b = random_array(r, kind, (n,))
        out = thc.Tensor.new(state, kind)
        out.call("cmul", out, to_device(state, a), to_device(state, b))
        if NP_OF_KIND[kind].kind == "f":
            want = (a.astype(np.float32) * b.astype(np.float32)).astype(a.dtype) if kind == "Half" else a * b
        else:
            want = (a.astype(np.int64) * b.astype(np.int64)).astype(a.dtype)
        assert_bit_equal(out.numpy(), want, f"{kind} cmul 1e6")


@pytest.mark.parametrize("kind", ["Byte", "Int", "Half", "Float", "Double"])
def test_rows_plan_expanded_and_padded_operands(state, oracle, kind):
    """Two collapsed dims with operands that are dense or constant along the inner one: per-row
    factors and bias rows seen through stride-0 (expanded) views, and rows with padding.  These
    take the `rows` kernel; results must equal the oracle's walk of the same strided views."""
    import ctypes as C
    lib = state.lib
    lib.thcb200_last_plan.restype = C.c_char_p
    r = rng("rows", kind)
    R, Cc = 301, 256
    x = make_view(r, kind, (R, Cc), "contiguous")
    per_row = np.broadcast_to(make_view(r, kind, (R, 1), "contiguous"), (R, Cc))     # strides (1, 0)
    per_col = np.broadcast_to(make_view(r, kind, (1, Cc), "contiguous"), (R, Cc))    # strides (0, 1)
    padded = random_array(r, kind, (R, Cc + 32))[:, :Cc]                             # row stride C + 32
    v = as_real(kind, 2)
    cases = [("cmul", "MUL", [x, per_row], ()), ("cadd", "CADD", [x, per_col], (v,)),
             ("addcmul", "ADDCMUL", [x, per_row, per_col], (v,)), ("cmul", "MUL", [padded, x], ()),
             ("cmax", "CMAX", [per_col, padded], ())]
    for name, op, ins, scal in cases:
        want = oracle.pointwise(OP[op], np.zeros((R, Cc), x.dtype), ins, *scal)
        dins = [to_device(state, a) for a in ins]
        out = thc.Tensor.new(state, kind)
        if name == "cadd":
            out.cadd(dins[0], v, dins[1])
        elif name == "addcmul":
            out.addcmul(dins[0], v, dins[1], dins[2])
        else:
            getattr(out, name)(dins[0], dins[1])
        assert lib.thcb200_last_plan().decode() == "rows", (name, lib.thcb200_last_plan().decode())
        check(kind, out.numpy(), want, True, f"{kind}.{name} rows plan")
        # into a padded output
        dout = to_device(state, random_array(r, kind, (R, Cc + 32))[:, :Cc])
        if name == "cadd":
            dout.cadd(dins[0], v, dins[1])
        elif name == "addcmul":
            dout.addcmul(dins[0], v, dins[1], dins[2])
        else:
            getattr(dout, name)(dins[0], dins[1])
        assert lib.thcb200_last_plan().decode() == "rows"
        check(kind, dout.numpy(), want, True, f"{kind}.{name} rows plan, padded output")


SPECIALS = [0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 2.0, 1e-3, -1e-3, 10.0, -10.0, 88.0, -88.0, 710.0, -710.0,
            float("inf"), float("-inf"), float("nan")]


@pytest.mark.parametrize("kind", FP_KINDS)
def test_unary_math_on_special_values(state, oracle, kind):
    """Zeros of both signs, infinities, NaN, the largest and smallest magnitudes of the type and
    its subnormals through every unary function: the results have to be the oracle's (NaN where
    it gives NaN, the same infinities and signed zeros), within the usual ulp bars elsewhere."""
    dt = NP_OF_KIND[kind]
    fi = np.finfo(dt)
    vals = SPECIALS + [float(fi.max), float(-fi.max), float(fi.tiny), float(-fi.tiny),
                       float(fi.smallest_subnormal), float(-fi.smallest_subnormal), float(fi.tiny) / 4]
    with np.errstate(over="ignore"):
        x = np.array(vals, dtype=np.float64).astype(dt)
    dx = to_device(state, x)
    for name, (op, _lo, _hi, exact) in sorted(UNARY_FP.items()):
        with np.errstate(all="ignore"):
            want = oracle.pointwise(OP[op], np.zeros(x.shape, dt), [x])
        out = thc.Tensor.new(state, kind)
        getattr(out, name)(dx)
        got = out.numpy()
        # same NaNs, same infinities, same zeros (with sign)
        assert np.array_equal(np.isnan(got), np.isnan(want)), f"{kind}.{name}: NaN pattern {got} vs {want}"
        fin = np.isfinite(want) & (want != 0)
        assert np.array_equal(got[~fin & ~np.isnan(want)].view(np.uint8), want[~fin & ~np.isnan(want)].view(np.uint8)), \
            f"{kind}.{name}: infinities / zeros differ: {got} vs {want}"
        ulp = ULP_EXCEPTIONS.get((kind, name), 2)
        if exact:
            assert_bit_equal(got[fin], want[fin], f"{kind}.{name} on special values")
        else:
            assert_ulp(got[fin], want[fin], 1 if kind == "Half" else ulp, f"{kind}.{name} on special values")
    for name in ("abs", "neg", "sign"):
        with np.errstate(all="ignore"):
            want = oracle.pointwise(OP[name.upper()], np.zeros(x.shape, dt), [x])
        out = thc.Tensor.new(state, kind)
        getattr(out, name)(dx)
        assert_bit_equal(out.numpy(), want, f"{kind}.{name} on special values")


def test_half_unary_math_over_every_bit_pattern(state, oracle):
    """A Half tensor has 65536 possible elements: every one of them through every unary function.
    Same NaNs, same infinities and zeros; finite results within one half ulp of the oracle's (which
    evaluates in double and rounds once); and, since the half evaluation runs in float, all but a
    sliver of them bit-equal."""
    x = np.arange(65536, dtype=np.uint16).view(np.float16)
    dx = to_device(state, x)
    for name, (op, _lo, _hi, exact) in sorted(UNARY_FP.items()):
        with np.errstate(all="ignore"):
            want = oracle.pointwise(OP[op], np.zeros(x.shape, np.float16), [x])
        out = thc.Tensor.new(state, "Half")
        getattr(out, name)(dx)
        got = out.numpy()
        assert np.array_equal(np.isnan(got), np.isnan(want)), f"Half.{name}: NaN pattern"
        rest = ~np.isnan(want)
        fin = np.isfinite(want) & (want != 0)
        edge = rest & ~fin
        assert np.array_equal(got[edge].view(np.uint16), want[edge].view(np.uint16)), f"Half.{name}: infinities / zeros"
        if exact:
            assert_bit_equal(got[fin], want[fin], f"Half.{name} over all inputs")
        else:
            assert_ulp(got[fin], want[fin], 1, f"Half.{name} over all inputs")
            differing = int((got[fin].view(np.uint16) != want[fin].view(np.uint16)).sum())
            assert differing <= 0.02 * fin.sum(), f"Half.{name}: {differing} of {int(fin.sum())} results off by one ulp"


def test_expand_gives_broadcast_views_that_take_the_rows_kernel(state, oracle):
    """tensor:expand (lib/THC/generic/THCTensor.c:297-330): size-1 dims and new leading dims repeat with
    stride 0; a per-row factor and a bias row expanded to the matrix go through cmul / cadd like full
    tensors (rows plan), and the geometry errors are TH's."""
    from cutorch_b200 import _lib
    lib = _lib.load_library()
    r = rng("expand")
    x = r.standard_normal((300, 256)).astype(np.float32)
    scale = r.standard_normal((300, 1)).astype(np.float32)
    bias = r.standard_normal((256,)).astype(np.float32)
    dx, ds, db = to_device(state, x), to_device(state, scale), to_device(state, bias)
    es, eb = ds.expand(300, 256), db.expand(300, 256)
    assert es.sizes == [300, 256] and es.strides == [1, 0]
    assert eb.sizes == [300, 256] and eb.strides == [0, 1]
    out = thc.Tensor.new(state, "Float")
    out.cmul(dx, es)
    assert lib.thcb200_last_plan() == b"rows"
    assert_bit_equal(out.numpy(), x * scale, "cmul with an expanded per-row factor")
    out.cadd(out, 1.0, eb)
    assert_bit_equal(out.numpy(), x * scale + bias, "cadd with an expanded bias row")
    assert db.expand(2, 3, 256).sizes == [2, 3, 256]
    assert ds.expand(-1, 4).sizes == [300, 4]
    with pytest.raises(thc.THCError, match="must match the existing size"):
        ds.expand(299, 256)
    with pytest.raises(thc.THCError, match="greater or equal"):
        ds.expand(300)
