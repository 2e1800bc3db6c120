"""cumsum / cumprod through the THC C API against the sequential oracle (oracle_scan_dim).

cutorch's own tests: test/test.lua:1456-1478 (cumsum, cumprod on every dim of random 2-D/3-D
tensors).  Bars: integer types bit-exact (wrap-around arithmetic is associative); floating types
within the reduction tolerance of the running sum (1e-5 fp32, 1e-3 fp16, 1e-12 fp64), measured
against the sum of absolute values up to that position."""
import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import load_library
from common import ALL_KINDS, INT_KINDS, NP_OF_KIND, assert_bit_equal, make_view, rng, to_device

pytestmark = pytest.mark.gpu

REL = {"Half": 1e-3, "Float": 1e-5, "Double": 1e-12}


def check_scan(kind, got, want, src, dim, prod, what):
    if kind in INT_KINDS:
        assert_bit_equal(got, want, what)
        return
    g, w = got.astype(np.float64), want.astype(np.float64)
    a = np.abs(src.astype(np.float64))
    with np.errstate(over="ignore"):
        scale = np.cumprod(np.maximum(a, 1.0), axis=dim) if prod else np.cumsum(a, axis=dim)
    # one output rounding of the element type on top of the accumulation tolerance
    eps = float(np.finfo(NP_OF_KIND[kind]).eps)
    tol = (REL[kind] + eps) * np.maximum(np.abs(w), scale * 1e-3) + eps * np.abs(w)
    bad = ~(np.abs(g - w) <= tol) & ~(np.isnan(g) & np.isnan(w)) & ~(g == w)
    if bad.any():
        k = tuple(np.argwhere(bad)[0])
        raise AssertionError(f"{what}: {bad.sum()} outputs off; first at {k}: got {got[k]!r}, want {want[k]!r}")


CASES = [
    # shape, dim, layout
    ((3000,), 0, "contiguous"),          # 1-D: row walk, one row
    ((300000,), 0, "contiguous"),        # 1-D, chunked over many warps
    ((37, 1000), 1, "contiguous"),       # rows
    ((37, 1001), 1, "contiguous"),       # odd length: no vector path
    ((37, 1000), 1, "holes"),            # padded rows
    ((500, 40), 0, "contiguous"),        # columns, short inner run
    ((3000, 64), 0, "contiguous"),       # columns, chunked
    ((6, 50, 9, 8), 1, "contiguous"),    # inner run of 72 over two dims
    ((6, 50, 9, 8), 1, "offset"),        # same, rows not adjacent
    ((20, 30), 1, "transposed"),         # scanned dim strided, no inner run: thread per slice
    ((7, 9, 11), 1, "permuted"),
    ((5, 4), 0, "strided"),
    ((1, 1), 0, "contiguous"),
    ((4, 1, 5), 1, "contiguous"),        # scanning a dim of size 1 is a copy
]


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("prod", [False, True], ids=["cumsum", "cumprod"])
def test_scan(state, oracle, kind, prod):
    r = rng("scan", kind, prod)
    name = "cumprod" if prod else "cumsum"
    for shape, dim, layout in CASES:
        x = make_view(r, kind, shape, layout)
        if kind in INT_KINDS:
            x[...] = r.integers(0 if kind == "Byte" else -3, 4, size=shape).astype(x.dtype)
        elif prod:
            x[...] = r.uniform(0.9, 1.1, size=shape).astype(x.dtype) * r.choice([-1, 1], size=shape).astype(x.dtype)
        else:
            x[...] = r.uniform(-1, 1, size=shape).astype(x.dtype)
        want = oracle.scan_dim(prod, x, dim)
        dx = to_device(state, x)
        out = thc.Tensor.new(state, kind)
        getattr(out, name)(dx, dim)
        assert out.sizes == list(shape)
        check_scan(kind, out.numpy(), want, x, dim, prod, f"{kind} {name} {shape} dim {dim} {layout}")
        # into an existing non-contiguous output of the right shape, and in place
        out2 = to_device(state, make_view(r, kind, shape, "offset"))
        getattr(out2, name)(dx, dim)
        check_scan(kind, out2.numpy(), want, x, dim, prod, f"{kind} {name} strided output {shape} dim {dim}")
        getattr(dx, name)(dx, dim)
        check_scan(kind, dx.numpy(), want, x, dim, prod, f"{kind} {name} in place {shape} dim {dim}")


def test_scan_exact_values_and_plans(state, oracle):
    """Multiples of 1/8 below 2^21: every partial sum is exact in fp32, so any order gives the
    same bits; also checks which walk each layout gets."""
    lib = load_library()
    lib.thcb200_last_plan.restype = __import__("ctypes").c_char_p
    r = rng("scan-exact")
    for shape, dim, plan in [((8192, 1024), 1, "scan_row_vec"), ((4, 1 << 20), 1, "scan_row_vec_chunked"),
                             ((4096, 2048), 0, "scan_col_vec_chunked"), ((64, 64, 256), 1, "scan_col_vec"),
                             ((300, 7), 0, "scan_strided")]:
        x = (r.integers(-1000, 1001, size=shape) / 8).astype(np.float32)
        dx = to_device(state, x)
        out = thc.Tensor.new(state, "Float")
        out.cumsum(dx, dim)
        assert lib.thcb200_last_plan().decode() == plan, (shape, dim, lib.thcb200_last_plan().decode())
        assert_bit_equal(out.numpy(), oracle.scan_dim(False, x, dim), f"exact cumsum {shape} dim {dim}")


@pytest.mark.parametrize("kind", ["Float", "Int", "Half", "Double", "Byte"])
def test_scan_long_rows_one_pass(state, oracle, kind):
    """Rows of millions of elements (thousands of chunks per row), ragged ends, more than one row."""
    r = rng("scan-long", kind)
    per_tile = 256 * 4 * (16 // NP_OF_KIND[kind].itemsize)
    for rows, tiles, extra in [(1, 1030, 8 * 3), (3, 2100, 16 * 5), (2, 33, 0)]:
        K = tiles * per_tile + extra
        x = make_view(r, kind, (rows, K), "contiguous")
        if kind in INT_KINDS:
            x[...] = r.integers(0, 3, size=x.shape).astype(x.dtype)
        elif kind == "Half":
            x[...] = (r.integers(-2, 3, size=x.shape) / 4).astype(x.dtype)   # running sums stay exact in float
        else:
            x[...] = (r.integers(-1000, 1001, size=x.shape) / 8).astype(x.dtype)
        dx = to_device(state, x)
        out = thc.Tensor.new(state, kind)
        out.cumsum(dx, 1)
        want = oracle.scan_dim(False, x, 1)
        if kind == "Half":
            check_scan(kind, out.numpy(), want, x, 1, False, f"{kind} long rows {rows}x{K}")
        else:
            assert_bit_equal(out.numpy(), want, f"{kind} long rows {rows}x{K}")
        dx.cumsum(dx, 1)
        assert_bit_equal(dx.numpy(), out.numpy(), f"{kind} long rows in place")


def test_scan_repeatable_and_errors(state):
    r = rng("scan-rep")
    x = r.standard_normal((8, 1 << 18)).astype(np.float32)
    dx = to_device(state, x)
    a, b = thc.Tensor.new(state, "Float"), thc.Tensor.new(state, "Float")
    a.cumsum(dx, 1)
    b.cumsum(dx, 1)
    assert_bit_equal(a.numpy(), b.numpy(), "two runs")
    with pytest.raises(thc.THCError, match="out of range"):
        a.cumsum(dx, 2)
