"""Seeded random cases against the oracle: shapes with size-1 and odd dims, every layout of
common.make_view on every operand, bases off the 16-byte grid, all element types.  The cases are
drawn from fixed seeds, so a failure names a reproducible case.  cutorch's own tests draw their
sizes at random per run (test/test.lua:13-30, minsize / maxsize); here the draw is pinned."""
import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import OP, PRE, RED
from common import ALL_KINDS, FP_KINDS, LAYOUTS, assert_bit_equal, assert_reduction_close, make_view, rng, to_device

pytestmark = pytest.mark.gpu


def random_shape(r, max_elems=60000):
    nd = int(r.integers(1, 5))
    while True:
        shape = tuple(int(r.choice([1, 2, 3, 5, 7, 8, 16, 31, 33, 64, 100, 257])) for _ in range(nd))
        if 0 < int(np.prod(shape)) <= max_elems:
            return shape


def long_shape(r):
    """One long dim (the reductions and scans split it over CTAs), the others short."""
    nd = int(r.integers(1, 4))
    shape = [int(r.choice([1, 2, 3, 5, 33])) for _ in range(nd)]
    shape[int(r.integers(0, nd))] = int(r.choice([1000, 4097, 20000, 70001]))
    return tuple(shape)


def shifted(state, view, shift):
    """The view on the device with its first element `shift` elements past where from_numpy would put it:
    the same strides inside a buffer that is `shift` elements longer."""
    if shift == 0:
        return to_device(state, view)
    item = view.dtype.itemsize
    strides = [s // item for s in view.strides]
    extent = 1 + sum((n - 1) * s for n, s in zip(view.shape, strides))
    flat = np.zeros(extent + shift, view.dtype)
    np.lib.stride_tricks.as_strided(flat[shift:], shape=view.shape, strides=view.strides)[...] = view
    base = to_device(state, flat)
    t = thc.Tensor.wrap(state, thc.KIND_OF_DTYPE[view.dtype], base.data_ptr + shift * item, view.shape, strides)
    t._owner = base
    return t


BINARY_OPS = [("cadd", "CADD", 2), ("cmul", "MUL", None), ("csub", "CADD", -3), ("cmax", "CMAX", None), ("cmin", "CMIN", None)]


@pytest.mark.parametrize("seed", range(24))
def test_pointwise_random_layouts(state, oracle, seed):
    r = rng("fuzz-pointwise", seed)
    for _ in range(12):
        kind = ALL_KINDS[int(r.integers(0, len(ALL_KINDS)))]
        shape = random_shape(r)
        la, lb, lo = (LAYOUTS[int(r.integers(0, len(LAYOUTS)))] for _ in range(3))
        a, b, o = make_view(r, kind, shape, la), make_view(r, kind, shape, lb), make_view(r, kind, shape, lo)
        name, opname, scalar = BINARY_OPS[int(r.integers(0, len(BINARY_OPS)))]
        sa, sb, so = (int(r.integers(0, 4)) for _ in range(3))
        da, db, do = shifted(state, a, sa), shifted(state, b, sb), shifted(state, o, so)
        if scalar is None:
            getattr(do, name)(da, db)
            want = oracle.pointwise(OP[opname], np.zeros(shape, a.dtype), [a, b])
        else:
            getattr(do, name)(da, abs(scalar), db)
            want = oracle.pointwise(OP[opname], np.zeros(shape, a.dtype), [a, b], scalar)
        assert_bit_equal(do.numpy(), want, f"seed {seed}: {kind} {name} {shape} {la}/{lb}->{lo} shifts {sa},{sb},{so}")
        # in place on a strided tensor
        da.add(da, 3)
        assert_bit_equal(da.numpy(), oracle.pointwise(OP["ADD_S"], np.zeros(shape, a.dtype), [a], 3), f"seed {seed}: {kind} add in place {shape} {la}")


@pytest.mark.parametrize("seed", range(24))
def test_reductions_random_layouts(state, oracle, seed):
    r = rng("fuzz-reduce", seed)
    for case in range(14):
        kind = ALL_KINDS[int(r.integers(0, len(ALL_KINDS)))]
        shape = random_shape(r, 200000) if case < 10 else long_shape(r)
        layout = LAYOUTS[int(r.integers(0, len(LAYOUTS)))]
        x = make_view(r, kind, shape, layout)
        if x.dtype.kind == "f":
            x[...] = (r.integers(-16, 17, size=shape) / 4).astype(x.dtype)       # exact sums, many ties
        if kind == "Half" and max(shape) > 4000:
            x[...] = (r.integers(-1, 2, size=shape) / 4).astype(x.dtype)         # running sums stay exact in half
        dim = int(r.integers(0, len(shape))) if case < 10 else int(np.argmax(shape)) if r.random() < 0.7 else int(r.integers(0, len(shape)))
        dx = shifted(state, x, int(r.integers(0, 4)))
        what = f"seed {seed}: {kind} {shape} {layout} dim {dim}"
        out = thc.Tensor.new(state, kind)
        out.sum(dx, dim, 1)
        assert_bit_equal(out.numpy(), oracle.reduce_dim(RED["SUM"], PRE["IDENTITY"], 0.0, x, dim), what + " sum")
        rop = "MAX" if r.random() < 0.5 else "MIN"
        v, i = thc.Tensor.new(state, kind), thc.Tensor.new(state, "Long")
        (v.max if rop == "MAX" else v.min)(i, dx, dim, 1)
        wv, wi = oracle.reduce_dim(RED[rop], PRE["IDENTITY"], 0.0, x, dim, with_index=True)
        assert_bit_equal(v.numpy(), wv, what + f" {rop} values")
        assert_bit_equal(i.numpy(), wi, what + f" {rop} positions")
        total = dx.sumall()
        want = oracle.reduce_all(RED["SUM"], PRE["IDENTITY"], 0.0, x)
        if x.dtype.kind == "f":
            assert float(total) == float(want), what + " sumall"       # multiples of 1/4: exact in every accumulate type
        else:
            assert int(total) == int(want), what + " sumall"
        sc = thc.Tensor.new(state, kind)
        sc.cumsum(dx, dim)
        assert_bit_equal(sc.numpy(), oracle.scan_dim(False, x, dim), what + " cumsum")


@pytest.mark.parametrize("seed", range(8))
def test_float_reductions_random_values(state, oracle, seed):
    """Unrestricted float values: sums within the stated tolerance (1e-5 float, 1e-3 half, 1e-12 double),
    max / min with NaNs sprinkled in, bit for bit."""
    r = rng("fuzz-float", seed)
    for _ in range(10):
        kind = FP_KINDS[int(r.integers(0, 3))]
        shape = random_shape(r, 200000)
        layout = LAYOUTS[int(r.integers(0, len(LAYOUTS)))]
        x = make_view(r, kind, shape, layout)
        if r.random() < 0.5 and x.size > 4:
            idx = tuple(int(r.integers(0, n)) for n in shape)
            x[idx] = np.nan
        dim = int(r.integers(0, len(shape)))
        dx = to_device(state, x)
        what = f"seed {seed}: {kind} {shape} {layout} dim {dim}"
        v, i = thc.Tensor.new(state, kind), thc.Tensor.new(state, "Long")
        v.max(i, dx, dim, 1)
        wv, wi = oracle.reduce_dim(RED["MAX"], PRE["IDENTITY"], 0.0, x, dim, with_index=True)
        assert_bit_equal(i.numpy(), wi, what + " max positions")
        assert_bit_equal(v.numpy(), wv, what + " max values")
        clean = np.nan_to_num(np.asarray(x))
        dc = to_device(state, clean)
        out = thc.Tensor.new(state, kind)
        out.sum(dc, dim, 1)
        rel = {"Half": 1e-3, "Float": 1e-5, "Double": 1e-12}[kind]
        assert_reduction_close(out.numpy(), oracle.reduce_dim(RED["SUM"], PRE["IDENTITY"], 0.0, clean, dim), rel,
                               np.abs(clean.astype(np.float64)).sum(axis=dim, keepdims=True), what + " sum")
