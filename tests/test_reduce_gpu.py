"""Parity of the THC reduction entry points with the CPU oracle, through the C ABI.

Follows cutorch's reduction tests (test/test.lua:1347-1391 max/min, 1474-1487 sum, 2183-2207 norm)
but also pins what they leave open: ties (first occurrence wins), NaNs, every element type, all
kernel families (row / column / strided, split and unsplit) and non-contiguous inputs.
Bars: bit-exact for integer types and for max/min values and positions; floating sums within
rel 1e-5 (Float), 1e-12 (Double), 1e-3 (Half)."""
import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import PRE, RED, load_library
from common import (ALL_KINDS, FP_KINDS, INT_KINDS, NP_OF_KIND, assert_bit_equal, assert_reduction_close, make_view,
                    random_array, rng, to_device)

pytestmark = pytest.mark.gpu

REL = {"Half": 1e-3, "Float": 1e-5, "Double": 1e-12}

# (shape, dim, layout): chosen to reach every kernel family of the reduce planner
SHAPES = [
    ((37, 300), 1, "contiguous"),      # row, warp per row
    ((5, 70000), 1, "contiguous"),     # row, block per row with a split
    ((300, 40), 0, "contiguous"),      # column tiles
    ((3000, 96), 0, "contiguous"),     # column tiles with a K split
    ((6, 50, 64), 1, "contiguous"),    # column tiles with outer slices
    ((9, 7, 5), 1, "contiguous"),      # strided fallback (short inner run)
    ((40, 33), 1, "transposed"),       # reduced dim strided, other dim unit stride
    ((12, 20, 11), 2, "strided"),      # inner stride 2
    ((8, 9, 10), 0, "permuted"),
    ((1, 17), 1, "contiguous"),
    ((17, 1), 1, "contiguous"),
]


def plan_name():
    return load_library().thcb200_last_plan().decode()


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("case", range(len(SHAPES)))
def test_sum_prod_dim(state, oracle, kind, case):
    shape, dim, layout = SHAPES[case]
    r = rng("sum", kind, case)
    x = make_view(r, kind, shape, layout)
    dx = to_device(state, x)
    for name, rop in (("sum", "SUM"), ("prod", "PROD")):
        xx = x
        if name == "prod":
            xx = x.copy()
            xx[...] = (r.integers(0, 2, size=shape) * 2 - 1).astype(x.dtype) if kind != "Byte" else 1
            dx = to_device(state, xx)
        want = oracle.reduce_dim(RED[rop], PRE["IDENTITY"], 0, xx, dim)
        out = thc.Tensor.new(state, kind)
        out.call(name, out, dx, dim, 1)
        got = out.numpy()
        if kind in INT_KINDS:
            assert_bit_equal(got, want, f"{kind}.{name} {shape} dim {dim} [{plan_name()}]")
        else:
            abs_sum = np.abs(xx.astype(np.float64)).sum(axis=dim, keepdims=True)
            assert_reduction_close(got, want, REL[kind], abs_sum, f"{kind}.{name} {shape} dim {dim} [{plan_name()}]")
        # keepdim = 0 squeezes the reduced dim
        out2 = thc.Tensor.new(state, kind)
        out2.call(name, out2, dx, dim, 0)
        exp_shape = [n for k, n in enumerate(shape) if k != dim] or [1]
        if len(shape) == 1:
            exp_shape = [1]
        assert out2.sizes == exp_shape


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("case", range(len(SHAPES)))
def test_max_min_dim_with_ties(state, oracle, kind, case):
    """Values from a small set so that ties are everywhere: the position must be the first
    occurrence (1-based), as TH's CPU scan returns it."""
    shape, dim, layout = SHAPES[case]
    r = rng("maxmin", kind, case)
    x = make_view(r, kind, shape, layout)
    x[...] = r.integers(0, 5, size=shape).astype(x.dtype)
    dx = to_device(state, x)
    for name, rop in (("max", "MAX"), ("min", "MIN")):
        want_v, want_i = oracle.reduce_dim(RED[rop], PRE["IDENTITY"], 0, x, dim, with_index=True)
        vals = thc.Tensor.new(state, kind)
        idx = thc.Tensor.new(state, "Long")
        vals.call(name, vals, idx, dx, dim, 1)
        assert_bit_equal(vals.numpy(), want_v, f"{kind}.{name} values {shape} dim {dim} [{plan_name()}]")
        assert_bit_equal(idx.numpy(), want_i, f"{kind}.{name} indices {shape} dim {dim} [{plan_name()}]")


@pytest.mark.parametrize("kind", FP_KINDS)
def test_max_min_nan_rule(state, oracle, kind):
    """TH's scan takes a NaN as soon as it meets one and stops: the first NaN of a slice wins."""
    r = rng("nan", kind)
    for shape, dim in (((6, 200), 1), ((200, 64), 0)):
        x = random_array(r, kind, shape)
        x[2, 17] = np.nan
        x[2, 40] = np.nan
        x[150 % shape[0], 3] = np.nan
        dx = to_device(state, x)
        for name, rop in (("max", "MAX"), ("min", "MIN")):
            want_v, want_i = oracle.reduce_dim(RED[rop], 0, 0, x, dim, with_index=True)
            vals, idx = thc.Tensor.new(state, kind), thc.Tensor.new(state, "Long")
            vals.call(name, vals, idx, dx, dim, 1)
            assert_bit_equal(idx.numpy(), want_i, f"{kind}.{name} NaN positions")
            assert np.array_equal(np.isnan(vals.numpy()), np.isnan(want_v))


@pytest.mark.parametrize("kind", FP_KINDS)
@pytest.mark.parametrize("p", [0, 1, 2, 3, 2.5])
def test_norm_dim(state, oracle, kind, p):
    r = rng("norm", kind, p)
    for shape, dim, layout in (((33, 257), 1, "contiguous"), ((257, 64), 0, "contiguous"), ((20, 30), 1, "transposed")):
        x = make_view(r, kind, shape, layout)
        pre = {0: "NONZERO", 1: "ABS", 2: "SQUARE"}.get(p, "POWABS")
        acc = oracle.reduce_dim(RED["SUM"], PRE[pre], p, x, dim)
        if p == 2:
            want = oracle.pointwise(__import__("cutorch_b200")._lib.OP["POW"], np.zeros_like(acc), [acc], 0.5)
        elif p not in (0, 1):
            inv = float(np.array(1.0 / p, dtype=NP_OF_KIND[kind]))
            want = oracle.pointwise(__import__("cutorch_b200")._lib.OP["POW"], np.zeros_like(acc), [acc], inv)
        else:
            want = acc
        out = thc.Tensor.new(state, kind)
        out.call("norm", out, to_device(state, x), p, dim, 1)
        assert_reduction_close(out.numpy(), want, REL[kind] * 4, np.abs(want.astype(np.float64)), f"{kind}.norm({p}) {shape}")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_mean_dim(state, oracle, kind):
    from cutorch_b200._lib import OP
    r = rng("mean", kind)
    x = make_view(r, kind, (64, 130), "contiguous")
    for dim in (0, 1):
        s = oracle.reduce_dim(RED["SUM"], 0, 0, x, dim)
        want = oracle.pointwise(OP["DIV_S"], np.zeros_like(s), [s], x.shape[dim])
        out = thc.Tensor.new(state, kind)
        out.call("mean", out, to_device(state, x), dim, 1)
        if kind in INT_KINDS:
            assert_bit_equal(out.numpy(), want, f"{kind}.mean dim {dim}")
        else:
            assert_reduction_close(out.numpy(), want, REL[kind], np.abs(x.astype(np.float64)).mean(axis=dim, keepdims=True),
                                   f"{kind}.mean dim {dim}")


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("n,layout", [(1, "contiguous"), (1000, "contiguous"), (300007, "contiguous"),
                                       (70001, "strided"), (4096 * 9, "offset")])
def test_full_reductions(state, oracle, kind, n, layout):
    r = rng("all", kind, n)
    x = make_view(r, kind, (n,), layout)
    dx = to_device(state, x)
    want = oracle.reduce_all(RED["SUM"], 0, 0, x)
    got = dx.call("sumall", dx)
    if kind in INT_KINDS:
        assert got == want
    else:
        assert_reduction_close(got, want, REL[kind], np.abs(x.astype(np.float64)).sum(), f"{kind}.sumall n={n} {layout}")
    assert dx.call("minall", dx) == NP_OF_KIND[kind].type(oracle.reduce_all(RED["MIN"], 0, 0, x))
    assert dx.call("maxall", dx) == NP_OF_KIND[kind].type(oracle.reduce_all(RED["MAX"], 0, 0, x))
    m = dx.call("meanall", dx)
    if kind in INT_KINDS:
        assert m == int(want / n) if want >= 0 else m == -((-want) // n)
    else:
        assert_reduction_close(m, want / n, REL[kind], np.abs(x.astype(np.float64)).mean(), f"{kind}.meanall")


def test_full_reduction_is_repeatable(state):
    """Fixed partitioning and combine order: the same input gives the same bits every time."""
    r = rng("repeat")
    x = r.standard_normal(3_000_001).astype(np.float32)
    dx = to_device(state, x)
    first = dx.call("sumall", dx)
    for _ in range(5):
        assert dx.call("sumall", dx) == first


def test_prodall_and_multi_dim_views(state, oracle):
    r = rng("prodall")
    x = make_view(r, "Double", (7, 9, 11), "permuted")
    x[...] = r.uniform(0.9, 1.1, size=x.shape)
    dx = to_device(state, x)
    assert_reduction_close(dx.call("prodall", dx), oracle.reduce_all(RED["PROD"], 0, 0, x), 1e-12, 1.0, "prodall")
    assert_reduction_close(dx.call("sumall", dx), oracle.reduce_all(RED["SUM"], 0, 0, x), 1e-12, np.abs(x).sum(), "sumall 3-D permuted")


@pytest.mark.parametrize("kind", FP_KINDS)
def test_normall_varall_stdall(state, oracle, kind):
    r = rng("var", kind)
    x = random_array(r, kind, (5, 4001))
    dx = to_device(state, x)
    xd = x.astype(np.float64)
    rel = REL[kind] * 4
    assert_reduction_close(dx.call("normall", dx, 2), np.sqrt((xd * xd).sum()), rel, 1.0, "normall 2")
    assert_reduction_close(dx.call("normall", dx, 1), np.abs(xd).sum(), rel, 1.0, "normall 1")
    assert_reduction_close(dx.call("normall", dx, 0), float((xd != 0).sum()), rel, 1.0, "normall 0")
    assert_reduction_close(dx.call("normall", dx, 3), (np.abs(xd) ** 3).sum() ** (1 / 3), rel, 1.0, "normall 3")
    assert_reduction_close(dx.call("varall", dx, 0), xd.var(ddof=1), rel, 1.0, "varall unbiased")
    assert_reduction_close(dx.call("varall", dx, 1), xd.var(ddof=0), rel, 1.0, "varall biased")
    assert_reduction_close(dx.call("stdall", dx, 0), xd.std(ddof=1), rel, 1.0, "stdall")


def test_logical_all_any(state):
    import ctypes as C
    lib = load_library()
    for f in (lib.THCudaByteTensor_logicalall, lib.THCudaByteTensor_logicalany):
        f.argtypes = [C.c_void_p, C.c_void_p]
    x = np.ones(100003, dtype=np.uint8)
    dx = to_device(state, x)
    assert lib.THCudaByteTensor_logicalall(state.ptr, dx.ptr) == 1
    x[77777] = 0
    dx = to_device(state, x)
    assert lib.THCudaByteTensor_logicalall(state.ptr, dx.ptr) == 0
    assert lib.THCudaByteTensor_logicalany(state.ptr, dx.ptr) == 1
    dz = to_device(state, np.zeros(5000, dtype=np.uint8))
    assert lib.THCudaByteTensor_logicalany(state.ptr, dz.ptr) == 0


def test_int_sum_is_exact_beyond_32_bits(state, oracle):
    r = rng("i64")
    x = r.integers(-2**30, 2**30, size=(4, 100001)).astype(np.int32)
    dx = to_device(state, x)
    assert dx.call("sumall", dx) == int(x.astype(np.int64).sum())
    out = thc.Tensor.new(state, "Int")
    out.call("sum", out, dx, 1, 1)
    assert_bit_equal(out.numpy(), x.astype(np.int64).sum(axis=1, keepdims=True).astype(np.int32), "Int.sum wraps on store only")


@pytest.mark.parametrize("kind", FP_KINDS)
@pytest.mark.parametrize("case", [0, 1, 2, 3, 4, 6, 7])
def test_var_std_dim(state, oracle, kind, case):
    """var / std along a dim (sum and sum of squares in the accumulate type, TH's formula)."""
    shape, dim, layout = SHAPES[case]
    r = rng("var_dim", kind, case)
    x = make_view(r, kind, shape, layout)
    dx = to_device(state, x)
    for biased in (0, 1):
        for name, take_sqrt in (("var", False), ("std", True)):
            want = oracle.var_dim(x, dim, bool(biased), take_sqrt)
            out = thc.Tensor.new(state, kind)
            out.call(name, out, dx, dim, biased, 1)
            scale = np.maximum(np.abs(want.astype(np.float64)), 1e-3)
            assert_reduction_close(out.numpy(), want, REL[kind] * 8, scale, f"{kind}.{name} biased={biased} {shape} dim {dim} [{plan_name()}]")


@pytest.mark.parametrize("kind", FP_KINDS)
def test_dist(state, oracle, kind):
    r = rng("dist", kind)
    a = make_view(r, kind, (37, 129), "transposed")
    b = make_view(r, kind, (37, 129), "contiguous")
    da, db = to_device(state, a), to_device(state, b)
    d = (np.ascontiguousarray(a) - np.ascontiguousarray(b)).astype(np.float64)   # difference rounded to the element type first
    for p, want in ((0, float((d != 0).sum())), (1, np.abs(d).sum()), (2, np.sqrt((d * d).sum())), (3, (np.abs(d) ** 3).sum() ** (1 / 3))):
        assert_reduction_close(da.call("dist", da, db, p), want, REL[kind] * 4, 1.0, f"{kind}.dist({p})")


def test_combine_of_gathered_value_position_pairs_on_the_gpu(state):
    """The combine step of a max / min with positions along a sharded dim (cutorch_b200.shard):
    on the GPU it is this library's max-with-positions over the rank dim plus a gather of the
    positions, and has to agree with the rule applied by plain torch operations on the host."""
    import torch
    from cutorch_b200.shard import combine_gathered
    r = rng("combine-gathered")
    world, n = 8, 5000
    vals = r.integers(-3, 4, size=(world, n)).astype(np.float32)      # many ties across ranks
    vals[r.uniform(size=vals.shape) < 0.01] = np.nan                  # a NaN wins, the first one
    rows_per_rank = 100
    poss = (r.integers(1, rows_per_rank + 1, size=(world, n)) + np.arange(world)[:, None] * rows_per_rank).astype(np.int64)
    stream = torch.cuda.current_stream()
    state.set_stream(stream.cuda_stream, 0)
    try:
        for is_max in (True, False):
            want_v, want_p = combine_gathered(torch.from_numpy(vals), torch.from_numpy(poss), is_max, None)
            got_v, got_p = combine_gathered(torch.from_numpy(vals).cuda(), torch.from_numpy(poss).cuda(), is_max, state)
            torch.cuda.synchronize()
            assert_bit_equal(got_v.cpu().numpy(), want_v.numpy(), f"combined values, max={is_max}")
            assert_bit_equal(got_p.cpu().numpy(), want_p.numpy(), f"combined positions, max={is_max}")
    finally:
        state.set_stream(0, 0)
