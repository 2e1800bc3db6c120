"""The CPU oracle against independent implementations (numpy and CPU torch).

torch7's TH, the parity target, is not available, so the TH-specific rules of
oracle/th_oracle.cpp are restated from its published behaviour: sums and products accumulate in
double (float) or int64 (integers) and round once; max / min along a dim return the FIRST
occurrence of the extreme, 1-based, and a NaN, once met, wins; scans run in the accumulate type.
numpy and torch's CPU kernels implement the same rules independently (np.argmax returns the first
maximum and treats NaN as the maximum; torch.max(dim) agrees).  They are a secondary check, as a
second opinion on the oracle -- the product is compared with the oracle, not with these."""
import numpy as np
import pytest
import torch

from cutorch_b200._lib import PRE, RED
from common import LAYOUTS, make_view, rng


@pytest.mark.parametrize("layout", LAYOUTS)
def test_sums_accumulate_in_double_and_round_once(oracle, layout):
    r = rng("xcheck-sum", layout)
    x = make_view(r, "Float", (37, 29, 11), layout)
    for dim in range(3):
        want = np.asarray(x, np.float64).sum(axis=dim, keepdims=True).astype(np.float32)
        got = oracle.reduce_dim(RED["SUM"], PRE["IDENTITY"], 0.0, x, dim)
        # numpy's pairwise double sum and the oracle's sequential double sum agree to the last bit after
        # rounding to float except where the double sums straddle a rounding boundary
        assert np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)) / np.maximum(np.abs(want), 1e-30)) <= 2 ** -23
    total = oracle.reduce_all(RED["SUM"], PRE["IDENTITY"], 0.0, x)
    assert abs(total - np.asarray(x, np.float64).sum()) <= 1e-12 * np.abs(x).astype(np.float64).sum()
    i = make_view(r, "Int", (50, 40), layout)
    i[...] = r.integers(-2**30, 2**30, size=(50, 40))
    assert oracle.reduce_all(RED["SUM"], PRE["IDENTITY"], 0.0, i) == int(np.asarray(i, np.int64).sum())    # no 32-bit wrap
    got = oracle.reduce_dim(RED["SUM"], PRE["IDENTITY"], 0.0, i, 0)
    assert np.array_equal(got, np.asarray(i, np.int64).sum(axis=0, keepdims=True).astype(np.int32))       # wraps once, at the end


@pytest.mark.parametrize("kind", ["Float", "Double", "Int", "Byte", "Half"])
def test_max_min_along_a_dim_return_the_first_occurrence(oracle, kind):
    r = rng("xcheck-arg", kind)
    for shape, dim in [((64, 50), 0), ((64, 50), 1), ((5, 33, 7), 1)]:
        x = make_view(r, kind, shape, "contiguous")
        x[...] = r.integers(0, 4, size=shape).astype(x.dtype)      # four values: ties everywhere
        for rop, np_arg, t_fn in (("MAX", np.argmax, torch.max), ("MIN", np.argmin, torch.min)):
            v, i = oracle.reduce_dim(RED[rop], PRE["IDENTITY"], 0.0, x, dim, with_index=True)
            want_i = np.expand_dims(np_arg(x, axis=dim), dim) + 1                      # numpy: first occurrence, 0-based
            assert np.array_equal(i, want_i), f"{kind} {rop} {shape} dim {dim}: positions differ from numpy's first occurrence"
            assert np.array_equal(v, np.take_along_axis(x, want_i - 1, axis=dim))
            if kind != "Half":
                tv, ti = t_fn(torch.from_numpy(np.ascontiguousarray(x)), dim=dim, keepdim=True)
                assert np.array_equal(v, tv.numpy())
                # torch documents no tie rule for max(dim); where it returns the first occurrence it must agree
                if np.array_equal(ti.numpy() + 1, want_i):
                    assert np.array_equal(i, ti.numpy() + 1)


def test_a_nan_wins_max_and_min_and_the_first_one_is_reported(oracle):
    x = np.array([[1.0, np.nan, 5.0, np.nan, 2.0], [3.0, 3.0, 1.0, 0.0, 3.0], [np.nan, 0.0, 0.0, 0.0, 0.0]], np.float32)
    for rop, np_arg in (("MAX", np.argmax), ("MIN", np.argmin)):
        v, i = oracle.reduce_dim(RED[rop], PRE["IDENTITY"], 0.0, x, 1, with_index=True)
        assert np.isnan(v[0, 0]) and i[0, 0] == 2          # the first NaN, 1-based
        assert np.isnan(v[2, 0]) and i[2, 0] == 1
        # numpy's argmax / argmin treat NaN the same way: the first NaN is the answer
        assert np.array_equal(i[:, 0], np_arg(x, axis=1) + 1)
    tv, ti = torch.max(torch.from_numpy(x), dim=1)
    assert torch.isnan(tv[0]) and int(ti[0]) + 1 == 2
    assert np.isnan(oracle.reduce_all(RED["MAX"], PRE["IDENTITY"], 0.0, x))
    assert np.isnan(oracle.reduce_all(RED["MIN"], PRE["IDENTITY"], 0.0, x))


def test_scans_and_products_follow_numpy_in_the_accumulate_type(oracle):
    r = rng("xcheck-scan")
    x = (r.integers(-8, 9, size=(40, 30)) / 4).astype(np.float32)         # exact partial sums
    for dim in (0, 1):
        assert np.array_equal(oracle.scan_dim(False, x, dim), np.cumsum(x.astype(np.float64), axis=dim).astype(np.float32))
    p = r.uniform(0.9, 1.1, size=(12, 9)).astype(np.float32)
    want = np.cumprod(p.astype(np.float64), axis=1).astype(np.float32)
    assert np.array_equal(oracle.scan_dim(True, p, 1), want)
    got = oracle.reduce_dim(RED["PROD"], PRE["IDENTITY"], 0.0, p, 1)
    assert np.array_equal(got[:, 0], np.prod(p.astype(np.float64), axis=1).astype(np.float32))
    i8 = r.integers(-100, 100, size=(3, 300)).astype(np.int8)
    assert np.array_equal(oracle.scan_dim(False, i8, 1), np.cumsum(i8.astype(np.int64), axis=1).astype(np.int8))


def test_norms_and_means_against_numpy(oracle):
    r = rng("xcheck-norm")
    x = r.standard_normal((33, 21)).astype(np.float32)
    for dim in (0, 1):
        s2 = oracle.reduce_dim(RED["SUM"], PRE["SQUARE"], 0.0, x, dim)
        assert np.allclose(s2, (x.astype(np.float64) ** 2).sum(axis=dim, keepdims=True), rtol=2e-7)
        s1 = oracle.reduce_dim(RED["SUM"], PRE["ABS"], 0.0, x, dim)
        assert np.allclose(s1, np.abs(x.astype(np.float64)).sum(axis=dim, keepdims=True), rtol=2e-7)
        nz = oracle.reduce_dim(RED["SUM"], PRE["NONZERO"], 0.0, x, dim)
        assert np.array_equal(nz, np.count_nonzero(x, axis=dim, keepdims=True).astype(np.float32))
        var = oracle.var_dim(x, dim, False, False)
        assert np.allclose(var, x.astype(np.float64).var(axis=dim, ddof=1, keepdims=True), rtol=1e-5)
        std = oracle.var_dim(x, dim, True, True)
        assert np.allclose(std, x.astype(np.float64).std(axis=dim, ddof=0, keepdims=True), rtol=1e-5)
