"""Shared helpers of the parity tests: seeded inputs, strided views, ulp distance, and the
CPU-vs-CUDA comparison in the style of cutorch's test/test.lua (compareCPUAndCUDATypeTensorArgs,
test/test.lua:371-440): run the same op through the oracle on the host array and through the
THC C API on an exact device clone, then compare every output."""
from __future__ import annotations

import numpy as np

from cutorch_b200 import thc
from cutorch_b200._lib import OP, PRE, RED

NP_OF_KIND = {k: np.dtype(v[1]) for k, v in thc.KINDS.items()}
INT_KINDS = ["Byte", "Char", "Short", "Int", "Long"]
FP_KINDS = ["Half", "Float", "Double"]
ALL_KINDS = INT_KINDS + FP_KINDS


def rng(*seed_parts):
    """Seeded generator; string parts are hashed with crc32 so seeds do not depend on PYTHONHASHSEED."""
    import zlib
    seed = 0
    for part in seed_parts:
        seed = (seed * 1000003 + (part if isinstance(part, int) else zlib.crc32(str(part).encode()))) % (2**63)
    return np.random.default_rng(seed)


def random_array(r, kind, shape, lo=-4.0, hi=4.0):
    dt = NP_OF_KIND[kind]
    if dt.kind == "f":
        return r.uniform(lo, hi, size=shape).astype(dt)
    info = np.iinfo(dt)
    l, h = max(info.min, int(lo * 10)), min(info.max, int(hi * 10))
    return r.integers(l, h + 1, size=shape).astype(dt)


def make_view(r, base_kind, shape, layout):
    """Returns a numpy view of the requested logical shape over a larger or permuted buffer.
    layout: contiguous | transposed | strided (step 2 in the last dim) | holes (padding between
    rows) | offset (a slice that starts inside the buffer) | permuted (random dim order)."""
    shape = tuple(shape)
    nd = len(shape)
    if layout == "contiguous" or nd == 0:
        return random_array(r, base_kind, shape)
    if layout == "transposed":
        if nd < 2:
            return random_array(r, base_kind, shape)
        perm = list(range(nd))
        perm[0], perm[-1] = perm[-1], perm[0]
        base = random_array(r, base_kind, tuple(shape[p] for p in perm))
        return base.transpose(perm)
    if layout == "permuted":
        perm = list(r.permutation(nd))
        base = random_array(r, base_kind, tuple(shape[p] for p in perm))
        inv = np.argsort(perm)
        return base.transpose(inv)
    if layout == "strided":
        big = list(shape)
        big[-1] = shape[-1] * 2
        return random_array(r, base_kind, tuple(big))[..., ::2]
    if layout == "holes":
        big = list(shape)
        big[-1] = shape[-1] + 3
        return random_array(r, base_kind, tuple(big))[..., : shape[-1]]
    if layout == "offset":
        big = [n + 2 for n in shape]
        sl = tuple(slice(1, 1 + n) for n in shape)
        return random_array(r, base_kind, tuple(big))[sl]
    raise ValueError(layout)


LAYOUTS = ["contiguous", "transposed", "permuted", "strided", "holes", "offset"]


def ulp_diff(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between same-typed float arrays (NaN == NaN)."""
    assert a.dtype == b.dtype
    it = {2: np.int16, 4: np.int32, 8: np.int64}[a.dtype.itemsize]
    ai = a.view(it).astype(np.int64)
    bi = b.view(it).astype(np.int64)
    mask = np.int64((1 << (8 * a.dtype.itemsize - 1)) - 1)
    # sign-magnitude bit patterns -> integers that are monotonic in the float value
    ai = np.where(ai < 0, -(ai & mask), ai)
    bi = np.where(bi < 0, -(bi & mask), bi)
    d = np.abs(ai - bi)
    both_nan = np.isnan(a) & np.isnan(b)
    d = np.where(both_nan, 0, d)
    one_nan = np.isnan(a) ^ np.isnan(b)
    d = np.where(one_nan, np.iinfo(np.int64).max, d)
    return d


def assert_bit_equal(got: np.ndarray, want: np.ndarray, what=""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    if got.dtype.kind == "f":
        bad = ulp_diff(got, want) != 0
    else:
        bad = got != want
    if bad.any():
        k = np.argwhere(bad)[0]
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements differ; first at {tuple(k)}: "
                             f"got {got[tuple(k)]!r}, want {want[tuple(k)]!r}")


def assert_ulp(got: np.ndarray, want: np.ndarray, max_ulp: int, what=""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    d = ulp_diff(got, want)
    if (d > max_ulp).any():
        k = np.unravel_index(np.argmax(d), d.shape)
        raise AssertionError(f"{what}: max ulp distance {d.max()} > {max_ulp} at {k}: got {got[k]!r}, want {want[k]!r}")


def assert_reduction_close(got, want, rel, abs_sum, what=""):
    """|got - want| <= rel * max(|want|, eps * sum|x|): the stated relative tolerance, with a floor
    so that sums that cancel to nearly zero do not fail on rounding noise."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    abs_sum = np.asarray(abs_sum, dtype=np.float64)
    tol = rel * np.maximum(np.abs(want), abs_sum * 1e-3)
    err = np.abs(got - want)
    bad = ~(err <= tol) & ~(np.isnan(got) & np.isnan(want)) & ~((got == want))
    if bad.any():
        k = np.unravel_index(np.argmax(np.where(bad, err, 0)), err.shape) if err.shape else ()
        raise AssertionError(f"{what}: error {err[k] if err.shape else err} exceeds {tol[k] if tol.shape else tol} "
                             f"(got {got[k] if got.shape else got}, want {want[k] if want.shape else want})")


def to_device(state, arr):
    return thc.Tensor.from_numpy(state, arr)
