"""User-defined functors through the C++ template face (include/THC/THCApply.cuh), compiled into
cutorch_b200/lib/libthcb200_usertest.so from tests/csrc/user_apply_test.cu the way a downstream CUDA
library (cunn) would use cutorch's installed templates (lib/THC/THCApply.cuh:124-640)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from cutorch_b200 import _lib, thc
from common import assert_bit_equal, make_view, rng, to_device

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def user():
    _lib.load_library()
    p = Path(_lib.library_path()).parent / "libthcb200_usertest.so"
    if not p.exists():
        pytest.fail(f"{p} is missing: run __graft_entry__.build()")
    lib = C.CDLL(str(p))
    lib.usertest_scale.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float]
    lib.usertest_add_one.argtypes = [C.c_void_p, C.c_void_p]
    lib.usertest_cross.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    lib.usertest_less_than.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    return lib


def test_apply2_user_functor_on_strided_views(state, user):
    r = rng("user2")
    for la, lb in (("contiguous", "contiguous"), ("transposed", "strided"), ("holes", "permuted")):
        src = make_view(r, "Float", (6, 9, 11), la)
        dst = make_view(r, "Float", (6, 9, 11), lb)
        dsrc, ddst = to_device(state, src), to_device(state, dst)
        assert user.usertest_scale(state.ptr, ddst.ptr, dsrc.ptr, 2.5) == 1
        want = (np.ascontiguousarray(src) * np.float32(2.5)).astype(np.float32) + np.float32(1)
        assert_bit_equal(ddst.numpy(), want, f"user functor {la}/{lb}")


def test_apply2_patch_walk_and_dense_runs(state, user):
    """Transposed matrices (walked in 32 x 32 patches, ragged at both edges), dense operands taken in
    16-byte runs with a tail, and a dense operand that starts off a 16-byte boundary."""
    r = rng("user2-patch")
    for shape, la, lb in (((100, 70), "transposed", "contiguous"), ((257, 33), "contiguous", "transposed"),
                          ((31, 16), "transposed", "transposed"), ((5, 40, 50), "permuted", "contiguous"),
                          ((1, 100003), "contiguous", "contiguous"), ((640, 512), "transposed", "contiguous")):
        src = make_view(r, "Float", shape, la)
        dst = make_view(r, "Float", shape, lb)
        dsrc, ddst = to_device(state, src), to_device(state, dst)
        assert user.usertest_scale(state.ptr, ddst.ptr, dsrc.ptr, 0.5) == 1
        want = (np.ascontiguousarray(src) * np.float32(0.5)).astype(np.float32) + np.float32(1)
        assert_bit_equal(ddst.numpy(), want, f"user functor {shape} {la}/{lb}")
    # three collapsed dims whose last two are transposed (padded rows keep the outer dim from merging): the patch walk
    # with the dim-by-dim decode
    base3 = r.standard_normal((5, 50, 43)).astype(np.float32)
    src3 = base3[:, :, :40].transpose(0, 2, 1)
    dst3 = thc.Tensor.new(state, "Float", 5, 40, 50)
    assert user.usertest_scale(state.ptr, dst3.ptr, to_device(state, src3).ptr, 2.0) == 1
    assert_bit_equal(dst3.numpy(), np.ascontiguousarray(src3) * np.float32(2.0) + np.float32(1), "3-D source, last two dims transposed")
    # same storage for both operands: a shifted dense window (not 16-byte aligned, may alias)
    base = r.standard_normal(5000).astype(np.float32)
    dbase = to_device(state, base)
    a = thc.Tensor.wrap(state, "Float", dbase.data_ptr + 4, (4000,), (1,), storage_elems=4999)
    out = thc.Tensor.new(state, "Float", 4000)
    assert user.usertest_scale(state.ptr, out.ptr, a.ptr, 3.0) == 1
    assert_bit_equal(out.numpy(), base[1:4001] * np.float32(3.0) + np.float32(1), "dense but unaligned source")
    big = r.standard_normal(10007).astype(np.float32)
    dbig = to_device(state, big)
    assert user.usertest_add_one(state.ptr, dbig.ptr) == 1
    assert_bit_equal(dbig.numpy(), big + np.float32(1), "apply1 on a dense tensor with a tail")
    da, db = r.standard_normal(10003), r.standard_normal(10003)
    mask = thc.Tensor.new(state, "Byte", 10003)
    assert user.usertest_less_than(state.ptr, mask.ptr, to_device(state, da).ptr, to_device(state, db).ptr) == 1
    assert_bit_equal(mask.numpy(), (da < db).astype(np.uint8), "dense byte mask from dense double operands")


def test_apply2_different_shapes_same_count(state, user):
    r = rng("user2b")
    src = make_view(r, "Float", (4, 30), "transposed")
    dst = thc.Tensor.new(state, "Float", 120)
    assert user.usertest_scale(state.ptr, dst.ptr, to_device(state, src).ptr, 1.0) == 1
    assert_bit_equal(dst.numpy(), np.ascontiguousarray(src).reshape(120) + np.float32(1), "1-D out, 2-D transposed in")
    bad = thc.Tensor.new(state, "Float", 7)
    assert user.usertest_scale(state.ptr, bad.ptr, dst.ptr, 1.0) == 0   # element counts differ -> false


def test_apply1_in_place_and_overlapping_receiver(state, user):
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    dx = to_device(state, x)
    assert user.usertest_add_one(state.ptr, dx.ptr) == 1
    assert_bit_equal(dx.numpy(), x + 1, "apply1 in place")
    # an expanded (stride 0) receiver aliases: the op runs on a contiguous copy and is copied back
    base = to_device(state, np.arange(4, dtype=np.float32).reshape(1, 4))
    view = thc.Tensor.wrap(state, "Float", base.data_ptr, (3, 4), (0, 1), storage_elems=4)
    assert user.usertest_add_one(state.ptr, view.ptr) == 1
    assert_bit_equal(base.numpy(), np.arange(4, dtype=np.float32).reshape(1, 4) + 1, "apply1 on an expanded view")
    empty = thc.Tensor.new(state, "Float")
    assert user.usertest_add_one(state.ptr, empty.ptr) == 1   # no dimensions: no-op, true


def test_apply3_functor_reaching_neighbours_through_pointers(state, user):
    r = rng("user3")
    x = make_view(r, "Float", (5, 3, 7), "contiguous")
    y = make_view(r, "Float", (5, 3, 7), "permuted")
    out = thc.Tensor.new(state, "Float", 5, 3, 7)
    assert user.usertest_cross(state.ptr, out.ptr, to_device(state, x).ptr, to_device(state, y).ptr, 1) == 1
    xs, ys = np.ascontiguousarray(x), np.ascontiguousarray(y)
    want = np.zeros_like(xs)
    for i in range(3):
        j, k = (i + 1) % 3, (i + 2) % 3
        want[:, i, :] = xs[:, j, :] * ys[:, k, :] - xs[:, k, :] * ys[:, j, :]
    assert_bit_equal(out.numpy(), want, "cross through element pointers")


def test_apply3_mixed_element_types(state, user):
    r = rng("user3b")
    a = make_view(r, "Double", (8, 13), "transposed")
    b = make_view(r, "Double", (8, 13), "contiguous")
    mask = thc.Tensor.new(state, "Byte", 8, 13)
    assert user.usertest_less_than(state.ptr, mask.ptr, to_device(state, a).ptr, to_device(state, b).ptr) == 1
    assert_bit_equal(mask.numpy(), (np.ascontiguousarray(a) < b).astype(np.uint8), "byte mask from double operands")


# ---- THC_reduceDim / THC_reduceAll with user functors (include/THC/THCReduce.cuh) ----

def test_reduce_dim_user_functors(state, user):
    user.usertest_sumsq_dim.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    r = rng("user-reduce-dim")
    for shape, layout in [((40, 1000), "contiguous"), ((1000, 40), "transposed"), ((6, 7, 50), "permuted"),
                          ((3000, 5), "contiguous"), ((9, 2000, 3), "holes"), ((300, 70), "contiguous"), ((17, 33, 65), "offset"),
                          ((5, 700, 33), "contiguous"), ((3000, 40), "contiguous"), ((1003,), "contiguous"), ((100003,), "contiguous"),
                          ((8, 4100), "contiguous"), ((37, 1028), "contiguous"), ((2100, 256), "contiguous"), ((64, 36, 128), "contiguous"),
                          ((513, 132), "holes"), ((700, 260), "offset"), ((5000, 64), "contiguous"), ((4800, 50), "contiguous"),
                          ((4801, 36), "holes"), ((4800, 133), "holes"), ((4750, 132), "contiguous"), ((9, 133), "holes")]:
        # multiples of 1/4 so that float sums of squares are exact in any order
        x = make_view(r, "Float", shape, layout)
        x[...] = (r.integers(-8, 9, size=shape) / 4).astype(np.float32)
        dx = to_device(state, x)
        for dim in range(len(shape)):
            for keepdim in (1, 0):
                out = thc.Tensor.new(state, "Float")
                assert user.usertest_sumsq_dim(state.ptr, out.ptr, dx.ptr, dim, keepdim) == 1
                want = (np.asarray(x, dtype=np.float64) ** 2).sum(axis=dim, keepdims=bool(keepdim)).astype(np.float32)
                # a 1-D tensor keeps its only dim when squeezed (TH tensors have no 0-dim form)
                assert out.sizes == (list(want.shape) or [1]), (shape, dim, keepdim)
                assert_bit_equal(out.numpy(), want.reshape(out.sizes), f"user sum of squares {shape} {layout} dim {dim}")
    out = thc.Tensor.new(state, "Float")
    assert user.usertest_sumsq_dim(state.ptr, out.ptr, dx.ptr, 7, 1) == 0   # bad dim -> false


def test_reduce_all_user_functors(state, user):
    user.usertest_absmax_all.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]
    user.usertest_count_positive_device.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    user.usertest_minmax_all.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    r = rng("user-reduce-all")
    for shape, layout in [((100003,), "contiguous"), ((300, 500), "transposed"), ((7, 9, 11), "strided"), ((5,), "contiguous"),
                          ((3_000_000,), "contiguous")]:
        x = make_view(r, "Float", shape, layout)
        res = C.c_float(-1)
        assert user.usertest_absmax_all(state.ptr, to_device(state, x).ptr, C.byref(res)) == 1
        assert res.value == float(np.abs(x).max()), (shape, layout)
        d = make_view(r, "Double", shape, layout)
        slot = to_device(state, np.zeros(1, np.int64))
        assert user.usertest_count_positive_device(state.ptr, to_device(state, d).ptr, C.c_void_p(slot.data_ptr)) == 1
        assert int(slot.numpy()[0]) == int((d > 0).sum()), (shape, layout)
        i = make_view(r, "Int", shape, layout)
        i[...] = r.integers(-2**31, 2**31 - 1, size=shape).astype(np.int32)
        lo, hi = C.c_int(0), C.c_int(0)
        assert user.usertest_minmax_all(state.ptr, to_device(state, i).ptr, C.byref(lo), C.byref(hi)) == 1
        assert (lo.value, hi.value) == (int(i.min()), int(i.max())), (shape, layout)
    # a tensor without dimensions yields the initial value
    res = C.c_float(-1)
    assert user.usertest_absmax_all(state.ptr, thc.Tensor.new(state, "Float").ptr, C.byref(res)) == 1
    assert res.value == 0.0


def test_host_threads_share_a_state_with_a_stream_each(state, user):
    """Four host threads on one THCState: the current stream is per thread, and the split
    reductions and chunked scans of concurrent streams keep their partials apart."""
    user.usertest_threads.argtypes = [C.c_void_p, C.c_int, C.c_int]
    assert user.usertest_threads(state.ptr, 4, 25) == 0
    state.check()


# ---- seeded random layouts through the template headers ----

def _fuzz_shape(r):
    nd = int(r.integers(1, 4))
    while True:
        shape = tuple(int(r.choice([1, 2, 3, 5, 16, 31, 33, 40, 64, 100, 129, 257])) for _ in range(nd))
        if 0 < int(np.prod(shape)) <= 200000:
            return shape


def _shifted(state, view, shift):
    """The view on the device, its first element `shift` elements past a 256-byte boundary."""
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


@pytest.mark.parametrize("seed", range(12))
def test_apply_and_reduce_random_layouts(state, user, seed):
    """Every layout of common.make_view on either operand, bases on and off the 16-byte grid: the dense runs, the
    patch walk, the two-dim and the dim-by-dim decode, the warp / CTA / column reductions with and without vector loads."""
    from common import LAYOUTS
    user.usertest_sumsq_dim.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    r = rng("user-fuzz", seed)
    for _ in range(10):
        shape = _fuzz_shape(r)
        la, lb = (LAYOUTS[int(r.integers(0, len(LAYOUTS)))] for _ in range(2))
        sa, sb = (int(r.integers(0, 4)) for _ in range(2))
        src, dst = make_view(r, "Float", shape, la), make_view(r, "Float", shape, lb)
        dsrc, ddst = _shifted(state, src, sa), _shifted(state, dst, sb)
        assert user.usertest_scale(state.ptr, ddst.ptr, dsrc.ptr, 0.75) == 1
        want = (np.ascontiguousarray(src) * np.float32(0.75)).astype(np.float32) + np.float32(1)
        assert_bit_equal(ddst.numpy(), want, f"seed {seed}: scale {shape} {la}->{lb} shifts {sa},{sb}")
        assert user.usertest_add_one(state.ptr, ddst.ptr) == 1
        assert_bit_equal(ddst.numpy(), want + np.float32(1), f"seed {seed}: add one in place {shape} {lb} shift {sb}")
        # sums of squares of multiples of 1/4 are exact in any order
        x = make_view(r, "Float", shape, la)
        x[...] = (r.integers(-8, 9, size=shape) / 4).astype(np.float32)
        dx = _shifted(state, x, sa)
        dim = int(r.integers(0, len(shape)))
        out = thc.Tensor.new(state, "Float")
        assert user.usertest_sumsq_dim(state.ptr, out.ptr, dx.ptr, dim, 1) == 1
        wantr = (np.asarray(x, dtype=np.float64) ** 2).sum(axis=dim, keepdims=True).astype(np.float32)
        assert_bit_equal(out.numpy(), wantr, f"seed {seed}: sum of squares {shape} {la} shift {sa} dim {dim}")
