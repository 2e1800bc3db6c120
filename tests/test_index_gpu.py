"""indexSelect / indexCopy / indexAdd / indexFill and gather / scatter / scatterAdd / scatterFill
through the THC C API against oracle/index_oracle.py.  Every result is a moved element, the fill
value, or (adds) a sum of values chosen so that it is exact: all comparisons are bit-exact.

cutorch's tests: test/test.lua:2345-2560 (index* over each dim, contiguous and transposed, 1-D to
3-D, duplicate-free index vectors for copy), :2880-3010 (gather / scatter / scatterFill with random
index tensors)."""
import ctypes as C

import numpy as np
import pytest

from cutorch_b200 import thc
from oracle import index_oracle as io
from common import ALL_KINDS, assert_bit_equal, make_view, rng, to_device

pytestmark = pytest.mark.gpu


def exact_values(r, kind, shape, layout):
    x = make_view(r, kind, shape, layout)
    if x.dtype.kind == "f":
        x[...] = (r.integers(-16, 17, size=shape) / 4).astype(x.dtype)
    else:
        x[...] = r.integers(0, 6, size=shape).astype(x.dtype)
    return x


SHAPES = [((40, 50), "contiguous"), ((40, 50), "transposed"), ((6, 7, 8), "permuted"), ((300,), "contiguous"),
          ((5, 9, 4, 3), "holes"), ((33, 65), "offset")]


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_index_select_copy_add_fill(state, kind):
    r = rng("index", kind)
    for shape, layout in SHAPES:
        src = exact_values(r, kind, shape, layout)
        dsrc = to_device(state, src)
        for dim in range(len(shape)):
            n = shape[dim]
            # select: any positions, duplicates allowed, index vector itself strided
            pick = r.integers(1, n + 1, size=2 * n + 3).astype(np.int64)
            didx = to_device(state, np.repeat(pick, 2)[::2])
            out = thc.Tensor.new(state, kind)
            out.indexSelect(dsrc, dim, didx)
            want = io.index_select(src, dim, pick)
            assert out.sizes == list(want.shape)
            assert_bit_equal(out.numpy(), want, f"{kind} indexSelect {shape} {layout} dim {dim}")
            # copy: a duplicate-free subset of positions, source slices in index order
            m = max(1, n // 2)
            perm = (r.permutation(n)[:m] + 1).astype(np.int64)
            sshape = list(shape)
            sshape[dim] = m
            part = exact_values(r, kind, tuple(sshape), "contiguous")
            dst = exact_values(r, kind, shape, layout)
            ddst = to_device(state, dst)
            ddst.indexCopy(dim, to_device(state, perm), to_device(state, part))
            assert_bit_equal(ddst.numpy(), io.index_copy(dst, dim, perm, part), f"{kind} indexCopy {shape} dim {dim}")
            # add: duplicates accumulate
            dup = r.integers(1, n + 1, size=m).astype(np.int64)
            ddst = to_device(state, dst)
            ddst.indexAdd(dim, to_device(state, dup), to_device(state, part))
            assert_bit_equal(ddst.numpy(), io.index_add(dst, dim, dup, part), f"{kind} indexAdd {shape} dim {dim}")
            # fill
            ddst = to_device(state, dst)
            ddst.indexFill(dim, to_device(state, dup), 3)
            assert_bit_equal(ddst.numpy(), io.index_fill(dst, dim, dup, 3), f"{kind} indexFill {shape} dim {dim}")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_gather_scatter(state, kind):
    r = rng("gather", kind)
    for shape, layout in SHAPES:
        src = exact_values(r, kind, shape, layout)
        dsrc = to_device(state, src)
        for dim in range(len(shape)):
            n = shape[dim]
            # gather: output (and index) may be longer or shorter than src along dim
            oshape = list(shape)
            oshape[dim] = n + 3
            index = r.integers(1, n + 1, size=oshape).astype(np.int64)
            out = thc.Tensor.new(state, kind, *oshape)
            out.gather(dsrc, dim, to_device(state, index))
            assert_bit_equal(out.numpy(), io.gather(src, dim, index), f"{kind} gather {shape} {layout} dim {dim}")
            # scatter: each source element goes to a distinct position along dim (a permutation per line)
            big = list(shape)
            big[dim] = n + 2
            dst = exact_values(r, kind, tuple(big), "contiguous")
            perm = np.argsort(r.uniform(size=big), axis=dim).astype(np.int64) + 1
            perm = np.take(perm, np.arange(n), axis=dim)
            dperm = to_device(state, np.ascontiguousarray(perm))
            ddst = to_device(state, dst)
            ddst.scatter(dim, dperm, dsrc)
            assert_bit_equal(ddst.numpy(), io.scatter(dst, dim, perm, src), f"{kind} scatter {shape} {layout} dim {dim}")
            # scatterAdd with collisions, scatterFill
            hits = r.integers(1, n + 3, size=shape).astype(np.int64)
            ddst = to_device(state, dst)
            ddst.scatterAdd(dim, to_device(state, hits), dsrc)
            assert_bit_equal(ddst.numpy(), io.scatter_add(dst, dim, hits, src), f"{kind} scatterAdd {shape} dim {dim}")
            ddst = to_device(state, dst)
            ddst.scatterFill(dim, to_device(state, hits), 2)
            assert_bit_equal(ddst.numpy(), io.scatter_fill(dst, dim, hits, 2), f"{kind} scatterFill {shape} dim {dim}")


def test_index_argument_errors_and_out_of_range_positions(state):
    lib = state.lib
    lib.thcb200_take_index_errors.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.c_void_p]
    r = rng("index-errors")
    src = exact_values(r, "Float", (10, 20), "contiguous")
    dsrc = to_device(state, src)
    out = thc.Tensor.new(state, "Float")
    with pytest.raises(thc.THCError, match="expecting vector of indices"):
        out.indexSelect(dsrc, 0, to_device(state, np.ones((2, 2), np.int64)))
    with pytest.raises(thc.THCError, match="Indexing dim is out of bounds"):
        out.indexSelect(dsrc, 2, to_device(state, np.ones(3, np.int64)))
    with pytest.raises(thc.THCError, match="not equal to length of indices"):
        dsrc.indexCopy(0, to_device(state, np.ones(3, np.int64)), dsrc)
    with pytest.raises(thc.THCError, match="same size as output tensor"):
        out.resize(4, 20)
        out.gather(dsrc, 0, to_device(state, np.ones((3, 20), np.int64)))
    # positions outside 1..size are skipped and counted, never dereferenced
    count = C.c_int64(-1)
    assert lib.thcb200_take_index_errors(C.c_void_p(state.context), C.byref(count), C.c_void_p(state.stream)) == 0
    idx = np.array([1, 0, 11, 5, -3], np.int64)
    out.indexSelect(dsrc, 0, to_device(state, idx))
    got = out.numpy()
    assert_bit_equal(got[[0, 3]], src[[0, 4]], "valid rows")
    assert lib.thcb200_take_index_errors(C.c_void_p(state.context), C.byref(count), C.c_void_p(state.stream)) == 0
    assert count.value in (3 * 20, 3 * 20 // 4)   # counted per move: elements, or 16-byte words on the vector path
    assert lib.thcb200_take_index_errors(C.c_void_p(state.context), C.byref(count), C.c_void_p(state.stream)) == 0
    assert count.value == 0


def test_index_select_large_rows(state):
    """An embedding-style lookup: 2^16 rows of 1024 floats picked from a 2^15-row table."""
    r = rng("index-large")
    table = r.standard_normal((1 << 15, 1024)).astype(np.float32)
    idx = r.integers(1, (1 << 15) + 1, size=1 << 16).astype(np.int64)
    out = thc.Tensor.new(state, "Float")
    out.indexSelect(to_device(state, table), 0, to_device(state, idx))
    assert_bit_equal(out.numpy(), table[idx - 1], "large indexSelect")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_gather_scatter_four_neighbours_per_thread(state, kind):
    """Contiguous tensors whose innermost size is a multiple of four take the kernel that handles
    four neighbours per thread (one 32-byte index load, one vector access on the plain side); same
    results bit for bit, out-of-range positions skipped and counted there too."""
    from cutorch_b200 import _lib
    lib = _lib.load_library()
    lib.thcb200_take_index_errors.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.c_void_p]
    r = rng("gather quads", kind)
    count = C.c_int64(-1)
    for shape in ((64, 256), (3, 20, 36)):
        src = exact_values(r, kind, shape, "contiguous")
        dsrc = to_device(state, src)
        for dim in range(len(shape)):
            n = shape[dim]
            oshape = list(shape)
            if dim != len(shape) - 1:
                oshape[dim] = n + 3
            index = r.integers(1, n + 1, size=oshape).astype(np.int64)
            out = thc.Tensor.new(state, kind, *oshape)
            out.gather(dsrc, dim, to_device(state, index))
            assert lib.thcb200_last_plan() == b"indexed_quad32"
            assert_bit_equal(out.numpy(), io.gather(src, dim, index), f"{kind} gather {shape} dim {dim}")
            dst = exact_values(r, kind, shape, "contiguous")
            perm = (np.argsort(r.uniform(size=shape), axis=dim).astype(np.int64) + 1)
            ddst = to_device(state, dst)
            ddst.scatter(dim, to_device(state, perm), dsrc)
            assert lib.thcb200_last_plan() == b"indexed_quad32"
            assert_bit_equal(ddst.numpy(), io.scatter(dst, dim, perm, src), f"{kind} scatter {shape} dim {dim}")
            hits = r.integers(1, n + 1, size=shape).astype(np.int64)
            ddst = to_device(state, dst)
            ddst.scatterAdd(dim, to_device(state, hits), dsrc)
            assert lib.thcb200_last_plan() == b"indexed_quad32"
            assert_bit_equal(ddst.numpy(), io.scatter_add(dst, dim, hits, src), f"{kind} scatterAdd {shape} dim {dim}")
            ddst = to_device(state, dst)
            ddst.scatterFill(dim, to_device(state, hits), 2)
            assert lib.thcb200_last_plan() == b"indexed_quad32"
            assert_bit_equal(ddst.numpy(), io.scatter_fill(dst, dim, hits, 2), f"{kind} scatterFill {shape} dim {dim}")
            # positions out of range: those elements keep what the output held
            lib.thcb200_take_index_errors(C.c_void_p(state.context), C.byref(count), C.c_void_p(state.stream))
            broken = index.copy()
            flat = broken.reshape(-1)
            where = r.choice(flat.size, size=37, replace=False)
            flat[where] = r.choice([0, -5, n + 1, n + 1000], size=37)
            before = exact_values(r, kind, tuple(oshape), "contiguous")
            dout = to_device(state, before)
            dout.gather(dsrc, dim, to_device(state, broken))
            want = io.gather(src, dim, np.where((broken >= 1) & (broken <= n), broken, 1))
            mask = ((broken < 1) | (broken > n))
            want[mask] = before[mask]
            assert_bit_equal(dout.numpy(), want, f"{kind} gather with positions out of range {shape} dim {dim}")
            lib.thcb200_take_index_errors(C.c_void_p(state.context), C.byref(count), C.c_void_p(state.stream))
            assert count.value == 37


@pytest.mark.parametrize("kind", ["Float", "Long", "Half"])
def test_index_calls_with_positions_in_a_cpu_tensor(state, kind):
    """index*_long: the positions come in a CPU LongTensor (lib/THC/generic/THCTensorIndex.h:10-13)."""
    r = rng("index-long", kind)
    src = exact_values(r, kind, (40, 50), "contiguous")
    dsrc = to_device(state, src)
    for dim in (0, 1):
        n = src.shape[dim]
        idx = r.integers(1, n + 1, size=17).astype(np.int64)
        out = thc.Tensor.new(state, kind)
        out.indexSelect_long(dsrc, dim, thc.CpuTensor(idx))
        assert_bit_equal(out.numpy(), io.index_select(src, dim, idx), f"{kind} indexSelect_long dim {dim}")
        perm = (r.permutation(n)[:9] + 1).astype(np.int64)
        shape = list(src.shape)
        shape[dim] = 9
        part = exact_values(r, kind, tuple(shape), "contiguous")
        dst = exact_values(r, kind, src.shape, "contiguous")
        ddst = to_device(state, dst)
        ddst.indexCopy_long(dim, thc.CpuTensor(perm), to_device(state, part))
        assert_bit_equal(ddst.numpy(), io.index_copy(dst, dim, perm, part), f"{kind} indexCopy_long dim {dim}")
        ddst = to_device(state, dst)
        ddst.indexAdd_long(dim, thc.CpuTensor(perm), to_device(state, part))
        assert_bit_equal(ddst.numpy(), io.index_add(dst, dim, perm, part), f"{kind} indexAdd_long dim {dim}")
        ddst = to_device(state, dst)
        ddst.indexFill_long(dim, thc.CpuTensor(perm[::2].copy()), 3)
        assert_bit_equal(ddst.numpy(), io.index_fill(dst, dim, perm[::2], 3), f"{kind} indexFill_long dim {dim}")
    with pytest.raises(thc.THCError, match="expecting vector of indices"):
        thc.Tensor.new(state, kind).indexSelect_long(dsrc, 0, thc.CpuTensor(np.ones((2, 2), np.int64)))
