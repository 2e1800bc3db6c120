"""The pointwise planner is host code: which kernel family a set of strided views gets can be
checked without a GPU (thcb200_pointwise_plan).  Views are described over fake, suitably aligned
addresses; nothing is dereferenced.

The layouts are those of the baseline configs (row d of the scope table: c1 contiguous, c2
transposed + stride-2 operands) and the ones the reference's apply meets through narrow /
transpose / expand (lib/THC/generic/THCTensor.c:440-499, 627-642)."""
import ctypes as C

import pytest

from cutorch_b200 import _lib

BASE = 0x7F0000000000   # 4 KiB aligned fake device addresses, far apart
F32 = _lib.F32


@pytest.fixture(scope="module")
def plan():
    lib = _lib.load_library()
    lib.thcb200_pointwise_plan.restype = C.c_char_p
    lib.thcb200_pointwise_plan.argtypes = [C.c_void_p] * 4 + [C.c_int]

    def run(*views, dtype=F32):
        descs = [_lib.make_desc(BASE + (k << 36) + off, dtype, sizes, strides) for k, (off, sizes, strides) in enumerate(views)]
        ptrs = [C.byref(d) for d in descs] + [None] * (4 - len(descs))
        r = lib.thcb200_pointwise_plan(*ptrs, len(descs) - 1)
        return r.decode() if r else None
    return run


def contiguous(sizes):
    strides, run = [], 1
    for n in reversed(sizes):
        strides.insert(0, run)
        run *= n
    return strides


def test_contiguous_operands_collapse_to_one_run(plan):
    s = (64, 256, 56, 56)
    v = (0, s, contiguous(s))
    assert plan(v, v, v) == "contig_vec"
    # the same transposition applied to every operand is still one run (dims are sorted by stride)
    t = (0, (56, 256), (1, 56))
    assert plan(t, t, t) == "contig_vec"
    # 16- but not 32-byte aligned
    assert plan((16, (1024,), (1,)), (16, (1024,), (1,))) == "contig_vec16"
    # one element past an alignment boundary: the per-element walk over a single dim
    assert plan((4, (1024,), (1,)), (4, (1024,), (1,))) == "generic32"


def test_c2_views_take_the_tiled_kernel(plan):
    s = (64, 256, 56, 56)
    out = (0, s, contiguous(s))
    y = (0, s, (802816, 1, 256, 14336))            # dims 1 and 3 of a (64,56,56,256) tensor swapped
    w = (0, s, (1605632, 6272, 112, 2))            # every second element of the last dim
    assert plan(out, out, y, w) == "tiled"


def test_dense_inner_dim_takes_the_row_kernels(plan):
    R, Cc = 1000, 256
    full = (0, (R, Cc), (Cc, 1))
    per_row = (0, (R, Cc), (1, 0))                 # an expanded (R, 1) factor
    per_col = (0, (R, Cc), (0, 1))                 # an expanded (1, C) bias
    assert plan(full, full, per_row) == "rows"
    assert plan(full, full, per_col) == "rows"
    assert plan(full, full, per_row, per_col) == "rows"
    padded = (0, (R, Cc), (Cc + 32, 1))
    assert plan(padded, full) == "rows"
    # an odd pitch breaks the 16-byte alignment from row to row: element-wise rows
    odd = (0, (R, 255), (259, 1))
    assert plan(odd, odd) == "rows_scalar"
    # a window of a larger 3-D tensor: three dims, none collapsible, inner one dense
    win = (4 * (514 * 1004 + 1004 + 2), (256, 512, 1000), (514 * 1004, 1004, 1))
    assert plan(win, win, win) == "rows_scalar"    # the window starts 8 bytes past a boundary
    win4 = (4 * (514 * 1004 + 1004 + 4), (256, 512, 1000), (514 * 1004, 1004, 1))
    assert plan(win4, win4, win4) == "rows"


def test_what_is_left_for_the_generic_walk(plan):
    # an inner stride of 2 on the output
    assert plan((0, (100, 50), (100, 2)), (0, (100, 50), (50, 1))) == "generic32"
    # operands of different shapes (only the element counts agree)
    assert plan((0, (12, 10), (10, 1)), (0, (120,), (2,))) == "generic32"
    # offsets beyond 32 bits
    assert plan((0, (2, 3, 2), (2**32 + 16, 5, 2)), (0, (2, 3, 2), (6, 2, 1)), dtype=_lib.U8) == "generic64"
    # more than eight dims that do not collapse
    deep_sizes = (2,) * 10
    deep_strides = tuple(3 * 4 ** k for k in reversed(range(10)))
    assert plan((0, deep_sizes, deep_strides), (0, deep_sizes, deep_strides)) == "deep"


def test_bad_arguments(plan):
    assert plan((0, (10,), (1,)), (0, (11,), (1,))) is None
    assert b"element counts" in _lib.load_library().thcb200_last_error()
