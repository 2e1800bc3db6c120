"""Comparisons into ByteTensors and Byte-masked fill / copy / select through the THC C API,
against the numpy restatement in oracle/mixed_oracle.py.  Bit-exact: every result is a copy of
an input element, a 0/1 byte, or the fill value.

cutorch's own tests of these calls: test/test.lua:1768-1800 (logical ops on every layout),
:2168-2330 (maskedSelect / maskedCopy / maskedFill, contiguous and transposed operands)."""
import numpy as np
import pytest

from cutorch_b200 import thc
from oracle import mixed_oracle as mo
from common import ALL_KINDS, LAYOUTS, NP_OF_KIND, assert_bit_equal, make_view, rng, to_device

pytestmark = pytest.mark.gpu

CMPS = ["lt", "gt", "le", "ge", "eq", "ne"]


def small_ints(r, kind, shape, layout):
    """Values from a small set so that equal elements are common."""
    x = make_view(r, kind, shape, layout)
    x[...] = r.integers(0, 5, size=shape).astype(x.dtype)
    return x


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("cmp", CMPS)
def test_compare_value_to_byte(state, kind, cmp):
    r = rng("cmpv", kind, cmp)
    for shape, layout in [((10007,), "contiguous"), ((65, 33), "transposed"), ((7, 9, 10), "strided"), ((4099,), "offset")]:
        x = small_ints(r, kind, shape, layout)
        dx = to_device(state, x)
        out = thc.Tensor.new(state, "Byte")
        dx.call(cmp + "Value", out, dx, 2)
        assert out.sizes == list(shape)
        assert_bit_equal(out.numpy(), mo.compare(cmp, x, 2), f"{kind} {cmp}Value {layout}")
        # same comparison into a tensor of the operand's type
        outT = thc.Tensor.new(state, kind)
        dx.call(cmp + "ValueT", outT, dx, 2)
        assert_bit_equal(outT.numpy(), mo.compare(cmp, x, 2).astype(x.dtype), f"{kind} {cmp}ValueT {layout}")


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("cmp", CMPS)
def test_compare_tensor_to_byte(state, kind, cmp):
    r = rng("cmpt", kind, cmp)
    cases = [((20011,), "contiguous", "contiguous"), ((40, 50), "contiguous", "transposed"),
             ((6, 5, 12), "permuted", "holes"), ((33, 17), "strided", "offset")]
    for shape, la, lb in cases:
        a, b = small_ints(r, kind, shape, la), small_ints(r, kind, shape, lb)
        da, db = to_device(state, a), to_device(state, b)
        out = thc.Tensor.new(state, "Byte")
        da.call(cmp + "Tensor", out, da, db)
        assert_bit_equal(out.numpy(), mo.compare(cmp, a, b), f"{kind} {cmp}Tensor {la}/{lb}")
        outT = thc.Tensor.new(state, kind)
        da.call(cmp + "TensorT", outT, da, db)
        assert_bit_equal(outT.numpy(), mo.compare(cmp, a, b).astype(a.dtype), f"{kind} {cmp}TensorT {la}/{lb}")


def test_compare_nan_and_half(state):
    x = np.array([0.0, np.nan, 1.0, -np.inf, np.inf, 65504.0, -0.0], dtype=np.float16)
    y = np.array([np.nan, np.nan, 1.0, -np.inf, 1.0, 65504.0, 0.0], dtype=np.float16)
    for kind in ["Half", "Float", "Double"]:
        a, b = x.astype(NP_OF_KIND[kind]), y.astype(NP_OF_KIND[kind])
        da, db = to_device(state, a), to_device(state, b)
        for cmp in CMPS:
            out = thc.Tensor.new(state, "Byte")
            da.call(cmp + "Tensor", out, da, db)
            assert_bit_equal(out.numpy(), mo.compare(cmp, a, b), f"{kind} {cmp} NaN")


def test_compare_into_strided_byte_output_and_different_shapes(state):
    r = rng("cmp-shapes")
    a = small_ints(r, "Float", (12, 10), "contiguous")
    b = small_ints(r, "Float", (120,), "contiguous")   # same element count, other shape
    da, db = to_device(state, a), to_device(state, b)
    out = thc.Tensor.new(state, "Byte")
    da.call("geTensor", out, da, db)
    assert out.sizes == [12, 10]
    assert_bit_equal(out.numpy(), mo.compare("ge", a, b), "different shapes")
    with pytest.raises(thc.THCError, match="sizes do not match"):
        da.call("geTensor", out, da, to_device(state, np.zeros(7, np.float32)))


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_masked_fill(state, kind):
    r = rng("mfill", kind)
    cases = [((10007,), "contiguous", "contiguous"), ((64, 48), "transposed", "contiguous"),
             ((64, 48), "contiguous", "transposed"), ((5, 6, 7), "strided", "holes"), ((4100,), "offset", "offset")]
    for shape, lt, lm in cases:
        t = make_view(r, kind, shape, lt)
        mask = make_view(r, "Byte", shape, lm)
        mask[...] = r.integers(0, 2, size=shape).astype(np.uint8)
        dt_, dm = to_device(state, t), to_device(state, mask)
        dt_.maskedFill(dm, 3)
        assert_bit_equal(dt_.numpy(), mo.masked_fill(t, mask, 3), f"{kind} maskedFill {lt}/{lm}")
    # all set, none set, and mask bytes other than 1 count as set
    for fill in (0, 1, 7):
        t = make_view(r, kind, (3000,), "contiguous")
        mask = np.full((3000,), fill, np.uint8)
        dt_ = to_device(state, t)
        dt_.maskedFill(to_device(state, mask), 1)
        assert_bit_equal(dt_.numpy(), mo.masked_fill(t, mask, 1), f"{kind} maskedFill mask={fill}")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_masked_select_and_copy(state, kind):
    r = rng("msel", kind)
    cases = [((10007,), "contiguous", "contiguous", 0.5), ((64, 130), "transposed", "contiguous", 0.1),
             ((70, 66), "contiguous", "transposed", 0.9), ((5, 6, 7), "strided", "holes", 0.5),
             ((9000,), "offset", "offset", 0.02), ((4096 * 3 + 5,), "contiguous", "contiguous", 1.0)]
    for shape, ls, lm, density in cases:
        src = make_view(r, kind, shape, ls)
        mask = make_view(r, "Byte", shape, lm)
        mask[...] = (r.uniform(size=shape) < density).astype(np.uint8)
        dsrc, dm = to_device(state, src), to_device(state, mask)
        out = thc.Tensor.new(state, kind)
        out.maskedSelect(dsrc, dm)
        want = mo.masked_select(src, mask)
        assert out.sizes == [want.size]
        assert_bit_equal(out.numpy(), want, f"{kind} maskedSelect {ls}/{lm}")
        # maskedCopy: the selected positions of t receive consecutive elements of a (strided) source
        t = make_view(r, kind, shape, ls)
        packed = make_view(r, kind, (int(mask.sum()) + 3,), "strided")
        dt_, dp = to_device(state, t), to_device(state, packed)
        dt_.maskedCopy(dm, dp)
        assert_bit_equal(dt_.numpy(), mo.masked_copy(t, mask, packed), f"{kind} maskedCopy {ls}/{lm}")


def test_masked_edge_cases(state):
    r = rng("medge")
    src = make_view(r, "Float", (1000,), "contiguous")
    dsrc = to_device(state, src)
    zero = to_device(state, np.zeros(1000, np.uint8))
    out = thc.Tensor.new(state, "Float")
    out.maskedSelect(dsrc, zero)
    assert out.nelement == 0
    # maskedCopy with too few source elements is an argument error
    ones = to_device(state, np.ones(1000, np.uint8))
    with pytest.raises(thc.THCError, match="source nElements"):
        dsrc.maskedCopy(ones, to_device(state, np.zeros(999, np.float32)))
    with pytest.raises(thc.THCError, match="sizes do not match"):
        out.maskedSelect(dsrc, to_device(state, np.ones(999, np.uint8)))
    with pytest.raises(thc.THCError, match="same number of elements"):
        dsrc.maskedCopy(to_device(state, np.ones(10, np.uint8)), dsrc)
    # two selects in a row on different masks must not reuse each other's positions
    m1 = (r.uniform(size=1000) < 0.3).astype(np.uint8)
    m2 = (r.uniform(size=1000) < 0.7).astype(np.uint8)
    for m in (m1, m2, m1):
        out.maskedSelect(dsrc, to_device(state, m))
        assert_bit_equal(out.numpy(), mo.masked_select(src, m), "alternating masks")


def test_masked_select_large(state):
    """2^26 elements: many tiles, the scan of tile counts runs over 16384 entries."""
    r = rng("mlarge")
    n = 1 << 26
    src = r.standard_normal(n).astype(np.float32)
    mask = (src > 0.25).astype(np.uint8)
    dsrc, dm = to_device(state, src), to_device(state, mask)
    out = thc.Tensor.new(state, "Float")
    out.maskedSelect(dsrc, dm)
    assert_bit_equal(out.numpy(), mo.masked_select(src, mask), "large maskedSelect")
    bytes_out = thc.Tensor.new(state, "Byte")
    dsrc.call("gtValue", bytes_out, dsrc, 0.25)
    assert_bit_equal(bytes_out.numpy(), mask, "large gtValue")
    dsrc.maskedFill(dm, 0.0)
    assert_bit_equal(dsrc.numpy(), mo.masked_fill(src, mask, 0.0), "large maskedFill")


@pytest.mark.parametrize("n", [4096 * 1024, 4096 * 1024 + 1, 4096 * 2500 + 77])
def test_masked_select_many_tiles(state, n):
    """More than 1024 tiles of 4096 elements: the tile offsets are scanned by several CTAs, each
    adding up the counts before its span.  Densities differ from region to region so that a wrong
    carry shows."""
    r = rng("msel tiles", str(n))
    src = r.integers(-2**31, 2**31 - 1, size=n, dtype=np.int64).astype(np.int32)
    density = np.repeat(r.uniform(0, 1, size=n // 65536 + 1), 65536)[:n]
    mask = (r.uniform(size=n) < density).astype(np.uint8)
    dsrc, dm = to_device(state, src), to_device(state, mask)
    out = thc.Tensor.new(state, "Int")
    out.maskedSelect(dsrc, dm)
    want = src[mask != 0]
    assert out.sizes == [want.size]
    assert_bit_equal(out.numpy(), want, f"maskedSelect over {n} elements")
    t = np.zeros(n, np.int32)
    dt_ = to_device(state, t)
    dt_.maskedCopy(dm, to_device(state, want))
    back = dt_.numpy()
    assert_bit_equal(back[mask != 0], want, "maskedCopy puts the selected elements back")
    assert not back[mask == 0].any()


@pytest.mark.parametrize("kind", ["Float", "Int", "Half"])
def test_masked_calls_with_the_mask_in_a_cpu_tensor(state, kind):
    """maskedFillByte / maskedCopyByte / maskedSelectByte: the mask is a CPU ByteTensor
    (lib/THC/generic/THCTensorMasked.h: the ...Byte variants), here a transposed view of one."""
    r = rng("masked-byte", kind)
    shape = (37, 53)
    src = make_view(r, kind, shape, "contiguous")
    mask = (r.uniform(size=shape[::-1]) < 0.4).astype(np.uint8).T      # transposed CPU view
    cm = thc.CpuTensor(mask)
    t = to_device(state, src)
    t.maskedFillByte(cm, 3)
    assert_bit_equal(t.numpy(), mo.masked_fill(src, mask, 3), f"{kind} maskedFillByte")
    out = thc.Tensor.new(state, kind)
    out.maskedSelectByte(to_device(state, src), cm)
    assert_bit_equal(out.numpy(), mo.masked_select(src, mask), f"{kind} maskedSelectByte")
    packed = make_view(r, kind, (int(mask.sum()),), "contiguous")
    t = to_device(state, src)
    t.maskedCopyByte(cm, to_device(state, packed))
    assert_bit_equal(t.numpy(), mo.masked_copy(src, mask, packed), f"{kind} maskedCopyByte")


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_nonzero(state, kind):
    """nonzero (lib/THC/generic/THCTensorMath.cu:262-356; cutorch's test: test/test.lua:2260-2300): rows of
    1-based coordinates of the non-zero elements in logical order, for 1-D to 4-D strided inputs, an
    all-zero input and one with more than a tile of elements."""
    r = rng("nonzero", kind)
    for shape, layout in [((1000,), "contiguous"), ((37, 53), "transposed"), ((6, 7, 8), "permuted"), ((3, 5, 4, 6), "holes"),
                          ((70, 300), "strided")]:
        x = make_view(r, kind, shape, layout)
        x[...] = (r.integers(0, 3, size=shape) * (r.uniform(size=shape) < 0.4)).astype(x.dtype)
        dx = to_device(state, x)
        out = thc.Tensor.new(state, "Long")
        dx.call("nonzero", out, dx)
        want = np.argwhere(np.asarray(x) != 0).astype(np.int64) + 1
        assert out.sizes == [want.shape[0], len(shape)]
        assert_bit_equal(out.numpy(), want, f"{kind} nonzero {shape} {layout}")
    zero = to_device(state, np.zeros((4, 5), NP_OF_KIND[kind]))
    out = thc.Tensor.new(state, "Long")
    zero.call("nonzero", out, zero)
    assert out.sizes == [0, 2]


@pytest.mark.parametrize("shift", [1, 3, 8, 16])
def test_mask_coords_of_a_mask_that_starts_off_a_16_byte_boundary(state, shift):
    """A narrowed ByteTensor is a dense mask whose first byte sits anywhere: the coordinates kernel must
    read it byte by byte then (its 16-byte loads need an aligned base).  Also: an output too short for
    the counted mask is refused instead of overrun."""
    import ctypes as C
    from cutorch_b200 import _lib
    lib = _lib.load_library()
    r = rng("coords-shift", shift)
    n = 3 * 4096 + 123
    base = (r.uniform(size=n + shift) < 0.3).astype(np.uint8)
    dbase = to_device(state, base)
    dmask = dbase.narrow(0, shift, n)
    assert dmask.data_ptr % 16 == shift % 16
    mask = base[shift:]
    want = np.argwhere(mask.reshape(-1) != 0).astype(np.int64) + 1
    ctx, stream = C.c_void_p(state.context), C.c_void_p(state.stream)
    P, vp = C.POINTER, C.c_void_p
    lib.thcb200_masked_count.argtypes = [vp, P(_lib.TensorDesc), P(C.c_int64), vp]
    lib.thcb200_mask_coords.argtypes = [vp, P(_lib.TensorDesc), P(_lib.TensorDesc), P(C.c_int64), C.c_int, vp, C.c_int]
    dm = dmask.descriptor()
    count = C.c_int64(-1)
    _lib.check(lib.thcb200_masked_count(ctx, C.byref(dm), C.byref(count), stream))
    assert count.value == want.shape[0]
    out = thc.Tensor.new(state, "Long", want.shape[0], 1)
    do = out.descriptor()
    sizes = (C.c_int64 * 1)(n)
    _lib.check(lib.thcb200_mask_coords(ctx, C.byref(do), C.byref(dm), sizes, 1, stream, 2))
    assert_bit_equal(out.numpy(), want, f"coordinates of a mask shifted by {shift}")
    short = thc.Tensor.new(state, "Long", want.shape[0] - 1, 1)
    ds = short.descriptor()
    _lib.check(lib.thcb200_masked_count(ctx, C.byref(dm), C.byref(count), stream))
    rc = lib.thcb200_mask_coords(ctx, C.byref(ds), C.byref(dm), sizes, 1, stream, 2)
    assert rc == -3, rc   # THCB200_ERR_SIZE
