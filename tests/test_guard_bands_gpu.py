"""Every kernel family between guard bands.

compute-sanitizer is not available for these runs, so out-of-bounds WRITES are looked for
directly: each operand of a call lives inside a larger device buffer whose every other byte holds
a sentinel -- 4 KiB in front of the operand, 4 KiB behind it, and the gaps a strided view leaves
between its elements.  After the call the whole buffer comes back to the host: the operand's
elements must equal the oracle's result and every other byte must still be the sentinel (inputs:
the whole buffer unchanged).  Reads that stray stay inside the big buffer, so nothing here can
fault.  The shapes are the edges of each kernel: odd lengths, bases 1 to 7 elements off a 16-byte
boundary, windows cut out of larger tensors, odd pitches, tile remainders, split lengths that do
not divide the reduced dim, 1-byte element types.

cutorch keeps bounds assertions alive in its kernels unless built with -DNDEBUG
(lib/THC/THCTensorInfo.cuh:228-278, lib/THC/CMakeLists.txt:7-16); this file is the counterpart for
kernels that peel heads and tails, walk windows and stage tiles."""
import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import OP, PRE, RED
from oracle import index_oracle as io
from oracle import matrix_oracle as xo
from oracle import mixed_oracle as mo
from common import NP_OF_KIND, assert_reduction_close, make_view, random_array, rng, to_device

pytestmark = pytest.mark.gpu

BAND = 4096
SENTINEL = 0xA5


class Guarded:
    """A numpy view (any non-negative strides) placed on the device between two sentinel bands, its
    first element `shift` elements past a 16-byte boundary."""

    def __init__(self, state, view: np.ndarray, shift: int = 0):
        self.state = state
        self.dtype, self.shape, self.strides = view.dtype, view.shape, view.strides
        item = view.dtype.itemsize
        assert all(s >= 0 for s in view.strides)
        span = (sum((n - 1) * s for n, s in zip(view.shape, view.strides)) + item) if view.size else item
        self.start = BAND + shift * item
        self.span = span
        host = np.full(self.start + span + BAND, SENTINEL, np.uint8)
        if view.size:
            # only the view's own elements travel; the gaps between them keep the sentinel
            self._on(host)[...] = view
        self.before = host
        self.buf = to_device(state, host)
        kind = thc.KIND_OF_DTYPE[view.dtype]
        self.t = thc.Tensor.wrap(state, kind, self.buf.data_ptr + self.start, view.shape, [s // item for s in view.strides])
        self.t._owner = self.buf

    def _on(self, raw: np.ndarray) -> np.ndarray:
        """The view's elements inside a host copy of the buffer."""
        return np.ndarray(self.shape, self.dtype, buffer=raw.data, offset=self.start, strides=self.strides)

    def check_untouched(self, what):
        after = self.buf.numpy()
        bad = np.flatnonzero(after != self.before)
        assert bad.size == 0, f"{what}: an input changed at byte {bad[0] - self.start} relative to its first element"

    def check_result(self, want: np.ndarray, what, rel=None, abs_sum=None):
        after = self.buf.numpy()
        got = np.array(self._on(after), copy=True, order="C")
        if rel is None:
            same = got.view(np.uint8) == np.ascontiguousarray(want).view(np.uint8) if got.size else np.ones(0, bool)
            if not np.all(same):
                k = np.argwhere(got != want)
                first = tuple(k[0]) if len(k) else "(NaN payloads)"
                raise AssertionError(f"{what}: result differs from the oracle, first at {first}")
        else:
            assert_reduction_close(got, want, rel, abs_sum, what)
        # everything that is not an element of the view: bands and gaps
        self._on(after)[...] = np.zeros((), self.dtype)
        ref = self.before.copy()
        self._on(ref)[...] = np.zeros((), self.dtype)
        bad = np.flatnonzero(after != ref)
        if bad.size:
            where = "in front of" if bad[0] < self.start else ("behind" if bad[0] >= self.start + self.span else "in a gap of")
            raise AssertionError(f"{what}: {bad.size} bytes written {where} the output (first at byte {bad[0] - self.start} from its first element)")


def run(state, what, call, outs, ins, shift=0):
    """outs: list of (initial view, expected array[, rel, abs_sum]); ins: list of views.  `call` gets
    the guarded tensors (outputs first) and runs the library call."""
    g_out = [Guarded(state, o[0], shift) for o in outs]
    g_in = [Guarded(state, v, shift) for v in ins]
    call(*[g.t for g in g_out], *[g.t for g in g_in])
    state.synchronize()
    for g, o in zip(g_out, outs):
        g.check_result(o[1], what, *(o[2:] if len(o) > 2 else ()))
    for g in g_in:
        g.check_untouched(what)


SHIFTS = [0, 1, 3, 7]


# ---- pointwise apply: contiguous vectors, rows, tiled transposes, generic walk ----------------
@pytest.mark.parametrize("shift", SHIFTS)
@pytest.mark.parametrize("kind", ["Float", "Byte", "Half", "Double"])
def test_apply_dense_runs(state, oracle, kind, shift):
    r = rng("guard-dense", kind, shift)
    for n in (1, 31, 3 * 8192 + 5, 16384):     # below a vector, tile remainder, whole tiles
        a, b = random_array(r, kind, (n,)), random_array(r, kind, (n,))
        out = np.zeros(n, NP_OF_KIND[kind])
        want = oracle.pointwise(OP["CADD"], out.copy(), [a, b], 2)
        run(state, f"{kind} cadd n={n} shift={shift}", lambda o, x, y: o.cadd(x, 2, y), [(out, want)], [a, b], shift)


@pytest.mark.parametrize("shift", [0, 1, 5])
def test_apply_rows_and_windows(state, oracle, shift):
    r = rng("guard-rows", shift)
    cases = [make_view(r, "Float", (37, 131), "holes"),            # pitch 134: rows start at every alignment
             make_view(r, "Float", (5, 7, 33), "offset"),          # a window of a larger tensor
             make_view(r, "Short", (9, 250), "holes"),
             make_view(r, "Float", (6, 40), "strided")]            # every second element: generic walk
    for a in cases:
        kind = thc.KIND_OF_DTYPE[a.dtype]
        b = make_view(r, kind, a.shape, "holes")
        out = make_view(r, kind, a.shape, "offset")
        want = oracle.pointwise(OP["MUL"], np.zeros(a.shape, a.dtype), [a, b])
        run(state, f"cmul {a.shape} {a.strides} shift={shift}", lambda o, x, y: o.cmul(x, y), [(out, want)], [a, b], shift)


@pytest.mark.parametrize("shift", [0, 2])
def test_apply_tiled_transposes(state, oracle, shift):
    r = rng("guard-tiled", shift)
    for shape in [(65, 70), (3, 50, 70), (257, 63), (64, 64)]:      # tile remainders in both tile dims
        a = make_view(r, "Float", shape, "transposed")
        b = make_view(r, "Float", shape, "contiguous")
        out = np.zeros(shape, np.float32)
        want = oracle.pointwise(OP["ADDCMUL"], np.zeros(shape, np.float32), [b, a, b], 0.5)
        run(state, f"addcmul transposed {shape} shift={shift}", lambda o, x, y: o.addcmul(y, 0.5, x, y), [(out, want)], [a, b], shift)
        # the transposed side as the output
        outT = make_view(r, "Float", shape, "transposed")
        want = oracle.pointwise(OP["ADD_S"], np.zeros(shape, np.float32), [b], 1.5)
        run(state, f"add into transposed {shape} shift={shift}", lambda o, x: o.add(x, 1.5), [(outT, want)], [b], shift)


def test_apply_generic_shapes_that_only_share_their_element_count(state, oracle):
    r = rng("guard-generic")
    a = make_view(r, "Int", (12, 35), "permuted")
    b = make_view(r, "Int", (420,), "strided")
    out = make_view(r, "Int", (12, 35), "holes")      # the output takes the first operand's shape (resizeAs)
    want = oracle.pointwise(OP["ADD"], np.zeros((12, 35), np.int32), [np.ascontiguousarray(a), b.reshape(12, 35)])
    run(state, "cadd over three shapes", lambda o, x, y: o.cadd(x, 1, y), [(out, want)], [a, b])


def test_converting_copy(state, oracle):
    r = rng("guard-convert")
    for shape, layout in [((1001,), "contiguous"), ((33, 65), "transposed"), ((7, 9, 11), "holes")]:
        src = make_view(r, "Float", shape, layout)
        out = make_view(r, "Half", shape, "offset")
        want = oracle.convert(np.zeros(shape, np.float16), src)
        run(state, f"float -> half {shape} {layout}", lambda o, x: o.copy_from(x), [(out, want)], [src], 1)


# ---- reductions ------------------------------------------------------------------------------
def _sum_case(state, oracle, x, dim, shift, what):
    shape = list(x.shape)
    shape[dim] = 1
    out = np.zeros(shape, x.dtype)
    want = oracle.reduce_dim(RED["SUM"], PRE["IDENTITY"], 0.0, x, dim)
    exact = x.dtype.kind != "f"
    extra = () if exact else (1e-3 if x.dtype == np.float16 else 1e-5, np.abs(x.astype(np.float64)).sum(axis=dim, keepdims=True))
    run(state, what + " sum", lambda o, t: o.sum(t, dim, 1), [(out, want) + extra], [x], shift)
    v, i = np.zeros(shape, x.dtype), np.zeros(shape, np.int64)
    wv, wi = oracle.reduce_dim(RED["MAX"], PRE["IDENTITY"], 0.0, x, dim, with_index=True)
    run(state, what + " max", lambda ov, oi, t: ov.max(oi, t, dim, 1), [(v, wv), (i, wi)], [x], shift)


@pytest.mark.parametrize("shift", [0, 1, 3])
def test_reduce_rows(state, oracle, shift):
    r = rng("guard-redrow", shift)
    for kind, shape, layout in [("Float", (37, 1003), "contiguous"),     # a warp per row, odd length
                                ("Float", (3, 70001), "contiguous"),     # a CTA per (row, split); 70001 is no multiple of the split
                                ("Half", (20, 515), "holes"), ("Byte", (11, 300), "contiguous"),
                                ("Double", (5, 6, 129), "offset"), ("Int", (20, 7), "contiguous")]:   # K < 64: a thread per slice
        x = make_view(r, kind, shape, layout)
        _sum_case(state, oracle, x, len(shape) - 1, shift, f"{kind} {shape} {layout} last dim shift={shift}")


@pytest.mark.parametrize("shift", [0, 1, 4])
def test_reduce_columns(state, oracle, shift):
    r = rng("guard-redcol", shift)
    for kind, shape, layout in [("Float", (3001, 96), "contiguous"),     # split along K, 3001 rows
                                ("Float", (515, 33), "contiguous"),      # odd narrow width: one column per lane
                                ("Float", (700, 131), "contiguous"),
                                ("Int", (300, 257), "holes"), ("Long", (200, 75), "contiguous"),
                                ("Float", (4000, 125), "contiguous"),    # the same with the rows split over CTAs
                                ("Byte", (300, 64), "contiguous"),       # 4-byte column words
                                ("Half", (1000, 72), "holes"), ("Short", (64, 5, 40), "contiguous"),
                                ("Double", (70, 130), "offset")]:
        x = make_view(r, kind, shape, layout)
        _sum_case(state, oracle, x, 0, shift, f"{kind} {shape} {layout} dim 0 shift={shift}")


@pytest.mark.parametrize("shift", [0, 1, 5])
def test_reduce_all_layouts(state, oracle, shift):
    r = rng("guard-redall", shift)
    for kind, shape, layout in [("Float", (100003,), "contiguous"), ("Float", (16, 20, 50), "offset"),
                                ("Float", (301, 77), "transposed"), ("Int", (9, 1000), "holes"), ("Byte", (5001,), "strided")]:
        x = make_view(r, kind, shape, layout)
        g = Guarded(state, x, shift)
        got = g.t.sumall()
        want = oracle.reduce_all(RED["SUM"], PRE["IDENTITY"], 0.0, x)
        if x.dtype.kind == "f":
            assert_reduction_close(got, want, 1e-5, np.abs(x.astype(np.float64)).sum(), f"sumall {shape} {layout}")
        else:
            assert int(got) == int(want)
        g.check_untouched(f"sumall {shape} {layout} shift={shift}")


# ---- scans -----------------------------------------------------------------------------------
@pytest.mark.parametrize("shift", [0, 1, 3])
def test_scans(state, oracle, shift):
    r = rng("guard-scan", shift)
    for kind, shape, dim, layout in [("Float", (5, 2003), 1, "contiguous"), ("Float", ((1 << 20) + 3,), 0, "contiguous"),   # chunked 1-D
                                     ("Float", (3000, 70), 0, "contiguous"), ("Int", (5000, 40), 0, "contiguous"),
                                     ("Double", (40, 50), 0, "transposed"), ("Short", (7, 300), 1, "holes")]:
        x = make_view(r, kind, shape, layout)
        if x.dtype.kind == "f":
            x[...] = (r.integers(-8, 9, size=shape) / 4).astype(x.dtype)     # exact partial sums
        out = make_view(r, kind, shape, layout)
        want = oracle.scan_dim(False, x, dim)
        run(state, f"cumsum {kind} {shape} dim {dim} {layout} shift={shift}", lambda o, t: o.cumsum(t, dim), [(out, want)], [x], shift)


# ---- comparisons into bytes, masks ------------------------------------------------------------
@pytest.mark.parametrize("shift", [0, 1, 7])
def test_compare_and_masks(state, shift):
    r = rng("guard-mask", shift)
    for n in (5, 4099, 3 * 4096 + 17):
        x = random_array(r, "Float", (n,))
        m = np.zeros(n, np.uint8)
        run(state, f"gtValue n={n} shift={shift}", lambda o, t: t.call("gtValue", o, t, 0.5), [(m, mo.compare("gt", x, 0.5))], [x], shift)
        mask = (r.uniform(size=n) < 0.4).astype(np.uint8)
        run(state, f"maskedFill n={n} shift={shift}", lambda o, mk: o.maskedFill(mk, 3.0), [(x.copy(), mo.masked_fill(x, mask, 3.0))], [mask], shift)
        sel = mo.masked_select(x, mask)
        if sel.size:
            run(state, f"maskedSelect n={n} shift={shift}", lambda o, t, mk: o.maskedSelect(t, mk), [(np.zeros(sel.size, np.float32), sel)], [x, mask], shift)
            packed = random_array(r, "Float", (sel.size,))
            run(state, f"maskedCopy n={n} shift={shift}", lambda o, mk, p: o.maskedCopy(mk, p), [(x.copy(), mo.masked_copy(x, mask, packed))],
                [mask, packed], shift)
    # strided operands
    x = make_view(r, "Int", (33, 65), "transposed")
    mask = (r.uniform(size=(33, 65)) < 0.5).astype(np.uint8)
    run(state, "maskedFill transposed", lambda o, mk: o.maskedFill(mk, 9), [(x, mo.masked_fill(np.ascontiguousarray(x), mask, 9))], [mask], shift)


# ---- indexed moves ---------------------------------------------------------------------------
def test_indexed_moves(state):
    r = rng("guard-index")
    src = make_view(r, "Float", (50, 36), "contiguous")
    idx = r.integers(1, 51, size=23).astype(np.int64)
    run(state, "indexSelect rows", lambda o, s, i: o.indexSelect(s, 0, i), [(np.zeros((23, 36), np.float32), io.index_select(src, 0, idx))], [src, idx], 1)
    idc = r.integers(1, 37, size=10).astype(np.int64)
    run(state, "indexSelect columns", lambda o, s, i: o.indexSelect(s, 1, i), [(np.zeros((50, 10), np.float32), io.index_select(src, 1, idc))], [src, idc], 3)
    gi = r.integers(1, 37, size=(50, 36)).astype(np.int64)
    run(state, "gather dim 1", lambda o, s, i: o.gather(s, 1, i), [(np.zeros((50, 36), np.float32), io.gather(src, 1, gi))], [src, gi])
    gi2 = r.integers(1, 51, size=(7, 33)).astype(np.int64)          # an odd width: the per-element walk
    src2 = make_view(r, "Float", (50, 33), "holes")
    run(state, "gather dim 0", lambda o, s, i: o.gather(s, 0, i), [(np.zeros((7, 33), np.float32), io.gather(np.ascontiguousarray(src2), 0, gi2))], [src2, gi2], 1)
    perm = np.stack([r.permutation(36) + 1 for _ in range(50)]).astype(np.int64)   # no duplicates: scatter is defined
    dst = make_view(r, "Float", (50, 36), "contiguous")
    run(state, "scatter dim 1", lambda o, i, s: o.scatter(1, i, s), [(dst, io.scatter(dst.copy(), 1, perm, src))], [perm, src], 2)


# ---- triangles, renorm -----------------------------------------------------------------------
@pytest.mark.parametrize("shift", [0, 1])
def test_tri_and_renorm(state, shift):
    r = rng("guard-tri", shift)
    for shape, layout in [((67, 45), "contiguous"), ((40, 132), "holes"), ((33, 33), "transposed")]:
        x = make_view(r, "Float", shape, layout)
        out = make_view(r, "Float", shape, "contiguous")
        run(state, f"tril {shape} {layout}", lambda o, t: o.tril(t, 1), [(out, xo.tri(np.ascontiguousarray(x), 1, False))], [x], shift)
        run(state, f"triu {shape} {layout}", lambda o, t: o.triu(t, -2), [(out, xo.tri(np.ascontiguousarray(x), -2, True))], [x], shift)
    for shape, dim in [((50, 36), 0), ((50, 33), 1), ((300, 8), 0)]:
        x = make_view(r, "Float", shape, "contiguous")
        out = np.zeros(shape, np.float32)
        want = xo.renorm(x, 2.0, dim, 1.0)
        run(state, f"renorm {shape} dim {dim}", lambda o, t: o.renorm(t, 2, dim, 1.0), [(out, want, 1e-5, np.abs(x) + 1.0)], [x], shift)
