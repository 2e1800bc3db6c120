"""tril / triu and renorm through the THC C API against oracle/matrix_oracle.py.

cutorch's tests: test/test.lua:1411-1452 (tril, triu with random k on random matrices and their
transposes), :1399-1409 (renorm over each dim of 2-D..4-D tensors).  tril / triu are bit-exact
(every output is an input element or 0); renorm is held to the reduction tolerance."""
import numpy as np
import pytest

from cutorch_b200 import thc
from oracle import matrix_oracle as mx
from common import ALL_KINDS, FP_KINDS, NP_OF_KIND, assert_bit_equal, make_view, rng, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_tril_triu(state, kind):
    r = rng("tri", kind)
    for shape, layout in [((37, 53), "contiguous"), ((53, 37), "transposed"), ((64, 1100), "holes"), ((1100, 9), "offset"),
                          ((1, 1), "contiguous"), ((130, 130), "strided")]:
        x = make_view(r, kind, shape, layout)
        if x.dtype.kind != "f":
            x[...] = r.integers(1, 9, size=shape).astype(x.dtype)
        dx = to_device(state, x)
        for k in (0, 1, -1, 5, -7, shape[1] + 3, -shape[0] - 3):
            for name, upper in (("tril", False), ("triu", True)):
                out = thc.Tensor.new(state, kind)
                getattr(out, name)(dx, k)
                assert out.sizes == list(shape)
                assert_bit_equal(out.numpy(), mx.tri(x, k, upper), f"{kind} {name} k={k} {shape} {layout}")
        # in place, and into a transposed output
        y = to_device(state, x)
        y.tril(y, 2)
        assert_bit_equal(y.numpy(), mx.tri(x, 2, False), f"{kind} tril in place {layout}")
        z = to_device(state, make_view(r, kind, shape, "transposed"))
        z.triu(dx, -1)
        assert_bit_equal(z.numpy(), mx.tri(x, -1, True), f"{kind} triu into transposed output {layout}")
    with pytest.raises(thc.THCError, match="expected a matrix"):
        thc.Tensor.new(state, kind).tril(to_device(state, make_view(r, kind, (3, 4, 5), "contiguous")), 0)


REL = {"Half": 2e-3, "Float": 1e-5, "Double": 1e-12}


@pytest.mark.parametrize("kind", FP_KINDS)
def test_renorm(state, kind):
    r = rng("renorm", kind)
    cases = [((200, 64), "contiguous"), ((64, 200), "transposed"), ((7, 30, 11), "contiguous"), ((5, 6, 7, 8), "permuted"),
             ((300, 33), "holes"), ((2, 5000), "contiguous")]
    for shape, layout in cases:
        x = make_view(r, kind, shape, layout)
        x[...] = (r.standard_normal(shape) * r.uniform(0.2, 3.0, size=shape[:1] + (1,) * (len(shape) - 1))).astype(x.dtype)
        dx = to_device(state, x)
        for dim in range(len(shape)):
            for p in (1, 2, 3, 2.5):
                # a threshold that some slices exceed and some do not
                moved = np.moveaxis(x.astype(np.float64), dim, 0).reshape(shape[dim], -1)
                norms = (np.abs(moved) ** p).sum(axis=1) ** (1.0 / p)
                maxnorm = float(x.dtype.type(float(np.median(norms)) * 1.003))   # as the `real` argument carries it
                want = mx.renorm(x, p, dim, maxnorm)
                out = thc.Tensor.new(state, kind)
                out.renorm(dx, p, dim, maxnorm)
                got = out.numpy()
                assert out.sizes == list(shape)
                tol = REL[kind] * np.maximum(np.abs(want.astype(np.float64)), 1e-30)
                bad = np.abs(got.astype(np.float64) - want.astype(np.float64)) > tol
                assert not bad.any(), f"{kind} renorm p={p} dim={dim} {shape} {layout}: {bad.sum()} off, first {np.argwhere(bad)[0]}"
                # slices below the threshold are copied bit for bit
                keep = np.moveaxis(np.broadcast_to(np.expand_dims(norms <= maxnorm * 0.999, tuple(range(1, len(shape)))),
                                                   np.moveaxis(x, dim, 0).shape), 0, dim)
                assert_bit_equal(got[keep], np.asarray(x)[keep], "slices under the threshold")
        y = to_device(state, x)
        y.renorm(y, 2, 0, 1.0)
        want = mx.renorm(x, 2, 0, 1.0)
        assert np.allclose(y.numpy().astype(np.float64), want.astype(np.float64), rtol=REL[kind], atol=0), "in place"
    with pytest.raises(thc.THCError, match="at least 2 dimensions"):
        thc.Tensor.new(state, kind).renorm(to_device(state, make_view(r, kind, (10,), "contiguous")), 2, 0, 1.0)
    with pytest.raises(thc.THCError, match="non-positive-norm"):
        thc.Tensor.new(state, kind).renorm(dx, -1, 0, 1.0)


@pytest.mark.parametrize("kind", FP_KINDS)
def test_renorm_one_pass_and_composed_forms_agree(state, kind):
    """Slices that are short dense runs take the one-pass kernel (a warp or a CTA keeps the slice in
    registers), every other layout the composed form; both against the oracle over the slice
    lengths where the kernel changes shape (vectors per thread, warp or CTA per slice)."""
    from cutorch_b200 import _lib
    lib = _lib.load_library()
    r = rng("renorm forms", kind)
    elems = {"Half": 8, "Float": 4, "Double": 2}[kind]   # elements per 16-byte vector
    for nvec in (1, 3, 32, 33, 64, 100, 128, 129, 256, 257, 512, 700, 1024, 1025, 2048, 2049):
        rows, length = 37, nvec * elems
        x = (r.standard_normal((rows, length)) * r.uniform(0.2, 3.0, size=(rows, 1))).astype(NP_OF_KIND[kind])
        dx = to_device(state, x)
        for p in (1, 2, 3):
            norms = (np.abs(x.astype(np.float64)) ** p).sum(axis=1) ** (1.0 / p)
            maxnorm = float(x.dtype.type(float(np.median(norms)) * 1.003))
            out = thc.Tensor.new(state, kind)
            out.renorm(dx, p, 0, maxnorm)
            assert (lib.thcb200_last_plan() == b"renorm_rows") == (nvec <= 2048), (nvec, lib.thcb200_last_plan())
            want = mx.renorm(x, p, 0, maxnorm)
            got = out.numpy()
            tol = REL[kind] * np.maximum(np.abs(want.astype(np.float64)), 1e-30)
            assert (np.abs(got.astype(np.float64) - want.astype(np.float64)) <= tol).all(), f"{kind} renorm rows of {length}, p={p}"
            keep = norms <= maxnorm * 0.999
            assert_bit_equal(got[keep], x[keep], "slices under the threshold")
    # an odd slice length, and slices along the inner dim of a contiguous matrix: composed form
    x = r.standard_normal((64, 255)).astype(NP_OF_KIND[kind])
    dx = to_device(state, x)
    for dim in (0, 1):
        out = thc.Tensor.new(state, kind)
        out.renorm(dx, 2, dim, 1.0)
        assert lib.thcb200_last_plan() != b"renorm_rows"
        want = mx.renorm(x, 2, dim, 1.0)
        assert np.allclose(out.numpy().astype(np.float64), want.astype(np.float64), rtol=REL[kind], atol=0)
    # the columns of a transposed matrix are dense runs: one pass again, in place
    base = r.standard_normal((48, 512)).astype(NP_OF_KIND[kind])
    dt = to_device(state, base)
    view = dt.transpose(0, 1)
    view.renorm(view, 2, 1, 1.0)
    assert lib.thcb200_last_plan() == b"renorm_rows"
    want = mx.renorm(base.T, 2, 1, 1.0)
    assert np.allclose(view.numpy().astype(np.float64), want.astype(np.float64), rtol=REL[kind], atol=0)


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_zeros_ones_reshape_diag_eye_trace(state, kind):
    """The construction calls that are thin callers of fill / copy / sumall
    (lib/THC/generic/THCTensorMath.cu:36-82,358-422; cutorch's tests: test/test.lua:236-330 zeros, ones,
    reshape; :3000-3050 diag, eye, trace)."""
    r = rng("construct", kind)
    dt = NP_OF_KIND[kind]
    t = thc.Tensor.new(state, kind)
    t.zeros((3, 5, 2))
    assert t.sizes == [3, 5, 2] and not t.numpy().any()
    t.ones((4, 7))
    assert_bit_equal(t.numpy(), np.ones((4, 7), dt), "ones")
    src = make_view(r, kind, (6, 10), "transposed")
    if src.dtype.kind != "f":
        src[...] = r.integers(0, 9, size=src.shape).astype(dt)
    else:
        src[...] = (r.integers(-16, 17, size=src.shape) / 4).astype(dt)
    dsrc = to_device(state, src)
    t.onesLike(dsrc)
    assert_bit_equal(t.numpy(), np.ones((6, 10), dt), "onesLike")
    t.zerosLike(dsrc)
    assert t.sizes == [6, 10] and not t.numpy().any()
    t.reshape(dsrc, (4, 15))
    assert_bit_equal(t.numpy(), np.asarray(src).reshape(4, 15), "reshape walks the source in logical order")
    assert dsrc.numel() == 60
    for k in (0, 2, -3, 9, -5, 12):
        d = thc.Tensor.new(state, kind)
        d.diag(dsrc, k)
        assert_bit_equal(d.numpy(), np.diag(np.asarray(src), k), f"diag of a matrix, k={k}")
    vec = np.asarray(src)[2].copy()
    dv = to_device(state, vec)
    for k in (0, 3, -2):
        d = thc.Tensor.new(state, kind)
        d.diag(dv, k)
        assert_bit_equal(d.numpy(), np.diag(vec, k), f"diag of a vector, k={k}")
    dv.diag(dv, 1)                                   # in place: the vector becomes the matrix
    assert_bit_equal(dv.numpy(), np.diag(vec, 1), "diag in place")
    e = thc.Tensor.new(state, kind)
    e.eye(5, 8)
    assert_bit_equal(e.numpy(), np.eye(5, 8, dtype=dt), "eye")
    e.eye(6, 0)
    assert_bit_equal(e.numpy(), np.eye(6, dtype=dt), "eye, square by default")
    want = np.trace(np.asarray(src).astype(np.float64 if src.dtype.kind == "f" else np.int64))
    assert float(dsrc.trace()) == float(want)
    with pytest.raises(thc.THCError, match="expected a matrix"):
        to_device(state, vec).trace()
    with pytest.raises(thc.THCError, match="matrix or a vector"):
        thc.Tensor.new(state, kind).diag(to_device(state, make_view(r, kind, (2, 3, 4), "contiguous")), 0)


@pytest.mark.parametrize("kind", ["Byte", "Float", "Half", "Long"])
def test_cat(state, kind):
    """cat / catArray (lib/THC/generic/THCTensorMath.cu:84-260; cutorch's tests: test/test.lua:3250-3330):
    every dim, strided inputs, an empty input, the last dim chosen with -2 (cutorch's -1), an input
    that is the result itself, and the size check."""
    r = rng("cat", kind)
    dt = NP_OF_KIND[kind]

    def rand(shape, layout="contiguous"):
        x = make_view(r, kind, shape, layout)
        x[...] = r.integers(0, 9, size=shape).astype(dt)
        return x

    for dim in range(3):
        shapes = []
        for n in (2, 5, 3):
            s = [4, 6, 5]
            s[dim] = n
            shapes.append(tuple(s))
        parts = [rand(shapes[0]), rand(shapes[1], "transposed"), rand(shapes[2], "strided")]
        out = thc.Tensor.new(state, kind)
        out.cat([to_device(state, p) for p in parts], dim)
        assert_bit_equal(out.numpy(), np.concatenate([np.asarray(p) for p in parts], axis=dim), f"{kind} cat dim {dim}")
    a, b = rand((3, 4)), rand((3, 2))
    out = thc.Tensor.new(state, kind)
    out.cat([to_device(state, a), thc.Tensor.new(state, kind), to_device(state, b)], -2)
    assert_bit_equal(out.numpy(), np.concatenate([a, b], axis=1), "empty input skipped, last dim by -2")
    da = to_device(state, a)
    da.cat([da, to_device(state, rand((2, 4)))], 0)
    assert da.sizes == [5, 4] and (da.numpy()[:3] == a).all()
    v1, v2 = rand((4,)), rand((3,))
    out.cat([to_device(state, v1), to_device(state, v2)], 0)
    assert_bit_equal(out.numpy(), np.concatenate([v1, v2]), "vectors")
    with pytest.raises(thc.THCError, match="inconsistent tensor sizes"):
        out.cat([to_device(state, a), to_device(state, rand((4, 5)))], 0)
