"""Error behaviour of the THC entry points (THArgCheck / THError in cutorch): bad calls are
reported with cutorch's messages and leave the library usable; nothing faults the GPU."""
import ctypes as C

import numpy as np
import pytest

from cutorch_b200 import _lib, thc
from cutorch_b200._lib import OP, PRE, RED
from common import rng, to_device

pytestmark = pytest.mark.gpu


def test_size_mismatch_is_an_argument_error(state):
    a = to_device(state, np.zeros((4, 5), np.float32))
    b = to_device(state, np.zeros((4, 6), np.float32))
    out = thc.Tensor.new(state, "Float")
    with pytest.raises(thc.THCError, match="sizes do not match"):
        out.cmul(a, b)
    with pytest.raises(thc.THCError, match="sizes do not match"):
        out.cadd(a, 2.0, b)
    with pytest.raises(thc.THCError, match="sizes do not match"):
        out.copy(b) if out.nelement else a.copy(b)
    # still usable afterwards
    out.cmul(a, a)
    assert out.sizes == [4, 5]


def test_ops_undefined_for_a_type(state):
    f = to_device(state, np.ones(8, np.float32))
    with pytest.raises(thc.THCError, match="integer type"):
        f.bitand(f, 3)
    with pytest.raises(thc.THCError, match="integer type"):
        f.cbitxor(f, f)
    h = to_device(state, np.ones(8, np.float16))
    with pytest.raises(thc.THCError, match="not supported for torch.CudaHalfTensor"):
        h.lshift(h, 1)
    i = to_device(state, np.ones(8, np.int32))
    with pytest.raises(AttributeError):
        state.fn("Int", "sigmoid")   # fp-only entry points are not exported for integer types


def test_division_by_zero_scalar(state):
    i = to_device(state, np.arange(8, dtype=np.int32))
    with pytest.raises(thc.THCError, match="divide by zero"):
        i.div(i, 0)


def test_dimension_checks(state):
    m = to_device(state, np.zeros((3, 4), np.float32))
    out = thc.Tensor.new(state, "Float")
    with pytest.raises(thc.THCError, match="dimension out of range"):
        out.sum(m, 2, 1)
    idx = thc.Tensor.new(state, "Long")
    with pytest.raises(thc.THCError, match="dimension out of range"):
        out.max(idx, m, -1, 1)
    with pytest.raises(thc.THCError, match="output must differ"):
        m.sum(m, 0, 1)


def test_more_than_25_dims_is_refused(state):
    """cutorch's 'tensor too large or too many (>25) dimensions' (lib/THC/THCTensorInfo.cuh:14-16)."""
    lib = _lib.load_library()
    d = _lib.TensorDesc()
    d.data = 4096
    d.dtype = _lib.F32
    d.ndim = 26
    rc = lib.thcb200_pointwise(C.c_void_p(state.context), OP["FILL"], C.byref(d), None, None, None, 0, _lib.scalar(1), _lib.scalar(0),
                               C.c_void_p(state.stream))
    assert rc == -2 and b"too many (>25) dimensions" in lib.thcb200_last_error()
    # 25 dims are fine
    shape = [2] * 3 + [1] * 22
    t = thc.Tensor.new(state, "Float", *shape)
    t.fill(2.0)
    assert t.sumall() == 16.0


def test_descriptor_level_argument_checks(state):
    lib = _lib.load_library()
    ctx, st = C.c_void_p(state.context), C.c_void_p(state.stream)
    a = to_device(state, np.zeros(16, np.float32))
    b = to_device(state, np.zeros(16, np.int32))
    da, db = a.descriptor(), b.descriptor()
    z = _lib.scalar(0)
    assert lib.thcb200_pointwise(ctx, OP["MUL"], C.byref(da), C.byref(da), C.byref(db), None, 2, z, z, st) == -1   # mixed dtypes
    assert lib.thcb200_pointwise(ctx, OP["MUL"], C.byref(da), C.byref(da), None, None, 1, z, z, st) == -1          # wrong arity
    assert lib.thcb200_pointwise(ctx, 9999, C.byref(da), C.byref(da), None, None, 1, z, z, st) == -1                # unknown op
    assert lib.thcb200_pointwise(ctx, OP["CBITAND"], C.byref(da), C.byref(da), C.byref(da), None, 2, z, z, st) == -5  # undefined for float
    assert lib.thcb200_reduce_all(ctx, RED["SUM"], PRE["SQUARE"], z, C.byref(db), C.c_void_p(a.data_ptr), st) == -5  # norm on ints
    assert lib.thcb200_reduce_all(ctx, RED["MAX"], PRE["ABS"], z, C.byref(da), C.c_void_p(a.data_ptr), st) == -1     # pre-op only with sum
    out = to_device(state, np.zeros((1, 4), np.float32))
    src = to_device(state, np.zeros((3, 5), np.float32))
    do, ds = out.descriptor(), src.descriptor()
    assert lib.thcb200_reduce_dim(ctx, RED["SUM"], 0, z, C.byref(do), C.byref(ds), 0, st) == -3                      # output shape


def test_empty_tensors_are_no_ops(state):
    e = thc.Tensor.new(state, "Float")
    out = thc.Tensor.new(state, "Float")
    out.cmul(e, e)
    assert out.nelement == 0
    assert e.sumall() == 0.0
    assert e.prodall() == 1.0


def test_scalar_tensor_and_size_one_dims(state, oracle):
    r = rng("ones")
    x = r.standard_normal((1, 1, 1)).astype(np.float32)
    dx = to_device(state, x)
    out = thc.Tensor.new(state, "Float")
    out.add(dx, 2.0)
    assert np.array_equal(out.numpy(), x + np.float32(2.0))
    assert dx.sumall() == float(x.sum())
    v, i = thc.Tensor.new(state, "Float"), thc.Tensor.new(state, "Long")
    v.max(i, dx, 1, 1)
    assert i.numpy().tolist() == [[[1]]]


def test_int64_indexing_path(state):
    """A view whose offsets exceed 32 bits runs the 64-bit index kernels (no 4 GiB tensor needed:
    the view skips through a 5 GiB byte buffer with a huge stride)."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda", 0)
    buf = torch.zeros(5 * 2**30, dtype=torch.uint8, device=dev)
    stride = 2**32 + 16
    buf[0] = 3
    buf[stride] = 4
    # three dims that do not collapse and an inner stride of 2: only the generic walk takes this
    t = thc.Tensor.wrap(state, "Byte", buf.data_ptr(), (2, 3, 2), (stride, 5, 2), storage_elems=5 * 2**30)
    assert _lib.load_library().thcb200_can_use_32bit(C.byref(t.descriptor())) == 0
    out = thc.Tensor.new(state, "Byte")
    out.add(t, 1)
    assert _lib.load_library().thcb200_last_plan() == b"generic64"
    assert out.numpy().reshape(2, 6).tolist() == [[4, 1, 1, 1, 1, 1], [5, 1, 1, 1, 1, 1]]
    t.fill(7)
    torch.cuda.synchronize()
    assert int(buf[stride + 12]) == 7 and int(buf[7]) == 7 and int(buf[8]) == 0 and int(buf[1]) == 0
    buf.zero_()
    buf[0] = 3
    buf[stride] = 4
    # two dims with a dense inner one: the row walk, whose row offsets are 64-bit as well
    t2 = thc.Tensor.wrap(state, "Byte", buf.data_ptr(), (2, 8), (stride, 1), storage_elems=5 * 2**30)
    out.add(t2, 1)
    assert _lib.load_library().thcb200_last_plan() == b"rows_scalar"
    assert out.numpy().tolist() == [[4, 1, 1, 1, 1, 1, 1, 1], [5, 1, 1, 1, 1, 1, 1, 1]]
    del buf
    torch.cuda.empty_cache()


def test_int64_offsets_in_the_mixed_type_scan_and_index_kernels(state):
    """The same huge-stride view through the calls that have their own kernels: comparison into
    bytes, masked fill / select, scans and indexed moves all have to carry 64-bit offsets."""
    torch = pytest.importorskip("torch")
    lib = _lib.load_library()
    dev = torch.device("cuda", 0)
    buf = torch.zeros(5 * 2**30, dtype=torch.uint8, device=dev)
    stride = 2**32 + 16
    host = np.arange(16, dtype=np.uint8).reshape(2, 8) + 1
    buf[0:8] = torch.from_numpy(host[0]).to(dev)
    buf[stride:stride + 8] = torch.from_numpy(host[1]).to(dev)
    t = thc.Tensor.wrap(state, "Byte", buf.data_ptr(), (2, 8), (stride, 1), storage_elems=5 * 2**30)
    # comparison into a dense byte tensor
    out = thc.Tensor.new(state, "Byte")
    t.call("gtValue", out, t, 8)
    assert lib.thcb200_last_plan() == b"compare_strided64"
    assert out.numpy().tolist() == (host > 8).astype(np.uint8).tolist()
    # masked select / fill with the huge view as source / target
    mask = thc.Tensor.from_numpy(state, (host % 2 == 0).astype(np.uint8))
    sel = thc.Tensor.new(state, "Byte")
    sel.maskedSelect(t, mask)
    assert lib.thcb200_last_plan() == b"masked_select64"
    assert sel.numpy().tolist() == host[host % 2 == 0].tolist()
    # scans along both dims (rows are 8 long: the per-slice walk; columns: strided)
    for dim in (0, 1):
        c = thc.Tensor.new(state, "Byte")
        c.cumsum(t, dim)
        assert c.numpy().tolist() == np.cumsum(host, axis=dim, dtype=np.uint64).astype(np.uint8).tolist()
    # indexed moves: pick rows, then write one back through the huge stride
    idx = thc.Tensor.from_numpy(state, np.array([2, 1, 2], np.int64))
    picked = thc.Tensor.new(state, "Byte")
    picked.indexSelect(t, 0, idx)
    assert picked.numpy().tolist() == host[[1, 0, 1]].tolist()
    t.indexFill(0, thc.Tensor.from_numpy(state, np.array([2], np.int64)), 9)
    t.maskedFill(mask, 0)
    torch.cuda.synchronize()
    want_row1 = np.where(host[1] % 2 == 0, 0, 9).astype(np.uint8)
    assert buf[stride:stride + 8].cpu().numpy().tolist() == want_row1.tolist()
    assert buf[0:8].cpu().numpy().tolist() == np.where(host[0] % 2 == 0, 0, host[0]).tolist()
    del buf
    torch.cuda.empty_cache()


def test_state_services(state):
    """The THCState services the path's callers consult: scratch space of the current device and
    the cached device properties (lib/THC/THCGeneral.h.in:146,188-192)."""
    lib = state.lib
    lib.THCState_getCurrentDeviceScratchSpace.restype = C.c_void_p
    lib.THCState_getCurrentDeviceScratchSpace.argtypes = [C.c_void_p]
    lib.THCState_getCurrentDeviceScratchSpaceSize.restype = C.c_size_t
    lib.THCState_getCurrentDeviceScratchSpaceSize.argtypes = [C.c_void_p]
    lib.THCState_getCurrentDeviceProperties.restype = C.c_void_p
    lib.THCState_getCurrentDeviceProperties.argtypes = [C.c_void_p]
    lib.THCState_getPeerToPeerAccess.argtypes = [C.c_void_p, C.c_int, C.c_int]
    p = lib.THCState_getCurrentDeviceScratchSpace(state.ptr)
    n = lib.THCState_getCurrentDeviceScratchSpaceSize(state.ptr)
    assert p and p % 256 == 0 and n >= 128 * 1024
    props = lib.THCState_getCurrentDeviceProperties(state.ptr)
    assert props
    name = C.string_at(props, 256).split(b"\0")[0].decode()     # cudaDeviceProp starts with char name[256]
    assert "NVIDIA" in name or len(name) > 0
    assert lib.THCState_getPeerToPeerAccess(state.ptr, 0, 0) == 1
    assert lib.THCState_getPeerToPeerAccess(state.ptr, 0, 99) == 0
    with pytest.raises(thc.THCError, match="is not a device"):
        state.check()


@pytest.mark.parametrize("kind", ["Byte", "Long", "Half", "Double"])
def test_single_element_accessors(state, kind):
    """THCStorage_(set/get) and THCTensor_(set1d..4d / get1d..4d) (lib/THC/generic/THCStorage.c:20-34,
    generic/THCTensor.c:840-900): one element by storage index or by coordinates of a strided view."""
    import ctypes as C
    from common import make_view, rng, to_device
    r = rng("accessors", kind)
    creal = thc.KINDS[kind][2]

    def as_c(v):
        return thc._half_from_float(v) if kind == "Half" else v

    def from_c(v):
        return thc._half_to_float(v) if kind == "Half" else v

    for shape, layout in (((7,), "strided"), ((4, 5), "transposed"), ((3, 4, 5), "permuted"), ((2, 3, 4, 5), "holes")):
        host = make_view(r, kind, shape, layout)
        host[...] = r.integers(0, 50, size=shape).astype(host.dtype)
        t = to_device(state, host)
        nd = len(shape)
        get = state.fn(kind, f"get{nd}d")
        get.restype = creal
        get.argtypes = [C.c_void_p, C.c_void_p] + [C.c_long] * nd
        setf = state.fn(kind, f"set{nd}d")
        setf.restype = None
        setf.argtypes = [C.c_void_p, C.c_void_p] + [C.c_long] * nd + [creal]
        for _ in range(5):
            x = tuple(int(r.integers(0, n)) for n in shape)
            assert from_c(get(state.ptr, t.ptr, *x)) == host[x]
            setf(state.ptr, t.ptr, *x, as_c(77))
            state.check()
            host[x] = 77
        assert (t.numpy() == np.asarray(host)).all()
        get(state.ptr, t.ptr, *([0] * (nd - 1) + [shape[-1]]))
        with pytest.raises(thc.THCError, match="out of range"):
            state.check()
    wrong = state.fn(kind, "get2d")
    wrong.restype = creal
    wrong.argtypes = [C.c_void_p, C.c_void_p, C.c_long, C.c_long]
    wrong(state.ptr, to_device(state, np.zeros(3, thc.KINDS[kind][1])).ptr, 0, 0)
    with pytest.raises(thc.THCError, match="two dimensions"):
        state.check()


def test_a_view_that_leaves_its_storage_is_refused_before_any_launch(state):
    """cutorch asserts on offsets inside its kernels in debug builds (lib/THC/THCTensorInfo.cuh:228-278);
    here every call checks on the host that the view's smallest and largest offset lie inside the
    storage, so a bad view costs an error message, not a stray write."""
    buf = to_device(state, np.arange(100, dtype=np.float32))
    launches = state.lib.thcb200_launch_count()
    inside = thc.Tensor.wrap(state, "Float", buf.data_ptr, (10, 10), (10, 1), storage_elems=100)
    inside.add(inside, 1.0)
    assert state.lib.thcb200_launch_count() == launches + 1
    # setStorage itself never builds such a view (it grows the storage or refuses); a view goes bad
    # when something writes the tensor's fields directly, as FFI callers of cutorch can
    for field, index, value in [("size", 1, 11), ("stride", 0, 12), ("size", 0, 11)]:
        bad = thc.Tensor.wrap(state, "Float", buf.data_ptr, (10, 10), (10, 1), storage_elems=100)
        raw = C.cast(bad.ptr, C.POINTER(thc._THTensor)).contents
        getattr(raw, field)[index] = value
        with pytest.raises(thc.THCError, match="storage of 100 elements"):
            bad.add(bad, 1.0)
        with pytest.raises(thc.THCError, match="storage of 100 elements"):
            bad.sumall()
    assert state.lib.thcb200_launch_count() == launches + 1     # nothing was launched for the bad views
    want = np.arange(100, dtype=np.float32) + 1
    assert np.array_equal(buf.numpy(), want)
