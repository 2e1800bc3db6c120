"""thcb200_reduce_dim_static: the dimension reduction that never allocates.

Some callers cannot call cudaMalloc when they need a reduction (their own pool owns all device
memory, or allocations are forbidden after start-up), so this entry point keeps the partials of
split reductions in a fixed device array inside the library.  It must give exactly what the
regular thcb200_reduce_dim gives -- the same kernels run -- call after call, although the array
still holds the previous call's partials, and it must refuse reductions whose partials do not
fit.  Collected last on purpose: a failure here cannot hide the other tests' results."""
import ctypes as C

import numpy as np
import pytest

from cutorch_b200 import _lib, thc
from cutorch_b200._lib import PRE, RED
from common import assert_bit_equal, assert_reduction_close, rng, to_device

pytestmark = pytest.mark.gpu

# (shape, dim, dtype): the first two split the reduced dim (column tiles / one block per row),
# so partials go through the static array; the third needs no partials at all
CASES = [((3000, 96), 0, np.float32), ((5, 70000), 1, np.float32), ((37, 300), 1, np.int32), ((4096, 512), 0, np.float64)]


def _free_device_bytes():
    """Free bytes on the current device as the CUDA runtime reports them."""
    rt = C.CDLL("libcudart.so.12")
    free, total = C.c_size_t(0), C.c_size_t(0)
    assert rt.cudaMemGetInfo(C.byref(free), C.byref(total)) == 0
    return free.value


def _static_fn(lib):
    f = lib.thcb200_reduce_dim_static
    f.argtypes = [C.c_int, C.c_int, _lib.Scalar, C.POINTER(_lib.TensorDesc), C.POINTER(_lib.TensorDesc), C.c_int, C.c_void_p]
    f.restype = C.c_int
    return f


@pytest.mark.parametrize("case", range(len(CASES)))
def test_static_scratch_matches_regular_entry_point_twice_in_a_row(state, oracle, case):
    shape, dim, dt = CASES[case]
    lib = _lib.load_library()
    static_fn = _static_fn(lib)
    out_shape = list(shape)
    out_shape[dim] = 1
    kind = thc.KIND_OF_DTYPE[np.dtype(dt)]
    zero = _lib.scalar(0)
    stream = C.c_void_p(state.stream)
    r = rng("no_alloc", case)
    # The first call on a device is the set-up call: it looks up the array's device address, and the
    # CUDA runtime loads the library's device code -- the array included -- at that moment.  A caller
    # makes it once at start-up; the check below is about every call after it.
    tiny_in, tiny_out = thc.Tensor.new(state, "Float", 4, 4), thc.Tensor.new(state, "Float", 1, 4)
    tiny_in.fill(1.0)
    dti, dto = tiny_in.descriptor(), tiny_out.descriptor()
    _lib.check(static_fn(RED["SUM"], PRE["IDENTITY"], zero, C.byref(dto), C.byref(dti), 0, stream))
    state.synchronize()
    for round_ in range(2):  # the second call finds the first call's partials in the array
        if np.dtype(dt).kind == "f":
            x = r.standard_normal(shape).astype(dt)
        else:
            x = r.integers(-1000, 1000, size=shape).astype(dt)
        dx = to_device(state, x)
        for rop in ("SUM", "MAX"):
            want = thc.Tensor.new(state, kind, *out_shape)
            got = thc.Tensor.new(state, kind, *out_shape)
            din, dw, dg = dx.descriptor(), want.descriptor(), got.descriptor()
            _lib.check(lib.thcb200_reduce_dim(C.c_void_p(state.context), RED[rop], PRE["IDENTITY"], zero, C.byref(dw), C.byref(din),
                                              dim, stream))
            # the claim in the name: the call leaves the device's free memory where it found it
            state.synchronize()
            free_before = _free_device_bytes()
            _lib.check(static_fn(RED[rop], PRE["IDENTITY"], zero, C.byref(dg), C.byref(din), dim, stream))
            state.synchronize()
            assert _free_device_bytes() == free_before, "the static entry point changed the free device memory"
            # identical kernels and partitioning: the tolerance of the other reduction tests (bit-exact
            # for integers, 1e-5 relative for float sums) tightens to bit equality here
            assert_bit_equal(got.numpy(), want.numpy(), f"static vs regular {rop} {shape} dim {dim} round {round_}")
            # and against the CPU oracle, as the other reduction tests do: max and integer sums bit for
            # bit, floating sums within 1e-5 relative (1e-12 for double)
            ref = oracle.reduce_dim(RED[rop], PRE["IDENTITY"], 0.0, x, dim)
            if rop == "MAX" or np.dtype(dt).kind != "f":
                assert_bit_equal(got.numpy(), ref, f"static vs oracle {rop} {shape} dim {dim} round {round_}")
            else:
                rel = 1e-12 if dt == np.float64 else 1e-5
                assert_reduction_close(got.numpy(), ref, rel, np.abs(x).sum(axis=dim, keepdims=True),
                                       f"static vs oracle {rop} {shape} dim {dim} round {round_}")


def test_static_scratch_refuses_what_does_not_fit(state):
    """fp16 8192 x 8192 summed over dim 0 is split so finely that its partials exceed the array."""
    lib = _lib.load_library()
    static_fn = _static_fn(lib)
    x = thc.Tensor.new(state, "Half", 8192, 8192)
    out = thc.Tensor.new(state, "Half", 1, 8192)
    din, dout = x.descriptor(), out.descriptor()
    rc = static_fn(RED["SUM"], PRE["IDENTITY"], _lib.scalar(0), C.byref(dout), C.byref(din), 0, C.c_void_p(state.stream))
    assert rc == -7, rc
    assert b"static scratch" in lib.thcb200_last_error()
    # a bad argument is reported, not executed
    rc = static_fn(RED["SUM"], PRE["IDENTITY"], _lib.scalar(0), C.byref(dout), C.byref(din), 5, C.c_void_p(state.stream))
    assert rc == -1
    # the running sums of var / std come with a post step this entry point has no argument for
    rc = static_fn(RED["SUM"], PRE["MOMENTS"], _lib.scalar(0), C.byref(dout), C.byref(din), 0, C.c_void_p(state.stream))
    assert rc == -1
    assert b"MOMENTS" in lib.thcb200_last_error()
