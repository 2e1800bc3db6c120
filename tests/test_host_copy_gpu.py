"""Copies between CPU tensors and GPU tensors (cutorch's :cuda(), :float(), tensor:copy(other) across
the two kinds; lib/THC/generic/THCTensorCopy.c:7-164) for every pair of element types and strided
views on both sides.  cutorch's tests: test/test.lua:495-640 (copyRandomizedTest: random type pairs,
contiguous and transposed / narrowed on either side).  The expected result is the C conversion of
every element in logical order (half through float), which numpy's astype gives for values that fit
the target type: bit-exact."""
import numpy as np
import pytest

from cutorch_b200 import thc
from common import ALL_KINDS, NP_OF_KIND, assert_bit_equal, make_view, rng, to_device

pytestmark = pytest.mark.gpu

def small_values(r, kind, shape, layout):
    """Values every element type holds exactly (0..100), so that each conversion is exact."""
    x = make_view(r, kind, shape, layout)
    x[...] = r.integers(0, 101, size=shape).astype(x.dtype)
    return x


@pytest.mark.parametrize("gpu_kind", ALL_KINDS)
def test_copy_between_cpu_and_gpu_tensors(state, gpu_kind):
    r = rng("hostcopy", gpu_kind)
    shape = (13, 22)
    for cpu_kind in ALL_KINDS:
        for cpu_layout, gpu_layout in [("contiguous", "contiguous"), ("transposed", "contiguous"), ("contiguous", "strided"),
                                       ("holes", "transposed")]:
            # CPU -> GPU
            src = small_values(r, cpu_kind, shape, cpu_layout)
            dst = to_device(state, make_view(r, gpu_kind, shape, gpu_layout))
            dst.copy_from_cpu(thc.CpuTensor(src))
            assert_bit_equal(dst.numpy(), np.asarray(src).astype(NP_OF_KIND[gpu_kind]),
                             f"{cpu_kind} CPU ({cpu_layout}) -> {gpu_kind} GPU ({gpu_layout})")
            # GPU -> CPU
            gsrc_host = small_values(r, gpu_kind, shape, gpu_layout)
            gsrc = to_device(state, gsrc_host)
            back = make_view(r, cpu_kind, shape, cpu_layout)
            gsrc.copy_to_cpu(thc.CpuTensor(back))
            assert_bit_equal(np.asarray(back), np.asarray(gsrc_host).astype(NP_OF_KIND[cpu_kind]),
                             f"{gpu_kind} GPU ({gpu_layout}) -> {cpu_kind} CPU ({cpu_layout})")


def test_element_counts_not_shapes_and_errors(state):
    r = rng("hostcopy-errors")
    src = small_values(r, "Float", (6, 10), "contiguous")
    dst = thc.Tensor.new(state, "Double", 60)
    dst.copy_from_cpu(thc.CpuTensor(src))           # same element count, different shapes: logical order
    assert_bit_equal(dst.numpy(), np.asarray(src).reshape(60).astype(np.float64), "6x10 CPU -> 60 GPU")
    with pytest.raises(thc.THCError, match="sizes do not match"):
        thc.Tensor.new(state, "Float", 59).copy_from_cpu(thc.CpuTensor(src))
    with pytest.raises(thc.THCError, match="sizes do not match"):
        dst.copy_to_cpu(thc.CpuTensor(np.zeros(61, np.float32)))
    empty = thc.Tensor.new(state, "Float")
    empty.copy_from_cpu(thc.CpuTensor(np.zeros(0, np.float32)))   # nothing to do


def test_large_transfer_both_ways(state):
    """64 MiB of fp32 up as halves into a transposed GPU tensor and back down as doubles."""
    r = rng("hostcopy-large")
    host = (r.integers(-1000, 1001, size=(4096, 4096)) / 8).astype(np.float32)     # exact in half
    gpu = to_device(state, np.zeros((4096, 4096), np.float16)).transpose(0, 1)
    gpu.copy_from_cpu(thc.CpuTensor(host))
    assert_bit_equal(gpu.numpy(), host.astype(np.float16), "fp32 CPU -> transposed half GPU")
    down = np.zeros((4096, 4096), np.float64)
    gpu.copy_to_cpu(thc.CpuTensor(down))
    assert_bit_equal(down, host.astype(np.float64), "transposed half GPU -> double CPU")


@pytest.mark.parametrize("cols,step", [(64, 2), (70000, 35000)])
def test_strided_cpu_views_keep_their_gaps(state, cols, step):
    """A CPU view with gaps in its span: shipped as its span and strided on the GPU when the span is
    close to the view's size, packed on the host when the view is sparse in it (second case).  Either
    way the elements between the view's elements stay as they were."""
    r = rng("hostcopy-gaps", str(cols))
    base = r.integers(0, 100, size=(64, cols)).astype(np.float32)
    view = base[:, ::step]
    dev = thc.Tensor.new(state, "Double", *view.shape)
    dev.copy_from_cpu(thc.CpuTensor(view))
    assert_bit_equal(dev.numpy(), view.astype(np.float64), "strided CPU view -> GPU")
    dev.add(dev, 1000)
    before = base.copy()
    dev.copy_to_cpu(thc.CpuTensor(view))
    want = before.copy()
    want[:, ::step] = before[:, ::step] + 1000
    assert_bit_equal(base, want, "GPU -> strided CPU view, gaps untouched")


def test_storage_copies(state):
    """Whole storages (lib/THC/generic/THCStorageCopy.h): CPU -> GPU with conversion, GPU -> GPU with
    conversion, GPU -> CPU, and the size check."""
    import ctypes as C
    lib = state.lib
    host = np.arange(1000, dtype=np.float32) / 4
    cpu = thc.CpuTensor(host)
    g16 = thc.Tensor.new(state, "Half", 1000)
    g64 = thc.Tensor.new(state, "Double", 1000)

    def storage_of(t):
        f = state.fn(t.kind, "storage")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p, C.c_void_p]
        return C.c_void_p(f(state.ptr, t.ptr))

    for name in ("THCudaHalfStorage_copyFloat", "THCudaDoubleStorage_copyCudaHalf", "THFloatStorage_copyCudaDouble"):
        getattr(lib, name).argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        getattr(lib, name).restype = None
    lib.THCudaHalfStorage_copyFloat(state.ptr, storage_of(g16), C.byref(cpu._storage))
    state.check()
    assert_bit_equal(g16.numpy(), host.astype(np.float16), "CPU float storage -> GPU half storage")
    lib.THCudaDoubleStorage_copyCudaHalf(state.ptr, storage_of(g64), storage_of(g16))
    state.check()
    assert_bit_equal(g64.numpy(), host.astype(np.float16).astype(np.float64), "GPU half storage -> GPU double storage")
    back = np.zeros(1000, np.float32)
    cb = thc.CpuTensor(back)
    lib.THFloatStorage_copyCudaDouble(state.ptr, C.byref(cb._storage), storage_of(g64))
    state.check()
    assert_bit_equal(back, host.astype(np.float16).astype(np.float32), "GPU double storage -> CPU float storage")
    short = thc.CpuTensor(np.zeros(999, np.float32))
    lib.THFloatStorage_copyCudaDouble(state.ptr, C.byref(short._storage), storage_of(g64))
    with pytest.raises(thc.THCError, match="size does not match"):
        state.check()
