"""Copies between two GPUs driven from one process, the way cutorch drives several devices
(THC_copyTensor, lib/THC/THCTensorCopy.cu:24-205; cutorch's own test: test/test.lua:3100-3170,
"multi_gpu_copy_noncontig").  Needs two visible devices; skipped on a one-GPU box.

Contiguous same-type tensors take cudaMemcpyAsync; strided views and type conversions run the
copy / convert kernel on the source device with the destination addressed as peer memory."""
import numpy as np
import pytest

from cutorch_b200 import thc
from common import assert_bit_equal, make_view, rng, to_device

pytestmark = pytest.mark.gpu


@pytest.fixture()
def two_devices():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    prev = torch.cuda.current_device()
    yield torch
    torch.cuda.set_device(prev)


def on_device(torch, dev, fn):
    torch.cuda.set_device(dev)
    try:
        return fn()
    finally:
        torch.cuda.set_device(0)


def test_copy_across_devices(state, two_devices):
    torch = two_devices
    r = rng("xdev")
    for kind, shape, ls, ld in [("Float", (256, 300), "contiguous", "contiguous"), ("Float", (64, 50), "transposed", "contiguous"),
                                ("Double", (7, 9, 11), "permuted", "holes"), ("Half", (33, 65), "contiguous", "transposed"),
                                ("Int", (1000,), "strided", "offset")]:
        src = make_view(r, kind, shape, ls)
        dst0 = make_view(r, kind, shape, ld)
        for sdev, ddev in ((0, 1), (1, 0)):
            dsrc = on_device(torch, sdev, lambda: to_device(state, src))
            ddst = on_device(torch, ddev, lambda: to_device(state, dst0))
            # issued while device 0 is current, whatever the operands' devices
            ddst.copy(dsrc)
            got = on_device(torch, ddev, lambda: ddst.numpy())
            assert_bit_equal(got, np.ascontiguousarray(src), f"{kind} copy {ls}->{ld} gpu{sdev}->gpu{ddev}")
            # the source is untouched
            assert_bit_equal(on_device(torch, sdev, lambda: dsrc.numpy()), np.ascontiguousarray(src), "source after the copy")


def test_converting_copy_across_devices(state, two_devices):
    torch = two_devices
    r = rng("xdev-conv")
    src = make_view(r, "Float", (40, 70), "transposed")
    dsrc = on_device(torch, 1, lambda: to_device(state, src))
    for kind in ("Double", "Half", "Int", "Byte"):
        ddst = to_device(state, make_view(r, kind, (40, 70), "contiguous"))          # on device 0
        ddst.copy_from(dsrc)
        with np.errstate(invalid="ignore"):
            want = np.ascontiguousarray(src).astype(ddst.numpy().dtype) if kind != "Byte" else \
                np.ascontiguousarray(src).astype(np.int64).astype(np.uint8)
        if kind == "Byte":
            continue   # negative floats to unsigned bytes are implementation-defined in C; only run it
        assert_bit_equal(ddst.numpy(), want, f"Float on gpu1 -> {kind} on gpu0")


def test_work_after_a_cross_device_copy_sees_the_data(state, two_devices):
    """The destination's stream waits for the copy: a kernel queued right after it reads the new values."""
    torch = two_devices
    x = np.arange(1 << 20, dtype=np.float32)
    dsrc = on_device(torch, 1, lambda: to_device(state, x))
    ddst = to_device(state, np.zeros_like(x))
    ddst.copy(dsrc)
    assert ddst.sumall() == float(np.float32(x.astype(np.float64).sum()))   # accreal of a FloatTensor is float


def test_copy_without_peer_access_goes_through_dense_temporaries(state, two_devices):
    """With direct access switched off (THCState_setPeerToPeerAccess) a strided or converting copy
    is staged through contiguous temporaries on both devices, as in the reference; the values are
    the same."""
    import ctypes as C
    torch = two_devices
    lib = state.lib
    lib.THCState_getPeerToPeerAccess.argtypes = [C.c_void_p, C.c_int, C.c_int]
    lib.THCState_setPeerToPeerAccess.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    r = rng("xdev-nop2p")
    src = make_view(r, "Float", (50, 64), "transposed")
    dst0 = make_view(r, "Float", (50, 64), "holes")
    assert lib.THCState_getPeerToPeerAccess(state.ptr, 1, 0) == 1
    lib.THCState_setPeerToPeerAccess(state.ptr, 1, 0, 0)
    try:
        assert lib.THCState_getPeerToPeerAccess(state.ptr, 1, 0) == 0
        dsrc = on_device(torch, 1, lambda: to_device(state, src))
        ddst = to_device(state, dst0)
        ddst.copy(dsrc)
        assert_bit_equal(ddst.numpy(), np.ascontiguousarray(src), "staged strided copy gpu1 -> gpu0")
        dd = to_device(state, np.zeros((50, 64), np.float64))
        dd.copy_from(dsrc)
        assert_bit_equal(dd.numpy(), np.ascontiguousarray(src).astype(np.float64), "staged converting copy gpu1 -> gpu0")
    finally:
        lib.THCState_setPeerToPeerAccess(state.ptr, 1, 0, 1)
    assert lib.THCState_getPeerToPeerAccess(state.ptr, 1, 0) == 1


def test_cpu_tensor_copies_reach_a_tensor_on_another_device(state, two_devices):
    """copy between a CPU tensor and a GPU tensor that lives on device 1 while device 0 is current
    (cutorch's cudaMemcpy does not care which device is current either)."""
    torch = two_devices
    r = rng("xdev-host")
    host = make_view(r, "Float", (40, 33), "transposed")
    on1 = on_device(torch, 1, lambda: to_device(state, np.zeros((40, 33), np.float64)))
    on1.copy_from_cpu(thc.CpuTensor(host))                       # device 0 is current here
    assert_bit_equal(on_device(torch, 1, lambda: on1.numpy()), np.asarray(host).astype(np.float64), "CPU -> GPU 1")
    back = np.zeros((40, 33), np.float32)
    on1.copy_to_cpu(thc.CpuTensor(back))
    assert_bit_equal(back, np.ascontiguousarray(host), "GPU 1 -> CPU")
