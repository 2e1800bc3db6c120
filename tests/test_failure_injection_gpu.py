"""Allocation failures injected on the host: a device allocator whose k-th malloc fails, and the
library's own allocations made to fail through thcb200_debug_fail_allocation.  Every entry point
that allocates must report the failure the way cutorch does (THCudaCheck -> THError,
lib/THC/THCGeneral.c:714-726), leak nothing, leave tensors and contexts usable for the next call,
and run the garbage-collection callback before one retry when one is registered
(lib/THC/THCGeneral.c:836-854).  Nothing here exhausts or faults a GPU: the failing calls are fakes."""
import ctypes as C

import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import OP, PRE, RED
from oracle import mixed_oracle as mo
from common import assert_bit_equal, rng, to_device

pytestmark = pytest.mark.gpu

MALLOC = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.c_size_t, C.c_void_p)
REALLOC = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.c_size_t, C.c_size_t, C.c_void_p)
FREE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p)
EMPTY = C.CFUNCTYPE(C.c_int, C.c_void_p)
INFO = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t))
GC = C.CFUNCTYPE(None, C.c_void_p)
CUDA_ERROR_MEMORY_ALLOCATION = 2


class AllocatorStruct(C.Structure):
    _fields_ = [("malloc", MALLOC), ("realloc", REALLOC), ("free", FREE), ("emptyCache", EMPTY), ("cacheInfo", INFO),
                ("state", C.c_void_p)]


class FailingAllocator:
    """THCDeviceAllocator that hands every request to the allocator it replaces, except the k-th
    malloc after arm(k), which fails without touching CUDA.  Keeps the set of live blocks."""

    def __init__(self, state):
        self.thc_state = state
        lib = state.lib
        lib.THCState_getDeviceAllocator.restype = C.POINTER(AllocatorStruct)
        lib.THCState_getDeviceAllocator.argtypes = [C.c_void_p]
        lib.THCState_setDeviceAllocator.argtypes = [C.c_void_p, C.POINTER(AllocatorStruct)]
        self.inner = lib.THCState_getDeviceAllocator(state.ptr)
        self.countdown, self.failed, self.live = 0, 0, set()

        def malloc(_ctx, out, size, stream):
            if self.countdown > 0:
                self.countdown -= 1
                if self.countdown == 0:
                    self.failed += 1
                    out[0] = None
                    return CUDA_ERROR_MEMORY_ALLOCATION
            rc = self.inner.contents.malloc(self.inner.contents.state, out, size, stream)
            if rc == 0 and out[0]:
                self.live.add(out[0])
            return rc

        def free(_ctx, ptr):
            self.live.discard(ptr)
            return self.inner.contents.free(self.inner.contents.state, ptr)

        self._keep = (MALLOC(malloc), FREE(free))
        self.struct = AllocatorStruct(self._keep[0], REALLOC(), self._keep[1], EMPTY(), INFO(), None)

    def __enter__(self):
        self.thc_state.lib.THCState_setDeviceAllocator(self.thc_state.ptr, C.byref(self.struct))
        return self

    def __exit__(self, *exc):
        self.thc_state.lib.THCState_setDeviceAllocator(self.thc_state.ptr, self.inner)

    def arm(self, k):
        self.countdown = k


_ALLOCATORS = []   # storages point at their allocator for life: the structs are never collected


@pytest.fixture()
def own_state():
    """A THCState of its own (fresh contexts with their first small workspace)."""
    s = thc.State()
    yield s
    s.shutdown()


def test_every_allocating_entry_point_survives_a_failing_allocator(own_state, oracle):
    state = own_state
    r = rng("fail-alloc")
    x = r.standard_normal((64, 96)).astype(np.float32)
    y = r.standard_normal((64, 96)).astype(np.float32)
    mask = (r.uniform(size=(64, 96)) < 0.3).astype(np.uint8)
    inj = FailingAllocator(state)
    _ALLOCATORS.append(inj)
    T = thc.Tensor
    with inj:
        dx, dy, dm = to_device(state, x), to_device(state, y), to_device(state, mask)
        dxT = dx.transpose(0, 1)          # a view: no allocation
        cases = [
            ("cmul into a new tensor", "Float", lambda o: o.cmul(dx, dy), lambda: oracle.pointwise(OP["MUL"], np.zeros_like(x), [x, y])),
            ("sum along dim 0", "Float", lambda o: o.sum(dx, 0, 1), lambda: oracle.reduce_dim(RED["SUM"], PRE["IDENTITY"], 0.0, x, 0)),
            ("cumsum", "Float", lambda o: o.cumsum(dx, 1), lambda: oracle.scan_dim(False, x, 1)),
            ("maskedSelect", "Float", lambda o: o.maskedSelect(dx, dm), lambda: mo.masked_select(x, mask)),
            ("gtValue into a byte tensor", "Byte", lambda o: dx.call("gtValue", o, dx, 0.0), lambda: mo.compare("gt", x, 0.0)),
            ("copy of a transposed view into a resized tensor", "Float", lambda o: (o.resizeAs(dxT), o.copy(dxT)), lambda: np.ascontiguousarray(x.T)),
        ]
        for what, kind, op, want in cases:
            live_before = set(inj.live)
            hit = False
            for k in range(1, 6):
                out = T.new(state, kind)
                inj.arm(k)
                failed_before = inj.failed
                try:
                    op(out)
                    done = True
                except thc.THCError as e:
                    done = False
                    assert "error (2)" in str(e) or "out of memory" in str(e).lower(), f"{what}: {e}"
                inj.arm(0)
                if inj.failed > failed_before:
                    hit = True
                    assert not done, f"{what}: the {k}-th allocation failed and the call reported success"
                    # the tensor is as it was (empty), and the same call works now
                    assert out.nelement == 0 or out.sizes, what
                    op(out)
                exp = want()
                got = out.numpy()
                if got.dtype.kind == "f" and "sum" in what:
                    assert np.allclose(got, exp, rtol=1e-5, atol=1e-5), what
                else:
                    assert_bit_equal(got.reshape(exp.shape), exp, f"{what} after a failure at allocation {k}")
                out.free()
                state.synchronize()
                assert inj.live == live_before, f"{what}: {len(inj.live - live_before)} blocks leaked after a failure at allocation {k}"
                if not (inj.failed > failed_before):
                    break    # the call needs fewer than k allocations: every one of them has been failed once
            assert hit, f"{what} never allocated through the state's allocator"
        for t in (dxT, dx, dy, dm):
            t.free()
        state.synchronize()
        assert not inj.live, f"{len(inj.live)} blocks were never returned to the allocator"


def test_gc_callback_runs_once_before_the_retry(own_state):
    state = own_state
    lib = state.lib
    lib.THCSetGCHandler.argtypes = [C.c_void_p, GC, C.c_void_p]
    inj = FailingAllocator(state)
    _ALLOCATORS.append(inj)
    calls = []
    handler = GC(lambda data: calls.append(data))
    with inj:
        lib.THCSetGCHandler(state.ptr, handler, None)
        try:
            inj.arm(1)
            t = thc.Tensor.new(state, "Float", 1000)      # the first attempt fails, the collector runs, the retry succeeds
            assert inj.failed == 1 and len(calls) == 1
            t.fill(2.0)
            assert float(t.sumall()) == 2000.0
            t.free()
        finally:
            lib.THCSetGCHandler(state.ptr, GC(), None)
        inj.arm(1)
        with pytest.raises(thc.THCError):
            thc.Tensor.new(state, "Float", 1000)           # no callback registered: the failure is reported
        assert len(calls) == 1
    state.synchronize()
    assert not inj.live


def test_the_librarys_own_allocations_can_fail_cleanly(own_state, oracle):
    """Workspace growth of a split reduction, the tile offsets of a masked select, the dense temporary
    of an apply whose output overlaps itself, and the staging buffer of a converting CPU -> GPU copy."""
    state = own_state
    lib = state.lib
    lib.thcb200_debug_fail_allocation.argtypes = [C.c_int]
    lib.thcb200_debug_fail_allocation.restype = None
    r = rng("fail-internal")
    x = (r.integers(-1000, 1001, (3000, 8192)) / 8).astype(np.float32)
    dx = to_device(state, x)
    out = thc.Tensor.new(state, "Float", 1, 8192)
    mask = (r.uniform(size=200000) < 0.5).astype(np.uint8)
    v = r.standard_normal(200000).astype(np.float32)
    dv, dm = to_device(state, v), to_device(state, mask)
    sel = thc.Tensor.new(state, "Float")
    base = to_device(state, np.arange(96, dtype=np.float32).reshape(1, 96))
    ones = to_device(state, np.ones((64, 96), np.float32))
    host = r.standard_normal((33, 65)).astype(np.float64)
    half = thc.Tensor.new(state, "Half", 33, 65)
    cases = [
        ("split column reduction (workspace growth)", lambda: out.sum(dx, 0, 1),
         lambda: assert_bit_equal(out.numpy(), oracle.reduce_dim(RED["SUM"], PRE["IDENTITY"], 0.0, x, 0), "sum dim 0")),
        ("maskedSelect (tile offsets)", lambda: sel.maskedSelect(dv, dm),
         lambda: assert_bit_equal(sel.numpy(), mo.masked_select(v, mask), "maskedSelect")),
        ("apply into an expanded view (dense temporary)", lambda: base.expand(64, 96).add(ones, 1.0),
         lambda: None),
        ("double CPU tensor into a half GPU tensor (staging buffer)", lambda: half.copy_from_cpu(thc.CpuTensor(host)),
         lambda: assert_bit_equal(half.numpy(), host.astype(np.float32).astype(np.float16), "converting copy")),
    ]
    try:
        for what, call, check in cases:
            lib.thcb200_debug_fail_allocation(1)
            with pytest.raises(thc.THCError, match="allocat|memory"):
                call()
            lib.thcb200_debug_fail_allocation(0)
            call()            # the context is usable and the same call now succeeds
            state.synchronize()
            check()
    finally:
        lib.thcb200_debug_fail_allocation(0)
