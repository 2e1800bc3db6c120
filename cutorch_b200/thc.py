"""Host-side mirror of cutorch's tensor interface over the THC C API of libthcb200.so.

cutorch exposes the THC entry points as tensor methods through cwrap-generated stubs
(TensorMath.lua:429-438,552-2258: fetch ``cutorch._state``, check argument types, call
``TH<Type>Tensor_<name>(state, ...)``).  :class:`Tensor` plays the role of those stubs from
Python: ``z.cadd(x, 2.5, y)`` calls ``THCudaTensor_cadd(state, z, x, 2.5f, y)``.  Every method
goes through the C ABI of the shared library; there is no other implementation behind it.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib


class THCError(RuntimeError):
    """A THC call reported an error (THError / THArgCheck in cutorch)."""


class _Half(C.Structure):
    _fields_ = [("x", C.c_ushort)]


# kind -> (CReal infix of the symbol names, numpy dtype, ctypes `real`, ctypes `accreal`, thcb200 dtype)
KINDS = {
    "Byte": ("CudaByte", np.uint8, C.c_ubyte, C.c_long, _lib.U8),
    "Char": ("CudaChar", np.int8, C.c_byte, C.c_long, _lib.I8),
    "Short": ("CudaShort", np.int16, C.c_short, C.c_long, _lib.I16),
    "Int": ("CudaInt", np.int32, C.c_int, C.c_long, _lib.I32),
    "Long": ("CudaLong", np.int64, C.c_long, C.c_long, _lib.I64),
    "Half": ("CudaHalf", np.float16, _Half, C.c_float, _lib.F16),
    "Float": ("Cuda", np.float32, C.c_float, C.c_float, _lib.F32),
    "Double": ("CudaDouble", np.float64, C.c_double, C.c_double, _lib.F64),
}
KIND_OF_DTYPE = {np.dtype(v[1]): k for k, v in KINDS.items()}


class _THStorage(C.Structure):
    """torch7's CPU storage (lib/TH/generic/THStorage.h): the same fields for every element type."""
    _fields_ = [("data", C.c_void_p), ("size", C.c_ssize_t), ("refcount", C.c_int), ("flag", C.c_char),
                ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p), ("view", C.c_void_p)]


class _THTensor(C.Structure):
    """torch7's CPU tensor (lib/TH/generic/THTensor.h)."""
    _fields_ = [("size", C.POINTER(C.c_long)), ("stride", C.POINTER(C.c_long)), ("nDimension", C.c_int),
                ("storage", C.POINTER(_THStorage)), ("storageOffset", C.c_ssize_t), ("refcount", C.c_int), ("flag", C.c_char)]


class CpuTensor:
    """A numpy array seen as a TH CPU tensor (TH<Type>Tensor): the argument of the copies between
    CPU and GPU tensors.  Any non-negative strides that are whole elements; the array is not copied."""

    def __init__(self, array: np.ndarray):
        if array.dtype not in KIND_OF_DTYPE:
            raise TypeError(f"no tensor type for {array.dtype}")
        if any(s < 0 or s % array.itemsize for s in array.strides):
            raise ValueError("strides must be non-negative multiples of the element size")
        self.array = array
        self.kind = KIND_OF_DTYPE[array.dtype]
        nd = array.ndim
        self._size = (C.c_long * max(nd, 1))(*array.shape)
        self._stride = (C.c_long * max(nd, 1))(*[s // array.itemsize for s in array.strides])
        extent = 1 + sum((n - 1) * (s // array.itemsize) for n, s in zip(array.shape, array.strides)) if array.size else 0
        self._storage = _THStorage(array.ctypes.data, extent, 1, b"\x00", None, None, None)
        self._tensor = _THTensor(self._size, self._stride, nd, C.pointer(self._storage), 0, 1, b"\x01")

    @property
    def ptr(self):
        return C.byref(self._tensor)
FLOATING = ("Half", "Float", "Double")

# Argument codes: T tensor of the receiver's type, L LongTensor, C / M CPU Long / Byte tensor (CpuTensor), r real, l long, i int, S sizes.
# Return codes: v void, a accreal, R real, n int.
_UNARY = ["sigmoid", "log", "lgamma", "log1p", "exp", "cos", "acos", "cosh", "sin", "asin", "sinh", "tan", "atan",
          "tanh", "sqrt", "rsqrt", "ceil", "floor", "round", "trunc", "frac", "cinv", "neg", "abs", "sign"]
SIGNATURES = {name: ("v", "TT") for name in _UNARY}
SIGNATURES.update({
    "pow": ("v", "TTr"), "tpow": ("v", "TrT"), "atan2": ("v", "TTT"), "lerp": ("v", "TTTr"),
    "clamp": ("v", "TTrr"), "cross": ("v", "TTTi"),
    "cadd": ("v", "TTrT"), "csub": ("v", "TTrT"),
    "cmul": ("v", "TTT"), "cpow": ("v", "TTT"), "cdiv": ("v", "TTT"), "clshift": ("v", "TTT"), "crshift": ("v", "TTT"),
    "cmax": ("v", "TTT"), "cmin": ("v", "TTT"), "cfmod": ("v", "TTT"), "cremainder": ("v", "TTT"),
    "cmaxValue": ("v", "TTr"), "cminValue": ("v", "TTr"),
    "cbitand": ("v", "TTT"), "cbitor": ("v", "TTT"), "cbitxor": ("v", "TTT"),
    "addcmul": ("v", "TTrTT"), "addcdiv": ("v", "TTrTT"),
    "add": ("v", "TTr"), "sub": ("v", "TTr"), "mul": ("v", "TTr"), "div": ("v", "TTr"),
    "lshift": ("v", "TTr"), "rshift": ("v", "TTr"), "fmod": ("v", "TTr"), "remainder": ("v", "TTr"),
    "bitand": ("v", "TTr"), "bitor": ("v", "TTr"), "bitxor": ("v", "TTr"),
    "equal": ("n", "TT"),
    "sum": ("v", "TTli"), "prod": ("v", "TTli"), "mean": ("v", "TTli"), "norm": ("v", "TTrli"),
    "sumall": ("a", "T"), "prodall": ("a", "T"), "meanall": ("a", "T"),
    "min": ("v", "TLTli"), "max": ("v", "TLTli"), "minall": ("R", "T"), "maxall": ("R", "T"),
    "var": ("v", "TTlii"), "std": ("v", "TTlii"), "dist": ("a", "TTr"),
    "normall": ("a", "Tr"), "varall": ("a", "Ti"), "stdall": ("a", "Ti"),
    "fill": ("v", "Tr"), "zero": ("v", "T"), "copy": ("v", "TT"), "copyIgnoringOverlaps": ("v", "TT"),
    "resizeAs": ("v", "TT"),
    "tril": ("v", "TTl"), "triu": ("v", "TTl"), "renorm": ("v", "TTrlr"),
    "indexSelect": ("v", "TTiL"), "indexCopy": ("v", "TiLT"), "indexAdd": ("v", "TiLT"), "indexFill": ("v", "TiLr"),
    # thin callers of fill / copy / sumall; code S: a tuple of sizes passed as a THLongStorage
    "zeros": ("v", "TS"), "ones": ("v", "TS"), "zerosLike": ("v", "TT"), "onesLike": ("v", "TT"), "reshape": ("v", "TTS"),
    "numel": ("p", "T"), "nonzero": ("v", "LT"), "diag": ("v", "TTl"), "eye": ("v", "Tll"), "trace": ("a", "T"),
    # masks in a CPU ByteTensor (code M)
    "maskedFillByte": ("v", "TMr"), "maskedCopyByte": ("v", "TMT"), "maskedSelectByte": ("v", "TTM"),
    # the same with a CPU LongTensor of positions (code C)
    "indexSelect_long": ("v", "TTiC"), "indexCopy_long": ("v", "TiCT"), "indexAdd_long": ("v", "TiCT"),
    "indexFill_long": ("v", "TiCr"),
    "gather": ("v", "TTiL"), "scatter": ("v", "TiLT"), "scatterAdd": ("v", "TiLT"), "scatterFill": ("v", "TiLr"),
    "cumsum": ("v", "TTl"), "cumprod": ("v", "TTl"),
    "maskedFill": ("v", "TBr"), "maskedCopy": ("v", "TBT"), "maskedSelect": ("v", "TTB"),
})
# comparisons: <op>Value / <op>Tensor write a Byte tensor ("B"), the ...T forms the operands' type
for _c in ("lt", "gt", "le", "ge", "eq", "ne"):
    SIGNATURES.update({_c + "Value": ("v", "BTr"), _c + "ValueT": ("v", "TTr"),
                       _c + "Tensor": ("v", "BTT"), _c + "TensorT": ("v", "TTT")})


def _half_from_float(v: float) -> _Half:
    return _Half(int(np.array(v, dtype=np.float16).view(np.uint16)))


def _half_to_float(h: _Half) -> float:
    return float(np.array(h.x, dtype=np.uint16).view(np.float16))


class State:
    """THCState: owns the per-device contexts; `stream` selects the current stream."""

    def __init__(self):
        self.lib = _lib.load_library()
        lib = self.lib
        lib.THCState_alloc.restype = C.c_void_p
        lib.THCudaInit.argtypes = [C.c_void_p]
        lib.THCudaShutdown.argtypes = [C.c_void_p]
        lib.THCState_free.argtypes = [C.c_void_p]
        lib.THCB200_errorMessage.restype = C.c_char_p
        lib.THCB200_streamFromRaw.restype = C.c_void_p
        lib.THCB200_streamFromRaw.argtypes = [C.c_void_p, C.c_int]
        lib.THCState_setStream.argtypes = [C.c_void_p, C.c_void_p]
        lib.THCStream_free.argtypes = [C.c_void_p]
        lib.THCState_getCurrentStream.restype = C.c_void_p
        lib.THCState_getCurrentStream.argtypes = [C.c_void_p]
        lib.THCB200_currentContext.restype = C.c_void_p
        lib.THCB200_currentContext.argtypes = [C.c_void_p]
        self.ptr = C.c_void_p(lib.THCState_alloc())
        lib.THCB200_clearError()
        lib.THCudaInit(self.ptr)
        self.check()
        self._fn_cache = {}

    def check(self):
        if self.lib.THCB200_errorOccurred():
            msg = self.lib.THCB200_errorMessage().decode()
            self.lib.THCB200_clearError()
            raise THCError(msg)

    def set_stream(self, raw_stream: int, device: int = 0):
        """Makes a stream created elsewhere (e.g. torch.cuda.Stream.cuda_stream) current."""
        s = self.lib.THCB200_streamFromRaw(C.c_void_p(raw_stream), device)
        self.lib.THCState_setStream(self.ptr, C.c_void_p(s))
        self.lib.THCStream_free(C.c_void_p(s))
        self.check()

    @property
    def stream(self) -> int:
        return self.lib.THCState_getCurrentStream(self.ptr) or 0

    @property
    def context(self) -> int:
        c = self.lib.THCB200_currentContext(self.ptr)
        self.check()
        return c

    def synchronize(self):
        _lib.check(self.lib.thcb200_stream_synchronize(C.c_void_p(self.stream)))

    def shutdown(self):
        if self.ptr:
            self.lib.THCudaShutdown(self.ptr)
            self.lib.THCState_free(self.ptr)
            self.ptr = None

    def fn(self, kind: str, name: str, prefix: str = "Tensor"):
        key = (kind, name, prefix)
        f = self._fn_cache.get(key)
        if f is None:
            # a private function object per symbol: ctypes caches attribute lookups, and the
            # argtypes set by one caller must not leak into another
            f = self.lib[f"TH{KINDS[kind][0]}{prefix}_{name}"]
            self._fn_cache[key] = f
        return f


class Tensor:
    """A THCuda<Kind>Tensor handle."""

    def __init__(self, state: State, kind: str, ptr: int):
        self.state, self.kind, self.ptr = state, kind, C.c_void_p(ptr)

    # ---- construction ------------------------------------------------------------------
    @classmethod
    def new(cls, state: State, kind: str = "Float", *sizes: int) -> "Tensor":
        f = state.fn(kind, "new")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p]
        t = cls(state, kind, f(state.ptr))
        if sizes:
            t.resize(*sizes)
        return t

    @classmethod
    def from_numpy(cls, state: State, arr: np.ndarray) -> "Tensor":
        """Clones a numpy array to the device with its exact sizes, strides and holes
        (cloneExactlyToGPUType, test/test.lua:348-361)."""
        kind = KIND_OF_DTYPE[arr.dtype]
        item = arr.dtype.itemsize
        if arr.ndim == 0:
            arr = arr.reshape(1)
        strides = [s // item for s in arr.strides]
        if any(s < 0 for s in strides):
            raise ValueError("negative strides are not representable as TH tensors")
        extent = 1 + sum((n - 1) * s for n, s in zip(arr.shape, strides)) if arr.size else 0
        t = cls.new(state, kind)
        if extent == 0:
            if arr.ndim:
                t.resize(*arr.shape)
            return t
        flat = np.lib.stride_tricks.as_strided(arr, shape=(extent,), strides=(item,))
        flat = np.ascontiguousarray(flat)
        st = state.fn(kind, "newWithSize", "Storage")
        st.restype = C.c_void_p
        st.argtypes = [C.c_void_p, C.c_ssize_t]
        storage = C.c_void_p(st(state.ptr, extent))
        state.check()
        data = state.fn(kind, "data", "Storage")
        data.restype = C.c_void_p
        data.argtypes = [C.c_void_p, C.c_void_p]
        dptr = data(state.ptr, storage)
        _lib.check(state.lib.thcb200_memcpy_h2d(C.c_void_p(dptr), flat.ctypes.data_as(C.c_void_p), flat.nbytes,
                                                 C.c_void_p(state.stream)))
        t._set_storage(storage, 0, arr.shape, strides)
        free = state.fn(kind, "free", "Storage")
        free.argtypes = [C.c_void_p, C.c_void_p]
        free(state.ptr, storage)
        return t

    @classmethod
    def wrap(cls, state: State, kind: str, device_ptr: int, sizes, strides=None, storage_elems=None) -> "Tensor":
        """A tensor over device memory owned by someone else (not freed, not resizable)."""
        sizes = list(sizes)
        if strides is None:
            strides, run = [], 1
            for n in reversed(sizes):
                strides.insert(0, run)
                run *= n
        if storage_elems is None:
            storage_elems = 1 + sum((n - 1) * s for n, s in zip(sizes, strides))
        nw = state.fn(kind, "newWithData", "Storage")
        nw.restype = C.c_void_p
        nw.argtypes = [C.c_void_p, C.c_void_p, C.c_ssize_t]
        storage = C.c_void_p(nw(state.ptr, C.c_void_p(device_ptr), storage_elems))
        clear = state.fn(kind, "clearFlag", "Storage")
        clear.argtypes = [C.c_void_p, C.c_void_p, C.c_char]
        clear(state.ptr, storage, bytes([4 | 2]))  # TH_STORAGE_FREEMEM | TH_STORAGE_RESIZABLE
        t = cls.new(state, kind)
        t._set_storage(storage, 0, sizes, strides)
        free = state.fn(kind, "free", "Storage")
        free.argtypes = [C.c_void_p, C.c_void_p]
        free(state.ptr, storage)
        return t

    def _long_storage(self, values):
        lib = self.state.lib
        lib.THLongStorage_newWithSize.restype = C.c_void_p
        lib.THLongStorage_newWithSize.argtypes = [C.c_ssize_t]
        lib.THLongStorage_set.argtypes = [C.c_void_p, C.c_ssize_t, C.c_long]
        lib.THLongStorage_free.argtypes = [C.c_void_p]
        s = C.c_void_p(lib.THLongStorage_newWithSize(len(values)))
        for k, v in enumerate(values):
            lib.THLongStorage_set(s, k, int(v))
        return s

    def _set_storage(self, storage, offset, sizes, strides):
        f = self.state.fn(self.kind, "setStorage")
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_ssize_t, C.c_void_p, C.c_void_p]
        sz, st = self._long_storage(sizes), self._long_storage(strides)
        f(self.state.ptr, self.ptr, storage, offset, sz, st)
        self.state.lib.THLongStorage_free(sz)
        self.state.lib.THLongStorage_free(st)
        self.state.check()

    def resize(self, *sizes):
        f = self.state.fn(self.kind, "resize")
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        sz = self._long_storage(sizes)
        f(self.state.ptr, self.ptr, sz, None)
        self.state.lib.THLongStorage_free(sz)
        self.state.check()
        return self

    def free(self):
        if self.ptr:
            f = self.state.fn(self.kind, "free")
            f.argtypes = [C.c_void_p, C.c_void_p]
            f(self.state.ptr, self.ptr)
            self.ptr = None

    # ---- views -------------------------------------------------------------------------
    def transpose(self, d1, d2) -> "Tensor":
        f = self.state.fn(self.kind, "newTranspose")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        t = Tensor(self.state, self.kind, f(self.state.ptr, self.ptr, d1, d2))
        self.state.check()
        return t

    def expand(self, *sizes) -> "Tensor":
        """tensor:expand(sizes): a broadcast view (THCTensor_(newExpand))."""
        f = self.state.fn(self.kind, "newExpand")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        sz = self._long_storage(sizes)
        p = f(self.state.ptr, self.ptr, sz)
        self.state.lib.THLongStorage_free(sz)
        self.state.check()
        return Tensor(self.state, self.kind, p)

    def narrow(self, dim, first, size) -> "Tensor":
        f = self.state.fn(self.kind, "newNarrow")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_long, C.c_long]
        t = Tensor(self.state, self.kind, f(self.state.ptr, self.ptr, dim, first, size))
        self.state.check()
        return t

    def select(self, dim, index) -> "Tensor":
        f = self.state.fn(self.kind, "newSelect")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_long]
        t = Tensor(self.state, self.kind, f(self.state.ptr, self.ptr, dim, index))
        self.state.check()
        return t

    def contiguous(self) -> "Tensor":
        f = self.state.fn(self.kind, "newContiguous")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p, C.c_void_p]
        t = Tensor(self.state, self.kind, f(self.state.ptr, self.ptr))
        self.state.check()
        return t

    # ---- metadata ----------------------------------------------------------------------
    @property
    def ndim(self) -> int:
        f = self.state.fn(self.kind, "nDimension")
        f.argtypes = [C.c_void_p, C.c_void_p]
        return f(self.state.ptr, self.ptr)

    def _dims(self, name):
        f = self.state.fn(self.kind, name)
        f.restype = C.c_long
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        return [f(self.state.ptr, self.ptr, d) for d in range(self.ndim)]

    @property
    def sizes(self):
        return self._dims("size")

    @property
    def strides(self):
        return self._dims("stride")

    @property
    def nelement(self) -> int:
        f = self.state.fn(self.kind, "nElement")
        f.restype = C.c_ssize_t
        f.argtypes = [C.c_void_p, C.c_void_p]
        return f(self.state.ptr, self.ptr)

    @property
    def data_ptr(self) -> int:
        f = self.state.fn(self.kind, "data")
        f.restype = C.c_void_p
        f.argtypes = [C.c_void_p, C.c_void_p]
        return f(self.state.ptr, self.ptr) or 0

    @property
    def is_contiguous(self) -> bool:
        f = self.state.fn(self.kind, "isContiguous")
        f.argtypes = [C.c_void_p, C.c_void_p]
        return bool(f(self.state.ptr, self.ptr))

    def descriptor(self) -> _lib.TensorDesc:
        return _lib.make_desc(self.data_ptr, KINDS[self.kind][4], self.sizes, self.strides)

    def numpy(self) -> np.ndarray:
        """Copies the view back to the host as a dense array in logical order."""
        sizes, strides = self.sizes, self.strides
        dt = np.dtype(KINDS[self.kind][1])
        if not sizes or self.nelement == 0:
            return np.zeros(sizes, dtype=dt)
        if any(s < 0 for s in strides):
            raise ValueError("negative strides")
        extent = 1 + sum((n - 1) * s for n, s in zip(sizes, strides))
        flat = np.empty(extent, dtype=dt)
        self.state.synchronize()
        _lib.check(self.state.lib.thcb200_memcpy_d2h(flat.ctypes.data_as(C.c_void_p), C.c_void_p(self.data_ptr), flat.nbytes,
                                                      C.c_void_p(self.state.stream)))
        view = np.lib.stride_tricks.as_strided(flat, shape=sizes, strides=[s * dt.itemsize for s in strides])
        return np.array(view, copy=True)

    # ---- THC calls ---------------------------------------------------------------------
    def _real(self, v):
        creal = KINDS[self.kind][2]
        if self.kind == "Half":
            return _half_from_float(float(v))
        if self.kind in FLOATING:
            return creal(float(v))
        return creal(int(v))

    def call(self, name: str, *args):
        """Calls TH<Kind>Tensor_<name>(state, ...) with `args` exactly in C order."""
        ret, spec = SIGNATURES[name]
        if len(args) != len(spec):
            raise TypeError(f"{name} takes {len(spec)} arguments ({spec}), got {len(args)}")
        f = self.state.fn(self.kind, name)
        creal, cacc = KINDS[self.kind][2], KINDS[self.kind][3]
        argtypes, cargs = [C.c_void_p], [self.state.ptr]
        storages = []
        for code, a in zip(spec, args):
            if code == "S":
                sz = self._long_storage(tuple(a))
                storages.append(sz)
                argtypes.append(C.c_void_p)
                cargs.append(sz)
                continue
            if code in "TLB":
                if not isinstance(a, Tensor):
                    raise TypeError(f"{name}: expected a tensor")
                want = {"L": "Long", "B": "Byte"}.get(code, self.kind)
                if a.kind != want:
                    raise TypeError(f"{name}: expected a {want} tensor, got {a.kind}")
                argtypes.append(C.c_void_p)
                cargs.append(a.ptr)
            elif code in "CM":
                want = "Long" if code == "C" else "Byte"
                if not isinstance(a, CpuTensor) or a.kind != want:
                    raise TypeError(f"{name}: expected a CPU {want} tensor")
                argtypes.append(C.c_void_p)
                cargs.append(a.ptr)
            elif code == "r":
                argtypes.append(creal)
                cargs.append(self._real(a))
            elif code == "l":
                argtypes.append(C.c_long)
                cargs.append(int(a))
            else:
                argtypes.append(C.c_int)
                cargs.append(int(a))
        f.argtypes = argtypes
        f.restype = {"v": None, "a": cacc, "R": creal, "n": C.c_int, "p": C.c_ssize_t}[ret]
        r = f(*cargs)
        for sz in storages:
            self.state.lib.THLongStorage_free(sz)
        self.state.check()
        if ret == "R" and self.kind == "Half":
            return _half_to_float(r)
        return r

    def copy_from(self, src: "Tensor"):
        """self:copy(src) with type conversion (THCTensor_(copyCuda<Type>))."""
        if src.kind == self.kind:
            return self.call("copy", self, src)
        f = self.state.fn(self.kind, "copyCudaFloat" if src.kind == "Float" else "copy" + KINDS[src.kind][0])
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        f.restype = None
        f(self.state.ptr, self.ptr, src.ptr)
        self.state.check()

    def copy_from_cpu(self, cpu: "CpuTensor"):
        """self:copy(cpuTensor): THCuda<T>Tensor_copy<CpuType> (lib/THC/generic/THCTensorCopy.c:33-62)."""
        f = self.state.fn(self.kind, "copy" + cpu.kind)
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        f.restype = None
        f(self.state.ptr, self.ptr, cpu.ptr)
        self.state.check()

    def copy_to_cpu(self, cpu: "CpuTensor"):
        """cpuTensor:copy(self): TH<CpuType>Tensor_copyCuda<T> (lib/THC/generic/THCTensorCopy.c:66-110)."""
        f = getattr(self.state.lib, f"TH{cpu.kind}Tensor_copyCuda{self.kind}")
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        f.restype = None
        f(self.state.ptr, cpu.ptr, self.ptr)
        self.state.check()

    def copy_async_from_cpu(self, cpu: "CpuTensor"):
        """THCuda<T>Tensor_copyAsyncCPU (lib/THC/generic/THCTensorCopy.c:112-137): same element type, both
        contiguous, one asynchronous copy in the order of the current stream; the CPU side should be pinned."""
        f = self.state.fn(self.kind, "copyAsyncCPU")
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        f.restype = None
        f(self.state.ptr, self.ptr, cpu.ptr)
        self.state.check()

    def copy_async_to_cpu(self, cpu: "CpuTensor"):
        """TH<T>Tensor_copyAsyncCuda (lib/THC/generic/THCTensorCopy.c:139-164): the way back."""
        f = getattr(self.state.lib, f"TH{self.kind}Tensor_copyAsyncCuda")
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        f.restype = None
        f(self.state.ptr, cpu.ptr, self.ptr)
        self.state.check()

    def cat(self, inputs, dimension: int):
        """result:cat(inputs, dimension): THCTensor_(catArray) (lib/THC/generic/THCTensorMath.cu:84-260)."""
        f = self.state.fn(self.kind, "catArray")
        arr = (C.c_void_p * len(inputs))(*[t.ptr for t in inputs])
        f.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int]
        f.restype = None
        f(self.state.ptr, self.ptr, arr, len(inputs), dimension)
        self.state.check()

    def sumall_to_device(self, result_dev_ptr: int):
        f = self.state.fn(self.kind, "sumallToDevice")
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        f.restype = None
        f(self.state.ptr, self.ptr, C.c_void_p(result_dev_ptr))
        self.state.check()

    def __getattr__(self, name):
        # tensor methods in the Lua style: the receiver is the first C argument
        if name in SIGNATURES:
            return lambda *args: self.call(name, self, *args)
        raise AttributeError(name)
