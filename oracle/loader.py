"""TEST INFRASTRUCTURE.  Loads the oracle libraries and wraps them for numpy arrays."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
MAX_DIMS = 25

DTYPE_ID = {np.dtype(np.uint8): 0, np.dtype(np.int8): 1, np.dtype(np.int16): 2, np.dtype(np.int32): 3,
            np.dtype(np.int64): 4, np.dtype(np.float16): 5, np.dtype(np.float32): 6, np.dtype(np.float64): 7}


def oracle_path() -> Path:
    return HERE / "_build" / "libth_oracle.so"


def ref_path() -> Path:
    return HERE / "_ref" / "libref_check.so"


def cutorch_tree():
    """Where a cutorch checkout lies, if anywhere: the environment variable CUTORCH_TREE, else a
    directory named `reference` beside the repository."""
    import os
    for cand in (os.environ.get("CUTORCH_TREE"), str(HERE.parent.parent / "reference")):
        if cand and (Path(cand) / "lib" / "THC").is_dir():
            return cand
    return None


def build_oracle() -> None:
    """make -C oracle: the restatement always, the reference-derived library when a cutorch
    tree is at hand (see cutorch_tree)."""
    cmd = ["make", "-C", str(HERE)]
    tree = cutorch_tree()
    if tree:
        cmd.append(f"REF={tree}")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the oracle failed:\n{r.stdout}\n{r.stderr}")


class _Desc(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("sizes", C.c_int64 * MAX_DIMS), ("strides", C.c_int64 * MAX_DIMS)]


def _desc(a: np.ndarray) -> _Desc:
    d = _Desc()
    d.data = a.ctypes.data
    d.dtype = DTYPE_ID[a.dtype]
    d.ndim = a.ndim
    for k in range(a.ndim):
        d.sizes[k] = a.shape[k]
        d.strides[k] = a.strides[k] // a.dtype.itemsize
    return d


class Oracle:
    """CPU results the GPU path has to reproduce.  Arrays may be arbitrary strided views."""

    def __init__(self, threads: int = 1):
        p = oracle_path()
        if not p.exists():
            build_oracle()
        self.lib = C.CDLL(str(p))
        P = C.POINTER
        self.lib.oracle_pointwise.argtypes = [C.c_int, P(_Desc), P(_Desc), P(_Desc), P(_Desc), C.c_int, C.c_double,
                                              C.c_double, C.c_int64, C.c_int64]
        self.lib.oracle_copy_convert.argtypes = [P(_Desc), P(_Desc)]
        self.lib.oracle_reduce_dim.argtypes = [C.c_int, C.c_int, C.c_double, P(_Desc), P(_Desc), P(_Desc), C.c_int]
        self.lib.oracle_var_dim.argtypes = [P(_Desc), P(_Desc), C.c_int, C.c_int, C.c_int]
        self.lib.oracle_reduce_all.argtypes = [C.c_int, C.c_int, C.c_double, P(_Desc), P(C.c_double), P(C.c_int64)]
        self.set_threads(threads)

    def set_threads(self, n: int) -> None:
        self.lib.oracle_set_threads(int(n))

    def max_threads(self) -> int:
        return int(self.lib.oracle_max_threads())

    def pointwise(self, op: int, out: np.ndarray, inputs=(), s0=0, s1=0) -> np.ndarray:
        descs = [_desc(x) for x in inputs]
        ptrs = [C.byref(d) for d in descs] + [None] * (3 - len(descs))

        def iv(v):
            try:
                i = int(v)
            except (OverflowError, ValueError):
                return 0
            return i if -(1 << 63) <= i < (1 << 63) else 0
        od = _desc(out)
        rc = self.lib.oracle_pointwise(op, C.byref(od), ptrs[0], ptrs[1], ptrs[2], len(descs), float(s0), float(s1),
                                       iv(s0), iv(s1))
        assert rc == 0
        return out

    def convert(self, out: np.ndarray, src: np.ndarray) -> np.ndarray:
        od, sd = _desc(out), _desc(src)
        assert self.lib.oracle_copy_convert(C.byref(od), C.byref(sd)) == 0
        return out

    def reduce_dim(self, rop: int, pre: int, s: float, src: np.ndarray, dim: int, with_index: bool = False):
        shape = list(src.shape)
        shape[dim] = 1
        out = np.zeros(shape, dtype=src.dtype)
        idx = np.zeros(shape, dtype=np.int64) if with_index else None
        od, sd = _desc(out), _desc(src)
        xd = _desc(idx) if with_index else None
        rc = self.lib.oracle_reduce_dim(rop, pre, float(s), C.byref(od), C.byref(xd) if with_index else None,
                                        C.byref(sd), dim)
        assert rc == 0
        return (out, idx) if with_index else out

    def var_dim(self, src: np.ndarray, dim: int, biased: bool, take_sqrt: bool) -> np.ndarray:
        shape = list(src.shape)
        shape[dim] = 1
        out = np.zeros(shape, dtype=src.dtype)
        od, sd = _desc(out), _desc(src)
        assert self.lib.oracle_var_dim(C.byref(od), C.byref(sd), dim, int(biased), int(take_sqrt)) == 0
        return out

    def scan_dim(self, prod: bool, src: np.ndarray, dim: int) -> np.ndarray:
        """cumsum (prod=False) / cumprod (prod=True) of src along dim, as a dense array."""
        out = np.zeros(src.shape, dtype=src.dtype)
        od, sd = _desc(out), _desc(src)
        assert self.lib.oracle_scan_dim(int(prod), C.byref(od), C.byref(sd), dim) == 0
        return out

    def reduce_all(self, rop: int, pre: int, s: float, src: np.ndarray):
        """Returns a float for floating element types (the double accumulator) and an int otherwise."""
        f, i = C.c_double(0), C.c_int64(0)
        sd = _desc(src)
        assert self.lib.oracle_reduce_all(rop, pre, float(s), C.byref(sd), C.byref(f), C.byref(i)) == 0
        return f.value if src.dtype.kind == "f" else i.value


class RefCheck:
    """cutorch's own TensorInfo / functor code compiled for the host (oracle/_ref)."""

    FUNCTOR = {
        "SIGMOID": 0, "SIGN": 1, "ADD": 2, "CADD": 3, "SUB": 4, "MUL": 5, "POW": 6, "TPOW": 7, "CPOW": 8, "DIV": 9,
        "CREMAINDER": 10, "CFMOD": 11, "CLAMP": 12, "LERP": 13, "CMAX": 14, "CMIN": 15, "MAX_S": 16, "MIN_S": 17,
        "ADDCMUL": 18, "ADDCDIV": 19, "CLSHIFT": 20, "CRSHIFT": 21, "CBITAND": 22, "CBITOR": 23, "CBITXOR": 24,
        "LOG": 100, "LGAMMA": 101, "LOG1P": 102, "EXP": 103, "COS": 104, "SIN": 105, "SQRT": 106, "RSQRT": 107,
        "CEIL": 108, "FLOOR": 109, "TRUNC": 110, "ACOS": 111, "COSH": 112, "ASIN": 113, "SINH": 114, "TAN": 115,
        "ATAN": 116, "TANH": 117, "ROUND": 118, "FRAC": 119, "CINV": 120, "NEG": 121, "ABS": 122,
    }

    @staticmethod
    def available() -> bool:
        return ref_path().exists()

    def __init__(self):
        self.lib = C.CDLL(str(ref_path()))
        P = C.POINTER
        self.lib.ref_collapse_dims.argtypes = [P(C.c_int64), P(C.c_int64), P(C.c_int), C.c_int]
        self.lib.ref_is_contiguous.argtypes = [P(C.c_int64), P(C.c_int64), C.c_int]
        self.lib.ref_index_to_offset.argtypes = [P(C.c_int64), P(C.c_int64), C.c_int, C.c_int64]
        self.lib.ref_index_to_offset.restype = C.c_int64
        self.lib.ref_apply_functor.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_void_p, C.c_double, C.c_double, C.c_int64, C.c_int64]

        self.lib.ref_compare.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_double, C.c_int64]
        self.lib.ref_masked.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_double, C.c_int64]

    CMP = {"lt": 0, "gt": 1, "le": 2, "ge": 3, "eq": 4, "ne": 5}

    def compare(self, name: str, a: np.ndarray, b, same_type: bool = False) -> np.ndarray:
        """TensorLTValueOp ... TensorNEOp (lib/THC/THCTensorMathCompare.cuh, THCTensorMathCompareT.cuh) on
        dense arrays; b is an array of a's dtype or a scalar; the result is uint8, or a's dtype with same_type."""
        a = np.ascontiguousarray(a)
        out = np.zeros(a.shape, a.dtype if same_type else np.uint8)
        if isinstance(b, np.ndarray):
            bb = np.ascontiguousarray(b)
            rc = self.lib.ref_compare(self.CMP[name], int(same_type), DTYPE_ID[a.dtype], a.size, out.ctypes.data, a.ctypes.data,
                                      bb.ctypes.data, 0.0, 0)
        else:
            rc = self.lib.ref_compare(self.CMP[name], int(same_type), DTYPE_ID[a.dtype], a.size, out.ctypes.data, a.ctypes.data,
                                      None, float(b), int(b) if a.dtype.kind != "f" else 0)
        assert rc == 0
        return out

    def masked(self, which: str, t: np.ndarray, mask: np.ndarray, other=None, value=0) -> np.ndarray:
        """TensorMaskedFillOp / CopyOp / SelectOp (lib/THC/THCTensorMasked.cuh:16-56) over the exclusive prefix
        sum of the mask.  fill / copy return t's new contents, select returns the packed elements."""
        t = np.array(t, copy=True, order="C")
        m = np.ascontiguousarray(mask, dtype=np.uint8)
        fp = t.dtype.kind == "f"
        if which == "fill":
            rc = self.lib.ref_masked(0, DTYPE_ID[t.dtype], t.size, t.ctypes.data, m.ctypes.data, None, float(value), 0 if fp else int(value))
            res = t
        elif which == "copy":
            src = np.ascontiguousarray(other)
            rc = self.lib.ref_masked(1, DTYPE_ID[t.dtype], t.size, t.ctypes.data, m.ctypes.data, src.ctypes.data, 0.0, 0)
            res = t
        else:
            res = np.zeros(int((m != 0).sum()), t.dtype)
            rc = self.lib.ref_masked(2, DTYPE_ID[t.dtype], t.size, t.ctypes.data, m.ctypes.data, res.ctypes.data, 0.0, 0)
        assert rc == 0
        return res

    def collapse_dims(self, sizes, strides, exclude_dim=-1):
        n = len(sizes)
        sz = (C.c_int64 * MAX_DIMS)(*sizes)
        st = (C.c_int64 * MAX_DIMS)(*strides)
        nd = C.c_int(n)
        r = self.lib.ref_collapse_dims(sz, st, C.byref(nd), exclude_dim)
        return list(sz[:nd.value]), list(st[:nd.value]), r

    def index_to_offset(self, sizes, strides, linear):
        n = len(sizes)
        sz = (C.c_int64 * MAX_DIMS)(*sizes)
        st = (C.c_int64 * MAX_DIMS)(*strides)
        return self.lib.ref_index_to_offset(sz, st, n, linear)

    def apply(self, name: str, out: np.ndarray, inputs, s0=0, s1=0) -> np.ndarray:
        """Dense arrays only."""
        arrs = [np.ascontiguousarray(x) for x in inputs]
        ptrs = [x.ctypes.data for x in arrs] + [None] * (3 - len(arrs))
        assert out.flags.c_contiguous
        rc = self.lib.ref_apply_functor(self.FUNCTOR[name], DTYPE_ID[out.dtype], out.size, out.ctypes.data, ptrs[0], ptrs[1],
                                        ptrs[2], float(s0), float(s1), int(s0) if out.dtype.kind != "f" else 0,
                                        int(s1) if out.dtype.kind != "f" else 0)
        if rc != 0:
            raise KeyError(f"functor {name} is not defined for {out.dtype}")
        return out
