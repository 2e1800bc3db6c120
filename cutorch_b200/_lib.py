"""ctypes loader for libthcb200.so and the descriptor structs of include/thcb200.h."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

MAX_DIMS = 25

U8, I8, I16, I32, I64, F16, F32, F64 = range(8)

STATUS = {0: "OK", -1: "ERR_ARG", -2: "ERR_DIMS", -3: "ERR_SIZE", -4: "ERR_CUDA", -5: "ERR_UNSUPPORTED",
          -6: "ERR_NOMEM", -7: "ERR_LIMIT"}

# thcb200_op, in header order
OPS = [
    "FILL", "COPY", "LOG", "LGAMMA", "LOG1P", "EXP", "COS", "SIN", "SQRT", "RSQRT", "CEIL", "FLOOR", "TRUNC", "ACOS",
    "COSH", "ASIN", "SINH", "TAN", "ATAN", "TANH", "ROUND", "FRAC", "CINV", "NEG", "ABS", "SIGN", "SIGMOID", "CLAMP",
    "POW", "TPOW", "ADD_S", "SUB_S", "MUL_S", "DIV_S", "LSHIFT_S", "RSHIFT_S", "FMOD_S", "REMAINDER_S", "BITAND_S",
    "BITOR_S", "BITXOR_S", "MAX_S", "MIN_S", "LT_S", "GT_S", "LE_S", "GE_S", "EQ_S", "NE_S",
    "ADD", "SUB", "CADD", "MUL", "DIV", "CPOW", "CLSHIFT", "CRSHIFT", "CMAX", "CMIN", "CFMOD", "CREMAINDER",
    "CBITAND", "CBITOR", "CBITXOR", "ATAN2", "LERP", "LT", "GT", "LE", "GE", "EQ", "NE",
    "ADDCMUL", "ADDCDIV",
]
OP = {name: i for i, name in enumerate(OPS)}
RED = {"SUM": 0, "PROD": 1, "MIN": 2, "MAX": 3, "ALL": 4, "ANY": 5}
PRE = {"IDENTITY": 0, "ABS": 1, "SQUARE": 2, "POWABS": 3, "NONZERO": 4, "SQDEV": 5, "MOMENTS": 6}
POST = {"NONE": 0, "DIV": 1, "POW": 2, "VAR_BIASED": 3, "VAR_UNBIASED": 4, "STD_BIASED": 5, "STD_UNBIASED": 6}
FLAG_IGNORE_OVERLAP = 1


def op_arity(op: int) -> int:
    if op == OP["FILL"]:
        return 0
    if OP["COPY"] <= op <= OP["NE_S"]:
        return 1
    if OP["ADD"] <= op <= OP["NE"]:
        return 2
    return 3


class TensorDesc(C.Structure):
    """struct thcb200_tensor"""
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("sizes", C.c_int64 * MAX_DIMS), ("strides", C.c_int64 * MAX_DIMS)]


class Scalar(C.Structure):
    """struct thcb200_scalar"""
    _fields_ = [("f", C.c_double), ("i", C.c_int64)]


def scalar(v) -> Scalar:
    f = float(v)
    try:
        i = int(v)
    except (OverflowError, ValueError):
        i = 0
    if not (-(1 << 63) <= i < (1 << 63)):
        i = 0
    return Scalar(f, i)


def make_desc(ptr: int, dtype: int, sizes, strides) -> TensorDesc:
    d = TensorDesc()
    d.data = ptr
    d.dtype = dtype
    d.ndim = len(sizes)
    for k, (s, t) in enumerate(zip(sizes, strides)):
        if k < MAX_DIMS:
            d.sizes[k] = s
            d.strides[k] = t
    return d


class LibraryMissing(RuntimeError):
    pass


def library_path() -> Path:
    return Path(__file__).resolve().parent / "lib" / "libthcb200.so"


_LIB = None


def load_library() -> C.CDLL:
    """Loads libthcb200.so.  There is no fallback: without the CUDA library nothing runs."""
    global _LIB
    if _LIB is not None:
        return _LIB
    p = library_path()
    if not p.exists():
        raise LibraryMissing(f"{p} is missing: build it with `python -m cutorch_b200.build` (needs nvcc)")
    lib = C.CDLL(str(p), mode=C.RTLD_GLOBAL)
    P = C.POINTER
    vp = C.c_void_p
    lib.thcb200_ctx_create.argtypes = [P(vp), C.c_int]
    lib.thcb200_ctx_create.restype = C.c_int
    lib.thcb200_ctx_destroy.argtypes = [vp]
    lib.thcb200_ctx_destroy.restype = None
    lib.thcb200_last_error.restype = C.c_char_p
    lib.thcb200_last_plan.restype = C.c_char_p
    lib.thcb200_launch_count.restype = C.c_int64
    lib.thcb200_memcpy_h2d.argtypes = [vp, vp, C.c_size_t, vp]
    lib.thcb200_memcpy_d2h.argtypes = [vp, vp, C.c_size_t, vp]
    lib.thcb200_stream_synchronize.argtypes = [vp]
    lib.thcb200_collapse_dims.argtypes = [P(C.c_int64), P(C.c_int64), P(C.c_int), C.c_int]
    lib.thcb200_collapse_dims.restype = C.c_int
    lib.thcb200_overlapping.argtypes = [P(TensorDesc)]
    lib.thcb200_can_use_32bit.argtypes = [P(TensorDesc)]
    lib.thcb200_index_to_offset.argtypes = [P(TensorDesc), C.c_int64]
    lib.thcb200_index_to_offset.restype = C.c_int64
    lib.thcb200_pointwise.argtypes = [vp, C.c_int, P(TensorDesc), P(TensorDesc), P(TensorDesc), P(TensorDesc), C.c_int,
                                      Scalar, Scalar, vp]
    lib.thcb200_pointwise_ex.argtypes = lib.thcb200_pointwise.argtypes + [C.c_int]
    lib.thcb200_copy_convert.argtypes = [vp, P(TensorDesc), P(TensorDesc), vp]
    lib.thcb200_reduce_dim.argtypes = [vp, C.c_int, C.c_int, Scalar, P(TensorDesc), P(TensorDesc), C.c_int, vp]
    lib.thcb200_reduce_dim_post.argtypes = [vp, C.c_int, C.c_int, Scalar, C.c_int, Scalar, P(TensorDesc), P(TensorDesc), C.c_int, vp]
    lib.thcb200_reduce_dim_index.argtypes = [vp, C.c_int, P(TensorDesc), P(TensorDesc), P(TensorDesc), C.c_int, vp]
    lib.thcb200_reduce_all.argtypes = [vp, C.c_int, C.c_int, Scalar, P(TensorDesc), vp, vp]
    lib.thcb200_reduce_all_host.argtypes = [vp, C.c_int, C.c_int, Scalar, P(TensorDesc), vp, vp]
    _LIB = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        lib = load_library()
        raise RuntimeError(f"thcb200 {STATUS.get(rc, rc)}: {lib.thcb200_last_error().decode()}")
