"""numpy restatement of the calls whose operands have two element types (test infrastructure,
not part of the product): comparisons into a Byte tensor and Byte-masked fill / copy / select.

Every function works on logical (row-major) order, which is what the reference's
THC_pointwiseApply walks (lib/THC/THCApply.cuh:19-122), so any numpy view can be passed.
Half operands compare as their float values (lib/THC/THCNumerics.cuh:126-533, float branch).
"""
from __future__ import annotations

import numpy as np

_CMP = {
    "lt": np.less, "gt": np.greater, "le": np.less_equal, "ge": np.greater_equal,
    "eq": np.equal, "ne": np.not_equal,
}


def _math(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float32) if a.dtype == np.float16 else a


def compare(name: str, a: np.ndarray, b) -> np.ndarray:
    """TensorLTValueOp ... TensorNEOp with TOut = unsigned char
    (lib/THC/THCTensorMathCompare.cuh:5-67, THCTensorMathCompareT.cuh:5-50): 1 where the
    comparison holds, else 0; the result has a's shape; b is a tensor with the same number of
    elements (walked in its own logical order) or a scalar already rounded to a's type."""
    x = _math(np.asarray(a))
    if isinstance(b, np.ndarray):
        y = _math(b).reshape(-1).reshape(x.shape) if b.shape != x.shape else _math(b)
    else:
        y = x.dtype.type(b)
    with np.errstate(invalid="ignore"):
        return _CMP[name](x, y).astype(np.uint8)


def masked_fill(t: np.ndarray, mask: np.ndarray, value) -> np.ndarray:
    """TensorMaskedFillOp (lib/THC/THCTensorMasked.cuh:16-26): t[i] = value where mask[i] != 0.
    Returns the new logical contents of t."""
    out = np.array(t, copy=True)
    flat = out.reshape(-1)
    flat[np.asarray(mask).reshape(-1) != 0] = t.dtype.type(value)
    return flat.reshape(t.shape)


def masked_copy(t: np.ndarray, mask: np.ndarray, src: np.ndarray) -> np.ndarray:
    """TensorMaskedCopyOp over an exclusive prefix sum of the mask
    (lib/THC/generic/THCTensorMasked.cu:35-104, THCTensorMasked.cuh:28-42): the k-th set mask
    element (logical order) receives src's k-th element (src's logical order)."""
    out = np.array(t, copy=True)
    flat = out.reshape(-1)
    sel = np.asarray(mask).reshape(-1) != 0
    flat[sel] = np.asarray(src).reshape(-1)[: int(sel.sum())]
    return flat.reshape(t.shape)


def masked_select(src: np.ndarray, mask: np.ndarray) -> np.ndarray:
    """TensorMaskedSelectOp (lib/THC/generic/THCTensorMasked.cu:119-177, THCTensorMasked.cuh:44-56):
    the elements of src whose mask element is set, in logical order, as a 1-D array."""
    return np.asarray(src).reshape(-1)[np.asarray(mask).reshape(-1) != 0].copy()
