"""numpy restatement of tril / triu and renorm (test infrastructure, not part of the product)."""
from __future__ import annotations

import numpy as np


def tri(src: np.ndarray, k: int, upper: bool) -> np.ndarray:
    """TensorTriOp (lib/THC/THCTensorMathPairwise.cu:373-406): element (r, c) is kept when
    c - r <= k (lower) or c - r >= k (upper), else 0."""
    r = np.arange(src.shape[0])[:, None]
    c = np.arange(src.shape[1])[None, :]
    keep = (c - r >= k) if upper else (c - r <= k)
    return np.where(keep, src, src.dtype.type(0))


def renorm(src: np.ndarray, p: float, dim: int, maxnorm: float) -> np.ndarray:
    """renorm as torch7's CPU tensors compute it, slice by slice along `dim`
    (the call cutorch mirrors in lib/THC/generic/THCTensorMathReduce.cu:47-74 with the kernel
    lib/THC/THCTensorMathReduce.cuh:132-183): norm = (sum |x|^p)^(1/p) rounded to the element
    type; a slice whose norm exceeds maxnorm is multiplied by maxnorm / (norm + 1e-7), that
    quotient formed in double and rounded once; other slices are copied.  Half tensors are
    computed as float tensors and rounded to half at the end.  The sum itself is taken in double
    here; tests compare within the reduction tolerance."""
    real = np.float32 if src.dtype == np.float16 else src.dtype.type
    work = np.array(src, dtype=real, copy=True)
    out = np.array(work, copy=True)
    maxn = real(maxnorm)
    for j in range(src.shape[dim]):
        idx = [slice(None)] * src.ndim
        idx[dim] = j
        row = work[tuple(idx)].astype(np.float64)
        total = np.sum(np.abs(row) ** float(p)) if p not in (1, 2) else (np.sum(np.abs(row)) if p == 1 else np.sum(row * row))
        norm = real(np.float64(real(total)) ** (1.0 / float(p)))   # sum rounded to real, pow in double, rounded
        if norm > maxn:
            factor = real(np.float64(maxn) / (np.float64(norm) + 1e-7))
            out[tuple(idx)] = work[tuple(idx)] * factor
    return out.astype(src.dtype)
