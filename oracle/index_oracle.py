"""numpy restatement of the indexed moves (test infrastructure, not part of the product).

Positions are 1-based as in torch7 (TH_INDEX_BASE = 1).  Every function returns the new logical
contents of the destination.  With duplicate positions, copies keep the last writer in logical
order here; the GPU calls do not define which duplicate lands (tests avoid duplicates for copy /
scatter), and adds accumulate all of them (tests use values whose sums are exact)."""
from __future__ import annotations

import numpy as np


def index_select(src: np.ndarray, dim: int, idx: np.ndarray) -> np.ndarray:
    """dst.select(dim, i) = src.select(dim, idx[i] - 1)  (lib/THC/THCTensorIndex.cu:259-340)."""
    return np.take(src, np.asarray(idx) - 1, axis=dim)


def index_copy(dst: np.ndarray, dim: int, idx: np.ndarray, src: np.ndarray) -> np.ndarray:
    """dst.select(dim, idx[i] - 1) = src.select(dim, i)  (lib/THC/THCTensorIndex.cu:22-101)."""
    out = np.array(dst, copy=True)
    for i, p in enumerate(np.asarray(idx)):
        sl = [slice(None)] * out.ndim
        sl[dim] = int(p) - 1
        out[tuple(sl)] = np.take(src, i, axis=dim)
    return out


def index_add(dst: np.ndarray, dim: int, idx: np.ndarray, src: np.ndarray) -> np.ndarray:
    """dst.select(dim, idx[i] - 1) += src.select(dim, i)  (lib/THC/THCTensorIndex.cu:105-183)."""
    out = np.array(dst, copy=True)
    for i, p in enumerate(np.asarray(idx)):
        sl = [slice(None)] * out.ndim
        sl[dim] = int(p) - 1
        out[tuple(sl)] = out[tuple(sl)] + np.take(src, i, axis=dim)
    return out


def index_fill(dst: np.ndarray, dim: int, idx: np.ndarray, value) -> np.ndarray:
    """dst.select(dim, idx[i] - 1) = value  (lib/THC/THCTensorIndex.cu:187-255)."""
    out = np.array(dst, copy=True)
    for p in np.asarray(idx):
        sl = [slice(None)] * out.ndim
        sl[dim] = int(p) - 1
        out[tuple(sl)] = dst.dtype.type(value)
    return out


def _redirected(index: np.ndarray, dim: int):
    coords = list(np.indices(index.shape))
    coords[dim] = np.asarray(index) - 1
    return tuple(coords)


def gather(src: np.ndarray, dim: int, index: np.ndarray) -> np.ndarray:
    """tensor[c] = src[c with c[dim] = index[c] - 1]  (lib/THC/THCTensorScatterGather.cu:78-103)."""
    return np.asarray(src)[_redirected(index, dim)]


def scatter(dst: np.ndarray, dim: int, index: np.ndarray, src: np.ndarray) -> np.ndarray:
    """tensor[c with c[dim] = index[c] - 1] = src[c]  (lib/THC/THCTensorScatterGather.cu:105-130)."""
    out = np.array(dst, copy=True)
    out[_redirected(index, dim)] = np.asarray(src)
    return out


def scatter_add(dst: np.ndarray, dim: int, index: np.ndarray, src: np.ndarray) -> np.ndarray:
    """tensor[c with c[dim] = index[c] - 1] += src[c]  (lib/THC/THCTensorScatterGather.cu:132-157)."""
    out = np.array(dst, copy=True)
    np.add.at(out, _redirected(index, dim), np.asarray(src))
    return out


def scatter_fill(dst: np.ndarray, dim: int, index: np.ndarray, value) -> np.ndarray:
    """tensor[c with c[dim] = index[c] - 1] = value  (lib/THC/THCTensorScatterGather.cu:159-184)."""
    out = np.array(dst, copy=True)
    out[_redirected(index, dim)] = dst.dtype.type(value)
    return out
