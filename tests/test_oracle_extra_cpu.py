"""Sanity of the oracle's scan and of the numpy restatements of the mixed-type calls against
independent numpy formulations (no GPU)."""
import numpy as np

from oracle import mixed_oracle as mo
from common import make_view, rng


def test_oracle_scan_matches_numpy_on_exact_inputs(oracle):
    r = rng("oracle-scan")
    for shape, dim, layout in [((5, 7), 0, "contiguous"), ((5, 7), 1, "transposed"), ((3, 4, 6), 1, "strided"), ((9,), 0, "offset")]:
        x = make_view(r, "Long", shape, layout)
        x[...] = r.integers(-5, 6, size=shape)
        assert np.array_equal(oracle.scan_dim(False, x, dim), np.cumsum(x, axis=dim))
        assert np.array_equal(oracle.scan_dim(True, x, dim), np.cumprod(x, axis=dim))
        f = make_view(r, "Float", shape, layout)
        f[...] = (r.integers(-100, 101, size=shape) / 4).astype(np.float32)   # sums exact in fp32
        assert np.array_equal(oracle.scan_dim(False, f, dim), np.cumsum(f.astype(np.float64), axis=dim).astype(np.float32))
    # integer accumulation wraps modulo 2^64, then truncates to the element type
    b = np.full((300,), 255, np.uint8)
    assert np.array_equal(oracle.scan_dim(False, b, 0), (np.cumsum(b.astype(np.uint64)) & 0xFF).astype(np.uint8))
    # half: accumulated wide, each output rounded to half
    h = np.full((4096,), 0.25, np.float16)
    assert np.array_equal(oracle.scan_dim(False, h, 0), (np.arange(1, 4097) * 0.25).astype(np.float16))


def test_mixed_oracle_on_small_known_cases():
    a = np.array([[1, 2, 3], [4, 5, 6]], np.int32)
    m = np.array([[1, 0, 2], [0, 0, 1]], np.uint8)
    assert mo.compare("ge", a, 3).tolist() == [[0, 0, 1], [1, 1, 1]]
    assert mo.compare("ne", a, a.T.reshape(-1)).tolist() == [[0, 1, 1], [1, 1, 0]]   # other operand in its own order
    assert mo.masked_fill(a, m, 9).tolist() == [[9, 2, 9], [4, 5, 9]]
    assert mo.masked_select(a.T, m.T).tolist() == [1, 3, 6]
    assert mo.masked_copy(a, m, np.array([7, 8, 9, 10], np.int32)).tolist() == [[7, 2, 8], [4, 5, 9]]
    h = np.array([np.nan, 1.0], np.float16)
    assert mo.compare("eq", h, h).tolist() == [0, 1] and mo.compare("ne", h, h).tolist() == [1, 0]
