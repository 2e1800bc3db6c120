"""The five baseline configurations, at their full sizes, through the THC C API.

c1-c4 are compared with the CPU oracle directly (it finishes each of them in seconds); c5 holds
2^32 elements per tensor, so it is checked through size-independent properties: sampled rows
against the oracle, and the sum of row sums against the full reduction."""
import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import OP, PRE, RED, load_library
from common import assert_bit_equal, assert_reduction_close, assert_ulp, rng, to_device

pytestmark = pytest.mark.gpu


def plan_name():
    return load_library().thcb200_last_plan().decode()


def test_c1_cadd_then_sumall(state, oracle):
    r = rng("c1")
    n = 16_777_216
    x = r.uniform(-1, 1, n).astype(np.float32)
    y = r.uniform(-1, 1, n).astype(np.float32)
    dz = thc.Tensor.new(state, "Float")
    dz.cadd(to_device(state, x), 2.5, to_device(state, y))
    assert plan_name() == "contig_vec"
    want = oracle.pointwise(OP["CADD"], np.zeros(n, np.float32), [x, y], 2.5)
    assert_bit_equal(dz.numpy(), want, "c1 cadd")
    s = dz.sumall()
    ws = oracle.reduce_all(RED["SUM"], 0, 0, want)
    assert_reduction_close(s, ws, 1e-5, np.abs(want.astype(np.float64)).sum(), "c1 sumall")
    # THC returns accreal = float: the double accumulator rounded once
    assert s == float(np.float32(s))


def test_c2_addcmul_transposed_and_strided(state, oracle):
    r = rng("c2")
    shape = (64, 256, 56, 56)
    x = r.standard_normal(shape, dtype=np.float32)
    ybase = r.standard_normal((64, 56, 56, 256), dtype=np.float32)
    y = ybase.transpose(0, 3, 2, 1)                       # dims 1 and 3 swapped: strides (802816, 1, 256, 14336)
    assert tuple(s // 4 for s in y.strides) == (802816, 1, 256, 14336)
    wbase = r.standard_normal((64, 256, 56, 112), dtype=np.float32)
    w = wbase[..., ::2]                                    # strides (1605632, 6272, 112, 2)
    assert tuple(s // 4 for s in w.strides) == (1605632, 6272, 112, 2)
    out = thc.Tensor.new(state, "Float")
    out.addcmul(to_device(state, x), 0.5, to_device(state, y), to_device(state, w))
    assert plan_name() == "tiled"
    assert out.is_contiguous and out.sizes == list(shape)
    want = oracle.pointwise(OP["ADDCMUL"], np.zeros(shape, np.float32), [x, y, w], 0.5)
    assert_bit_equal(out.numpy(), want, "c2 addcmul")


def test_c3_dim_reductions_with_ties(state, oracle):
    r = rng("c3")
    m = (r.integers(-1000, 1001, (32768, 8192)) / 8).astype(np.float32)
    dm = to_device(state, m)
    for dim, plan in ((1, "row_warp_vec"), (0, "col_tile_split")):
        s = thc.Tensor.new(state, "Float")
        s.sum(dm, dim, 1)
        assert plan_name() == plan
        # every partial sum is a multiple of 1/8 far below 2^24/8: the order cannot matter, so bit-exact
        assert_bit_equal(s.numpy(), oracle.reduce_dim(RED["SUM"], 0, 0, m, dim), f"c3 sum dim {dim}")
        v, i = thc.Tensor.new(state, "Float"), thc.Tensor.new(state, "Long")
        v.max(i, dm, dim, 1)
        wv, wi = oracle.reduce_dim(RED["MAX"], 0, 0, m, dim, with_index=True)
        assert_bit_equal(v.numpy(), wv, f"c3 max values dim {dim}")
        assert_bit_equal(i.numpy(), wi, f"c3 argmax (first occurrence, 1-based) dim {dim}")


def test_c4_half_sigmoid_mean_norm(state, oracle):
    r = rng("c4.1")
    h = (r.standard_normal((8192, 8192)) * 2).astype(np.float16)
    dh = to_device(state, h)
    h2 = thc.Tensor.new(state, "Half")
    h2.sigmoid(dh)
    want = oracle.pointwise(OP["SIGMOID"], np.zeros(h.shape, np.float16), [h])
    got = h2.numpy()
    assert_ulp(got, want, 1, "c4 half sigmoid")
    # mean and 2-norm along dim 0 with fp32 accumulation, compared on the GPU's own sigmoid output
    mean = thc.Tensor.new(state, "Half")
    mean.mean(h2, 0, 1)
    ssum = oracle.reduce_dim(RED["SUM"], 0, 0, got, 0)
    wmean = oracle.pointwise(OP["DIV_S"], np.zeros_like(ssum), [ssum], 8192)
    assert_reduction_close(mean.numpy(), wmean, 1e-3, np.abs(wmean.astype(np.float64)), "c4 half mean dim 0")
    norm = thc.Tensor.new(state, "Half")
    norm.norm(h2, 2, 0, 1)
    sq = oracle.reduce_dim(RED["SUM"], PRE["SQUARE"], 0, got, 0)
    wnorm = oracle.pointwise(OP["POW"], np.zeros_like(sq), [sq], 0.5)
    assert_reduction_close(norm.numpy(), wnorm, 1e-3, np.abs(wnorm.astype(np.float64)), "c4 half norm dim 0")


def test_c4_int_cmul_exact_sum(state, oracle):
    r = rng("c4.2")
    n = 134_217_728
    a = r.integers(-2**20, 2**20 + 1, n, dtype=np.int32)
    b = r.integers(-7, 8, n, dtype=np.int32)
    c = thc.Tensor.new(state, "Int")
    c.cmul(to_device(state, a), to_device(state, b))
    want = a * b
    assert_bit_equal(c.numpy(), want, "c4 int cmul")
    assert c.sumall() == int(want.astype(np.int64).sum())


def test_c4_double_sumall(state, oracle):
    r = rng("c4.3")
    d = r.uniform(0, 1, 134_217_728)
    dd = to_device(state, d)
    assert_reduction_close(dd.sumall(), oracle.reduce_all(RED["SUM"], 0, 0, d), 1e-12, d.sum(), "c4 double sumall")


def test_c5_full_size_properties(state, oracle):
    """2^32 elements per tensor on one GPU (64-bit indexing end to end).  Inputs are generated on
    the device; correctness is established on sampled rows (against the oracle) and by the
    checksum-of-checksums identity sum(z) == sum(row sums of z)."""
    torch = pytest.importorskip("torch")
    free, _ = torch.cuda.mem_get_info()
    if free < 60 * 2**30:
        pytest.skip("needs 50 GiB of free device memory")
    rows, cols = 524288, 8192
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    x = torch.empty(rows, cols, device=dev)
    y = torch.empty(rows, cols, device=dev)
    for r0 in range(0, rows, 16384):
        x[r0:r0 + 16384].normal_(generator=g)
        y[r0:r0 + 16384].normal_(generator=g)
    z = torch.empty(rows, cols, device=dev)
    state.set_stream(torch.cuda.current_stream().cuda_stream, 0)
    W = lambda t, kind: thc.Tensor.wrap(state, kind, t.data_ptr(), tuple(t.shape), tuple(t.stride()))
    tx, ty, tz = W(x, "Float"), W(y, "Float"), W(z, "Float")
    tz.cmul(tx, ty)
    assert plan_name() == "contig_vec"
    tz.add(tz, 1.0)
    v, i = thc.Tensor.new(state, "Float"), thc.Tensor.new(state, "Long")
    v.max(i, tz, 1, 1)
    total = tz.sumall()
    rowsum = thc.Tensor.new(state, "Float")
    rowsum.sum(tz, 1, 1)
    torch.cuda.synchronize()
    # sampled rows, including the first and the last (offsets beyond 2^32 elements)
    sample = [0, 1, 131071, 262144, 400000, rows - 2, rows - 1]
    xs = x[sample].cpu().numpy()
    ys = y[sample].cpu().numpy()
    zs = oracle.pointwise(OP["MUL"], np.zeros_like(xs), [xs, ys])
    zs = oracle.pointwise(OP["ADD_S"], zs, [zs], 1.0)
    assert_bit_equal(z[sample].cpu().numpy(), zs, "c5 z = x*y + 1 on sampled rows")
    wv, wi = oracle.reduce_dim(RED["MAX"], 0, 0, zs, 1, with_index=True)
    vs, is_ = v.numpy(), i.numpy()
    assert_bit_equal(vs[sample], wv, "c5 row max on sampled rows")
    assert_bit_equal(is_[sample], wi, "c5 row argmax on sampled rows")
    assert is_.min() >= 1 and is_.max() <= cols
    rs = rowsum.numpy().astype(np.float64)
    wrs = oracle.reduce_dim(RED["SUM"], 0, 0, zs, 1).astype(np.float64)
    assert_reduction_close(rs[sample], wrs, 1e-5, np.abs(zs.astype(np.float64)).sum(axis=1, keepdims=True), "c5 row sums")
    # checksum of checksums: the full reduction equals the sum of the row sums (each rounded to float)
    abs_bound = float(rows) * cols
    assert_reduction_close(total, rs.sum(), 1e-5, abs_bound, "c5 sum-all vs sum of row sums")
    del x, y, z
    torch.cuda.empty_cache()
