"""The C library's communicator (thcb200_comm_* / thcb200_sharded_*) with a single rank: NCCL is
bound, a communicator comes up, and the sharded calls reduce to the unsharded ones (the exchange
between ranks is checked on boxes with two or more GPUs by bench.py's `sharded_check`)."""
import ctypes as C

import numpy as np
import pytest

from cutorch_b200 import thc
from cutorch_b200._lib import RED
from cutorch_b200.shard import Comm
from common import assert_bit_equal, rng, to_device

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm(state):
    c = Comm(state, 1, 0)
    yield c
    c.close()


def test_communicator_reports_its_shape_and_nccl(comm):
    assert comm.nranks == 1 and comm.rank == 0
    assert comm.nccl_version() >= 22000


def test_sharded_calls_with_one_rank_equal_the_unsharded_ones(state, comm, oracle):
    r = rng("comm-one-rank")
    x = (r.integers(-1000, 1001, (300, 257)) / 8).astype(np.float32)
    x[17, 3] = np.nan
    dx = to_device(state, x)
    osum = thc.Tensor.new(state, "Float", 1, 257)
    comm.reduce_dim(osum, dx, 0, "SUM")
    assert_bit_equal(osum.numpy(), oracle.reduce_dim(RED["SUM"], 0, 0.0, x, 0), "sum along the sharded dim")
    v, i = thc.Tensor.new(state, "Float", 1, 257), thc.Tensor.new(state, "Long", 1, 257)
    comm.reduce_dim_index(v, i, dx, 0, 1000, "MAX")      # 1000 rows in front of this block
    wv, wi = oracle.reduce_dim(RED["MAX"], 0, 0.0, x, 0, with_index=True)
    assert_bit_equal(v.numpy(), wv, "max along the sharded dim")
    assert_bit_equal(i.numpy(), wi + 1000, "global positions")
    slot = thc.Tensor.new(state, "Double", 1)
    comm.reduce_all(dx, slot.data_ptr, "MAX")
    assert np.isnan(slot.numpy()[0])                      # a NaN wins, as in TH
    y = r.integers(-2**20, 2**20, 100003).astype(np.int32)
    islot = thc.Tensor.new(state, "Long", 1)
    comm.reduce_all(to_device(state, y), islot.data_ptr, "SUM")
    assert int(islot.numpy()[0]) == int(y.astype(np.int64).sum())
    # the overlapped mode and its wait are accepted with one rank too (there is nothing to overlap)
    comm.set_overlap(True)
    comm.reduce_all(to_device(state, y), islot.data_ptr, "SUM")
    comm.wait()
    comm.set_overlap(False)
    assert int(islot.numpy()[0]) == int(y.astype(np.int64).sum())


def test_all_reduce_and_bad_arguments(state, comm):
    lib = comm.lib
    buf = to_device(state, np.arange(8, dtype=np.float64))
    comm.all_reduce(buf.data_ptr, 8, 7, "SUM")           # one rank: unchanged
    assert_bit_equal(buf.numpy(), np.arange(8, dtype=np.float64), "all-reduce over one rank")
    rc = lib.thcb200_comm_all_reduce(comm.handle, C.c_void_p(buf.data_ptr), 8, 2, 0, C.c_void_p(state.stream))
    assert rc == -5      # int16 has no NCCL type
    handle = C.c_void_p()
    rc = lib.thcb200_comm_create(C.byref(handle), 2, 5, comm._id, 128)
    assert rc == -1 and b"rank 5 outside 2 ranks" in lib.thcb200_last_error()
