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


# ---- exchange through peer memory, on one GPU: the other rank's part is played by the host -----------
class _Block(C.Structure):
    """ExchangeBlock of cutorch_b200/csrc/core.cuh: [parity][writer rank] accumulators and epochs, 16 ranks."""
    _fields_ = [("slot", (C.c_uint64 * 16) * 2), ("flag", (C.c_uint32 * 16) * 2)]


def _local_comm(state, nranks, rank, blocks, max_polls):
    lib = state.lib
    vp = C.c_void_p
    lib.thcb200_comm_create_local.argtypes = [C.POINTER(vp), C.c_int, C.c_int]
    lib.thcb200_comm_peer_block_bytes.restype = C.c_size_t
    lib.thcb200_comm_peer_attach_local.argtypes = [vp, C.POINTER(vp)]
    lib.thcb200_comm_set_peer_exchange.argtypes = [vp, C.c_int, C.c_uint]
    lib.thcb200_comm_peer_status.argtypes = [vp, C.POINTER(C.c_int), vp]
    lib.thcb200_comm_destroy.argtypes = [vp]
    lib.thcb200_comm_destroy.restype = None
    assert lib.thcb200_comm_peer_block_bytes() == C.sizeof(_Block)
    handle = vp()
    from cutorch_b200 import _lib
    _lib.check(lib.thcb200_comm_create_local(C.byref(handle), nranks, rank))
    arr = (vp * nranks)(*[b.data_ptr for b in blocks])
    _lib.check(lib.thcb200_comm_peer_attach_local(handle, arr))
    _lib.check(lib.thcb200_comm_set_peer_exchange(handle, 1, max_polls))
    return handle


def _sharded_sum(state, handle, x_dev, slot):
    from cutorch_b200 import _lib
    lib = state.lib
    lib.thcb200_sharded_reduce_all.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, _lib.Scalar, C.POINTER(_lib.TensorDesc), C.c_void_p, C.c_void_p]
    d = x_dev.descriptor()
    _lib.check(lib.thcb200_sharded_reduce_all(C.c_void_p(state.context), handle, RED["SUM"], 0, _lib.scalar(0), C.byref(d),
                                              C.c_void_p(slot.data_ptr), C.c_void_p(state.stream)))


def test_peer_exchange_folds_what_the_other_rank_left_and_gives_up_when_it_never_comes(state):
    """Two ranks, one GPU, one process: this process is rank 0; rank 1 never runs.  First its part of call 1
    (accumulator 1000.5, epoch 1) is written into rank 0's block from the host BEFORE the launch, so the
    finishing CTA finds it there: the result is the local sum plus 1000.5 and rank 0's own column shows up in
    rank 1's block.  Call 2 finds nothing from rank 1: the bounded wait runs out, the status word reports it,
    the slot holds rank 0's own sum, and the library works on.  No kernel here waits for another kernel."""
    r = rng("peer-exchange")
    x = (r.integers(-100, 101, 50000) / 4).astype(np.float32)          # exact sum
    local = float(x.astype(np.float64).sum())
    dx = to_device(state, x)
    nbytes = C.sizeof(_Block)
    blocks = [to_device(state, np.zeros(nbytes, np.uint8)) for _ in range(2)]
    handle = _local_comm(state, 2, 0, blocks, max_polls=2000)
    try:
        # rank 1's column of rank 0's block, parity 1 (epoch 1): accumulator then epoch
        host = _Block()
        host.slot[1][1] = np.float64(1000.5).view(np.uint64).item()
        host.flag[1][1] = 1
        raw = np.frombuffer(bytes(host), dtype=np.uint8).copy()
        blocks[0].copy_from_cpu(thc.CpuTensor(raw))
        slot = thc.Tensor.new(state, "Double", 1)
        _sharded_sum(state, handle, dx, slot)
        timed_out = C.c_int(-1)
        state.lib.thcb200_comm_peer_status(handle, C.byref(timed_out), C.c_void_p(state.stream))
        assert timed_out.value == 0
        assert slot.numpy()[0] == local + 1000.5
        theirs = _Block.from_buffer_copy(blocks[1].numpy().tobytes())
        assert theirs.flag[1][0] == 1 and np.uint64(theirs.slot[1][0]).view(np.float64) == local
        # call 2 (epoch 2, parity 0): nothing arrives from rank 1
        _sharded_sum(state, handle, dx, slot)
        state.lib.thcb200_comm_peer_status(handle, C.byref(timed_out), C.c_void_p(state.stream))
        assert timed_out.value == 1
        assert slot.numpy()[0] == local
        state.lib.thcb200_comm_peer_status(handle, C.byref(timed_out), C.c_void_p(state.stream))
        assert timed_out.value == 0           # reading the status clears it
        # the context is still usable
        assert float(dx.sumall()) == np.float32(local)
    finally:
        state.lib.thcb200_comm_destroy(handle)
