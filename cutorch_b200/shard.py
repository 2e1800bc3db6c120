"""Row sharding of the apply / reduce path over the GPUs of one box (one process per GPU).

Tensors are split along their outermost non-reduced dim into contiguous row blocks.  Pointwise
ops and reductions along a dim that is not sharded need no communication.  What crosses ranks is
tiny and goes through ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests):

* a full reduction: every rank's kernel leaves its accumulator (double / int64) on the device and
  the partials are all-reduced (8 bytes per rank);
* a reduction along the sharded dim: the per-rank outputs are all-reduced with the matching op;
* max / min with positions along the sharded dim: NCCL has no arg-reduce, so (value, global
  position) pairs are all-gathered and combined with the first-occurrence rule.

cutorch itself has no multi-process layer (it drives several devices from one process,
lib/THC/THCGeneral.h.in:57-123); this module exists for the sharded benchmark configuration.

On GPUs the exchange itself lives in the C library (`Comm`: thcb200_comm_* / thcb200_sharded_* in
include/thcb200.h, NCCL bound by the library); torch.distributed only carries the 128-byte NCCL id
from rank 0 to the others.  The torch.distributed functions below are the same rules on any
backend: the CPU double of the C layer, which the gloo tests run.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class Comm:
    """A communicator of the C library: one rank per GPU, this process's device current.

    `Comm.from_process_group(state)` bootstraps it over an initialised torch.distributed group (rank 0
    draws the NCCL id, a broadcast hands it round); `Comm(state, 1, 0)` is the single-rank form."""

    def __init__(self, state, nranks: int, rank: int, comm_id: bytes | None = None):
        import ctypes as C
        from . import _lib
        self.state, self.nranks, self.rank = state, nranks, rank
        self._C, self._lib_mod = C, _lib
        lib = self.lib = _lib.load_library()
        P, vp = C.POINTER, C.c_void_p
        lib.thcb200_comm_unique_id.argtypes = [vp, C.c_size_t]
        lib.thcb200_comm_create.argtypes = [P(vp), C.c_int, C.c_int, vp, C.c_size_t]
        lib.thcb200_comm_destroy.argtypes = [vp]
        lib.thcb200_comm_destroy.restype = None
        lib.thcb200_comm_info.argtypes = [vp, P(C.c_int), P(C.c_int), P(C.c_int)]
        lib.thcb200_comm_all_reduce.argtypes = [vp, vp, C.c_int64, C.c_int, C.c_int, vp]
        lib.thcb200_comm_peer_export.argtypes = [vp, vp, C.c_size_t]
        lib.thcb200_comm_peer_attach.argtypes = [vp, vp, C.c_size_t]
        lib.thcb200_comm_set_peer_exchange.argtypes = [vp, C.c_int, C.c_uint]
        lib.thcb200_comm_peer_status.argtypes = [vp, P(C.c_int), vp]
        lib.thcb200_comm_set_overlap.argtypes = [vp, C.c_int]
        lib.thcb200_comm_wait.argtypes = [vp, vp]
        lib.thcb200_comm_all_gather.argtypes = [vp, vp, vp, C.c_int64, vp]
        TD, SC = _lib.TensorDesc, _lib.Scalar
        lib.thcb200_sharded_reduce_all.argtypes = [vp, vp, C.c_int, C.c_int, SC, P(TD), vp, vp]
        lib.thcb200_sharded_reduce_dim.argtypes = [vp, vp, C.c_int, C.c_int, SC, P(TD), P(TD), C.c_int, vp]
        lib.thcb200_sharded_reduce_dim_index.argtypes = [vp, vp, C.c_int, P(TD), P(TD), P(TD), C.c_int, C.c_int64, vp]
        if comm_id is None:
            comm_id = self.new_id()
        self._id = C.create_string_buffer(comm_id, 128)
        handle = vp()
        _lib.check(lib.thcb200_comm_create(C.byref(handle), nranks, rank, self._id, 128))
        self.handle = handle

    @staticmethod
    def new_id() -> bytes:
        import ctypes as C
        from . import _lib
        lib = _lib.load_library()
        lib.thcb200_comm_unique_id.argtypes = [C.c_void_p, C.c_size_t]
        buf = C.create_string_buffer(128)
        _lib.check(lib.thcb200_comm_unique_id(buf, 128))
        return buf.raw

    @classmethod
    def from_process_group(cls, state, group=None) -> "Comm":
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        box = [cls.new_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=group)
        return cls(state, world, rank, box[0])

    def nccl_version(self) -> int:
        C = self._C
        v = C.c_int(0)
        self._lib_mod.check(self.lib.thcb200_comm_info(self.handle, None, None, C.byref(v)))
        return v.value

    def _ctx_stream(self):
        C = self._C
        return C.c_void_p(self.state.context), C.c_void_p(self.state.stream)

    def reduce_all(self, t, result_dev_ptr: int, rop: str = "SUM", pre: str = "IDENTITY", s=0):
        """Full reduction of a row-sharded tensor; the global accumulator (double / int64) lands at
        `result_dev_ptr` on every rank."""
        C, L = self._C, self._lib_mod
        ctx, st = self._ctx_stream()
        d = t.descriptor()
        L.check(self.lib.thcb200_sharded_reduce_all(ctx, self.handle, L.RED[rop], L.PRE[pre], L.scalar(s), C.byref(d),
                                                    C.c_void_p(result_dev_ptr), st))

    def reduce_dim(self, out, t, dim: int, rop: str = "SUM", pre: str = "IDENTITY", s=0):
        """Reduction along the sharded dim `dim`; `out` (dense, size 1 there) holds the global result on every rank."""
        C, L = self._C, self._lib_mod
        ctx, st = self._ctx_stream()
        do, di = out.descriptor(), t.descriptor()
        L.check(self.lib.thcb200_sharded_reduce_dim(ctx, self.handle, L.RED[rop], L.PRE[pre], L.scalar(s), C.byref(do), C.byref(di), dim, st))

    def reduce_dim_index(self, values, indices, t, dim: int, shard_start: int, rop: str = "MAX"):
        """max / min with global 1-based positions along the sharded dim."""
        C, L = self._C, self._lib_mod
        ctx, st = self._ctx_stream()
        dv, dx, di = values.descriptor(), indices.descriptor(), t.descriptor()
        L.check(self.lib.thcb200_sharded_reduce_dim_index(ctx, self.handle, L.RED[rop], C.byref(dv), C.byref(dx), C.byref(di), dim,
                                                          shard_start, st))

    def all_reduce(self, dev_ptr: int, count: int, dtype: int, rop: str = "SUM"):
        C, L = self._C, self._lib_mod
        L.check(self.lib.thcb200_comm_all_reduce(self.handle, C.c_void_p(dev_ptr), count, dtype, L.RED[rop], C.c_void_p(self.state.stream)))

    def enable_peer_exchange(self, group=None, max_polls: int = 0) -> str:
        """Full reductions exchange their accumulators through peer memory from now on, inside the reducing
        kernel (thcb200_comm_peer_export / _attach / _set_peer_exchange): every rank exports a handle of its
        exchange block, torch.distributed gathers the handles, every rank maps the others' blocks.  Returns ""
        when every rank succeeded; otherwise the first rank's reason, with the exchange left off everywhere
        (all ranks take the same decision)."""
        C = self._C

        def agree(err):
            errs = [None] * self.nranks
            dist.all_gather_object(errs, err, group=group)
            return next((f"rank {r}: {e}" for r, e in enumerate(errs) if e), "")

        mine = C.create_string_buffer(64)
        rc = self.lib.thcb200_comm_peer_export(self.handle, mine, 64)
        why = agree(self.lib.thcb200_last_error().decode() if rc else "")
        if why:
            return why
        handles = [None] * self.nranks
        dist.all_gather_object(handles, mine.raw, group=group)
        table = C.create_string_buffer(b"".join(handles), 64 * self.nranks)
        rc = self.lib.thcb200_comm_peer_attach(self.handle, table, 64)
        why = agree(self.lib.thcb200_last_error().decode() if rc else "")      # also: every block is mapped everywhere
        if why:
            return why
        self._lib_mod.check(self.lib.thcb200_comm_set_peer_exchange(self.handle, 1, max_polls))
        return ""

    def disable_peer_exchange(self):
        self._lib_mod.check(self.lib.thcb200_comm_set_peer_exchange(self.handle, 0, 0))

    def resume_peer_exchange(self):
        """Switches the exchange back on after disable_peer_exchange (the blocks stay mapped)."""
        self._lib_mod.check(self.lib.thcb200_comm_set_peer_exchange(self.handle, 1, 0))

    def peer_timed_out(self) -> bool:
        """Waits for the current stream; True when an exchange gave up waiting for a rank since the last call."""
        C = self._C
        v = C.c_int(0)
        self._lib_mod.check(self.lib.thcb200_comm_peer_status(self.handle, C.byref(v), C.c_void_p(self.state.stream)))
        return bool(v.value)

    def set_overlap(self, on: bool):
        """Full reductions all-reduce on the communicator's own stream from now on (see thcb200_comm_set_overlap)."""
        self._lib_mod.check(self.lib.thcb200_comm_set_overlap(self.handle, int(on)))

    def wait(self):
        """The current stream waits for the last overlapped all-reduce."""
        self._lib_mod.check(self.lib.thcb200_comm_wait(self.handle, self._C.c_void_p(self.state.stream)))

    def close(self):
        if self.handle:
            self.lib.thcb200_comm_destroy(self.handle)
            self.handle = None


def shard_rows(total_rows: int, world: int, rank: int) -> tuple[int, int]:
    """(first row, row count) of `rank`'s block; the first `total_rows % world` ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside a world of {world}")
    base, extra = divmod(total_rows, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


_REDUCE_OPS = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}


def combine_partials(partial: torch.Tensor, op: str = "sum", group=None) -> torch.Tensor:
    """All-reduces per-rank accumulators in place (a full reduction, or the outputs of a
    reduction along the sharded dim).  A single-process run returns the tensor unchanged."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=_REDUCE_OPS[op], group=group)
    return partial


def combine_index_partials(values: torch.Tensor, positions: torch.Tensor, shard_start: int, is_max: bool = True,
                           group=None, state=None) -> tuple[torch.Tensor, torch.Tensor]:
    """max / min with 1-based positions along the sharded dim.

    `values` / `positions` are this rank's results over its own block (positions 1-based inside
    the block).  Returns the global values and 1-based global positions on every rank: the largest
    (smallest) value wins, a NaN beats any number, and among equals the lowest global position --
    the result of one scan over the unsharded dim."""
    gpos = positions + shard_start
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return values, gpos
    world = dist.get_world_size(group)
    vs = [torch.empty_like(values) for _ in range(world)]
    ps = [torch.empty_like(gpos) for _ in range(world)]
    dist.all_gather(vs, values.contiguous(), group=group)
    dist.all_gather(ps, gpos.contiguous(), group=group)
    return combine_gathered(torch.stack(vs), torch.stack(ps), is_max, state)


_KIND_OF_TORCH = {torch.uint8: "Byte", torch.int8: "Char", torch.int16: "Short", torch.int32: "Int", torch.int64: "Long",
                  torch.float16: "Half", torch.float32: "Float", torch.float64: "Double"}


def combine_gathered(vals: torch.Tensor, poss: torch.Tensor, is_max: bool = True, state=None):
    """Combines per-rank (value, global position) pairs stacked along dim 0 (rank order = block
    order) into the values and positions one scan over the unsharded dim would give.

    With a THC `state` and CUDA tensors the combine runs on this library's kernels: a max / min
    with positions along dim 0 (first occurrence, a NaN wins: the rule of the unsharded call, and
    the lowest rank among equals is the lowest global position) followed by a gather of the
    positions.  Without one (the CPU tests) the same rule is applied with torch operations."""
    if state is not None and vals.is_cuda:
        from . import thc

        def wrap(t, kind):
            w = thc.Tensor.wrap(state, kind, t.data_ptr(), tuple(t.shape), tuple(t.stride()))
            w._owner = t
            return w
        vals, poss = vals.contiguous(), poss.contiguous()
        kind = _KIND_OF_TORCH[vals.dtype]
        best_v = torch.empty((1,) + tuple(vals.shape[1:]), dtype=vals.dtype, device=vals.device)
        which = torch.empty((1,) + tuple(vals.shape[1:]), dtype=torch.int64, device=vals.device)
        best_p = torch.empty_like(which)
        tv, tw = wrap(best_v, kind), wrap(which, "Long")
        (tv.max if is_max else tv.min)(tw, wrap(vals, kind), 0, 1)
        wrap(best_p, "Long").gather(wrap(poss, "Long"), 0, tw)
        return best_v[0], best_p[0]
    best_v, best_p = vals[0].clone(), poss[0].clone()
    for v, p in zip(vals[1:], poss[1:]):
        if vals.is_floating_point():
            bn, vn = torch.isnan(best_v), torch.isnan(v)
        else:
            bn = vn = torch.zeros_like(v, dtype=torch.bool)
        better = (v > best_v) if is_max else (v < best_v)
        # ranks are visited in block order, so on ties the earlier (lower position) entry stays
        take = (~bn) & (vn | better)
        best_v = torch.where(take, v, best_v)
        best_p = torch.where(take, p, best_p)
    return best_v, best_p
