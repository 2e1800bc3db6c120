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
"""
from __future__ import annotations

import torch
import torch.distributed as dist


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
