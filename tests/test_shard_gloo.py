"""The multi-process path on CPU: two gloo ranks shard a tensor by rows, each computes its block's
partials, and the collectives of cutorch_b200.shard combine them.  The per-block arithmetic is
done by the oracle here (no GPU in this test); what is under test is the host logic of the N > 1
path: block boundaries, the all-reduce of full-reduction partials, the all-reduce of a reduction
along the sharded dim, and the first-occurrence combine of (value, position) pairs."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from cutorch_b200.shard import combine_index_partials, combine_partials, shard_rows  # noqa: E402


def test_shard_rows_cover_everything_once():
    for total in (0, 1, 7, 8, 524288, 1000003):
        for world in (1, 2, 3, 4, 8):
            seen = 0
            for rank in range(world):
                start, count = shard_rows(total, world, rank)
                assert start == seen and count >= 0
                seen += count
            assert seen == total
            counts = [shard_rows(total, world, r)[1] for r in range(world)]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import Oracle
        from cutorch_b200._lib import OP, RED
        o = Oracle()
        rows, cols = 1001, 96   # odd row count: the blocks differ in size
        rng = np.random.default_rng(99)
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        y = (rng.integers(-3, 4, (rows, cols))).astype(np.float32)   # small value set: ties across blocks
        y[500, 7] = np.nan
        y[900, 7] = np.nan
        start, count = shard_rows(rows, world, rank)
        xs, ys = x[start:start + count], y[start:start + count]

        # pointwise + full reduction: z = x*y + 1 (NaNs cleaned for the sum), partials all-reduced
        z = np.zeros_like(xs)
        o.pointwise(OP["MUL"], z, [xs, np.nan_to_num(ys)])
        o.pointwise(OP["ADD_S"], z, [z], 1.0)
        partial = torch.tensor([o.reduce_all(RED["SUM"], 0, 0, z)], dtype=torch.float64)
        total = combine_partials(partial, "sum").item()

        # reduction along the sharded dim (dim 0): per-block column sums all-reduced
        col = torch.from_numpy(o.reduce_dim(RED["SUM"], 0, 0, xs, 0).astype(np.float64))
        col = combine_partials(col, "sum")
        colmax = torch.from_numpy(o.reduce_dim(RED["MAX"], 0, 0, xs, 0))
        colmax = combine_partials(colmax, "max")

        # max with positions along the sharded dim, ties and NaNs included
        v, p = o.reduce_dim(RED["MAX"], 0, 0, ys, 0, with_index=True)
        gv, gp = combine_index_partials(torch.from_numpy(v), torch.from_numpy(p), start, is_max=True)
        mv, mp_ = o.reduce_dim(RED["MIN"], 0, 0, ys, 0, with_index=True)
        gmv, gmp = combine_index_partials(torch.from_numpy(mv), torch.from_numpy(mp_), start, is_max=False)

        # row max along the unsharded dim stays local: gather the blocks only to check them
        rv, rp = o.reduce_dim(RED["MAX"], 0, 0, xs, 1, with_index=True)

        if rank == 0:
            zf = np.zeros_like(x)
            o.pointwise(OP["MUL"], zf, [x, np.nan_to_num(y)])
            o.pointwise(OP["ADD_S"], zf, [zf], 1.0)
            want_total = o.reduce_all(RED["SUM"], 0, 0, zf)
            ok = abs(total - want_total) <= 1e-9 * np.abs(zf).sum()
            want_col = o.reduce_dim(RED["SUM"], 0, 0, x, 0).astype(np.float64)
            ok &= bool(np.allclose(col.numpy(), want_col, rtol=1e-5, atol=1e-4))
            ok &= bool(np.array_equal(colmax.numpy(), o.reduce_dim(RED["MAX"], 0, 0, x, 0)))
            wv, wp = o.reduce_dim(RED["MAX"], 0, 0, y, 0, with_index=True)
            ok &= bool(np.array_equal(gp.numpy(), wp)) and bool(np.array_equal(np.isnan(gv.numpy()), np.isnan(wv)))
            ok &= bool(np.array_equal(np.nan_to_num(gv.numpy()), np.nan_to_num(wv)))
            wmv, wmp = o.reduce_dim(RED["MIN"], 0, 0, y, 0, with_index=True)
            ok &= bool(np.array_equal(gmp.numpy(), wmp)) and bool(np.array_equal(np.nan_to_num(gmv.numpy()), np.nan_to_num(wmv)))
            wrv, wrp = o.reduce_dim(RED["MAX"], 0, 0, x, 1, with_index=True)
            ok &= bool(np.array_equal(rv, wrv[start:start + count])) and bool(np.array_equal(rp, wrp[start:start + count]))
            results.put(("ok" if ok else "mismatch", float(total), float(want_total)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharded_reductions():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 300)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    status, total, want = q.get(timeout=10)
    assert status == "ok", (total, want)


def test_single_process_combine_is_identity():
    t = torch.tensor([3.5], dtype=torch.float64)
    assert combine_partials(t, "sum").item() == 3.5
    v, p = combine_index_partials(torch.tensor([1.0, 2.0]), torch.tensor([4, 1]), 10)
    assert v.tolist() == [1.0, 2.0] and p.tolist() == [14, 11]


def _worker_with_a_failing_rank(rank, world, port, results):
    """Rank 1 fails on the host between steps (an exception before its collective) and leaves; rank 0
    must come out of its collective with an error inside the process group's timeout, not wait for ever."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    partial = torch.tensor([float(rank + 1)], dtype=torch.float64)
    combine_partials(partial, "sum")          # a first step that works: 1 + 2
    assert partial.item() == 3.0
    if rank == 1:
        results.put(("rank1", "leaving"))
        results.close()
        results.join_thread()                 # the message is on its way before the process goes
        os._exit(17)                          # the rank dies without joining the next collective
    t0 = time.time()
    try:
        combine_partials(torch.tensor([1.0], dtype=torch.float64), "sum")
        results.put(("rank0", "no error", time.time() - t0))
    except Exception as e:                    # gloo reports the lost peer (or the timeout) as a RuntimeError
        results.put(("rank0", "error", time.time() - t0, type(e).__name__))
    results.close()
    results.join_thread()
    os._exit(0)


def test_a_rank_that_leaves_gives_the_others_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 90)
    procs = [ctx.Process(target=_worker_with_a_failing_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert p.exitcode is not None, "a rank is still waiting: the collective hung"
    got = {}
    while not q.empty():
        item = q.get(timeout=5)
        got[item[0]] = item[1:]
    assert got.get("rank1") == ("leaving",)
    assert got["rank0"][0] == "error", got
    assert got["rank0"][1] < 60, f"rank 0 needed {got['rank0'][1]:.0f} s to notice"
    assert procs[1].exitcode == 17 and procs[0].exitcode == 0
