#!/usr/bin/env python
"""Benchmark of the THC apply / reduceDim / reduceAll path on B200.

Workload (config "c5" of the baseline): two fp32 tensors of 524288 x 8192 (2^32 elements,
16 GiB each), N(0,1), split by rows over the ranks.  One step, per rank, through the THC C API:
    THCudaTensor_cmul(z, x, y); THCudaTensor_add(z, z, 1); THCudaTensor_max(v, i, z, 1, 1);
    sum-all of z left on the device; NCCL all-reduce of the per-rank partials (N > 1).
metric = algorithmic HBM bytes of those four calls per second, summed over all ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Under torchrun every rank runs this file; rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS_TOTAL = 524288
COLS = 8192
# algorithmic bytes per element of one step (compulsory reads + writes of the logical elements):
# cmul 3*4, add in place 2*4, max read 4, sumall read 4; plus 12 bytes per row of max outputs
BYTES_PER_ELEM = 12 + 8 + 4 + 4
BYTES_PER_ROW_EXTRA = 12
CMUL_TRAFFIC_BYTES_PER_ELEM = (1073.752e6 + 497.472e6) / (16384 * 8192)
METRIC = "thc_apply_reduce_algorithmic_hbm_throughput"
UNIT = "GB/s"


def step_bytes(rows: int) -> int:
    return rows * COLS * BYTES_PER_ELEM + rows * BYTES_PER_ROW_EXTRA


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Samples taken before this call are dropped (nvidia-smi is started ahead of the timed
        region because it needs a moment to come up)."""
        self.first = len(self.lines)

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines[getattr(self, "first", 0):]:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the TH CPU restatement (oracle port) on the host cores
# --------------------------------------------------------------------------------------------
def cpu_step(oracle, np, x, y, z, v, i, OP, RED):
    """One step of the workload on host arrays through the oracle (all of its threads)."""
    oracle.pointwise(OP["MUL"], z, [x, y])
    oracle.pointwise(OP["ADD_S"], z, [z], 1.0)
    vv, ii = oracle.reduce_dim(RED["MAX"], 0, 0, z, 1, with_index=True)
    s = oracle.reduce_all(RED["SUM"], 0, 0, z)
    return vv, ii, s


def run_cpu(rows: int, steps: int, warmup: int, threads: int | None):
    import numpy as np
    from oracle import Oracle
    from cutorch_b200._lib import OP, RED
    o = Oracle()
    # all the host threads this process may run on (torchrun sets OMP_NUM_THREADS=1 for its
    # children, which would otherwise leave the CPU arm with one thread)
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    nthreads = threads or max(avail, o.max_threads())
    o.set_threads(nthreads)
    rng = np.random.default_rng(1234)
    x = rng.standard_normal((rows, COLS), dtype=np.float32)
    y = rng.standard_normal((rows, COLS), dtype=np.float32)
    z = np.empty_like(x)
    for _ in range(warmup):
        cpu_step(o, np, x, y, z, None, None, OP, RED)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(o, np, x, y, z, None, None, OP, RED)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return step_bytes(rows) / dt / 1e9, dt, nthreads


def host_description():
    """CPU model name and the number of hardware threads this process may use."""
    model = "unknown"
    try:
        with open("/proc/cpuinfo") as f:
            for ln in f:
                if ln.lower().startswith("model name"):
                    model = ln.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    return {"cpu_model": model, "nproc": os.cpu_count(), "usable_threads": avail}


def one_thread_baseline():
    """TH's own strided apply and reduce loops are serial: the same step on one host thread (2048 rows, 3 steps)."""
    gbs, _, _ = run_cpu(2048, 3, 1, 1)
    return {"value": gbs, "unit": UNIT, "cores": 1, "sample": f"2048 of {ROWS_TOTAL} rows x {COLS} (3 steps after 1 warm-up)"}


def reference_main(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    rows = 32768  # bounded sample: 1/16 of the rows per step, 1 GiB per tensor (about 0.3 s of host work per step)
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    gbs, dt, nthreads = run_cpu(rows, steps, warmup, None)
    sample = f"{rows} of {ROWS_TOTAL} rows x {COLS} per step ({steps} steps); GB/s is measured on the sample"
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        # measured: one step of the arm is one pass over the row sample; the full-size figure is a
        # separate, extrapolated key
        "warmup": warmup, "ms_per_step": dt * 1e3, "ms_per_step_full_size_extrapolated": dt * 1e3 * (ROWS_TOTAL / rows),
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c5: cmul, add 1, row max+argmax, sum-all on fp32 524288x8192 (row sample on the host)",
                   "impl_note": "TH CPU semantics restated in oracle/th_oracle.cpp (torch7's TH is not in the cutorch tree)"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": nthreads, "kind": "port", "sample": sample,
                         "one_thread": one_thread_baseline(), "host": host_description()},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def ours_main(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from cutorch_b200 import thc, _lib
    from cutorch_b200.shard import Comm, shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    row_start, rows = shard_rows(ROWS_TOTAL, world, rank)
    if args.rows:
        rows = args.rows
    n = rows * COLS

    state = thc.State()
    stream = torch.cuda.current_stream()
    state.set_stream(stream.cuda_stream, local)
    lib = _lib.load_library()
    # N > 1: the exchange runs inside the C library (NCCL bound by libthcb200); torch.distributed only
    # hands the NCCL id round and provides the barriers of the timing protocol
    comm = Comm.from_process_group(state) if world > 1 else None
    checks = multi_gpu_checks(np, torch, thc, state, comm, dev, world, rank, stream, args.collective) if world > 1 else {}
    peer_ok = checks.get("peer_check") == "ok"
    peer_on = peer_ok and args.collective == "peer"
    if peer_ok and not peer_on:
        comm.disable_peer_exchange()      # checked and available; the timed loop uses the collective asked for

    # synthetic inputs, generated on the device per shard from seed + rank
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    x = torch.empty(rows, COLS, dtype=torch.float32, device=dev)
    y = torch.empty(rows, COLS, dtype=torch.float32, device=dev)
    z = torch.empty(rows, COLS, dtype=torch.float32, device=dev)
    chunk = 8192
    for r0 in range(0, rows, chunk):
        x[r0:r0 + chunk].normal_(generator=g)
        y[r0:r0 + chunk].normal_(generator=g)
    v = torch.empty(rows, 1, dtype=torch.float32, device=dev)
    idx = torch.empty(rows, 1, dtype=torch.int64, device=dev)
    partial = torch.zeros(1, dtype=torch.float64, device=dev)

    tx = thc.Tensor.wrap(state, "Float", x.data_ptr(), (rows, COLS))
    ty = thc.Tensor.wrap(state, "Float", y.data_ptr(), (rows, COLS))
    tz = thc.Tensor.wrap(state, "Float", z.data_ptr(), (rows, COLS))
    tv = thc.Tensor.wrap(state, "Float", v.data_ptr(), (rows, 1))
    ti = thc.Tensor.wrap(state, "Long", idx.data_ptr(), (rows, 1))

    def step():
        tz.cmul(tx, ty)
        tz.add(tz, 1.0)
        tv.max(ti, tz, 1, 1)
        if comm is None:
            tz.sumall_to_device(partial.data_ptr())
        else:
            # the finishing CTA leaves this rank's double in `partial`; ncclAllReduce runs on that slot,
            # on the same stream, inside thcb200_sharded_reduce_all
            comm.reduce_all(tz, partial.data_ptr(), "SUM")

    def barrier():
        torch.cuda.synchronize()       # nothing of the library's communicator is in flight when torch's runs
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if comm is not None and not peer_on and not args.no_overlap:
        # the 8-byte all-reduce runs on the communicator's stream: the next step's kernels do not wait for it
        comm.set_overlap(True)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    if rank == 0:
        time.sleep(0.3)  # let nvidia-smi reach its sampling loop
        sampler.mark()
    launches0 = lib.thcb200_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    if comm is not None:
        comm.wait()                   # the timed region ends when the last all-reduce has landed
    e1.record(stream)
    barrier()
    launches = lib.thcb200_launch_count() - launches0
    lt = torch.tensor([launches], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(lt)
    launches = int(lt.item())
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    if peer_on:
        checks["peer_exchange_timed_out"] = bool(comm.peer_timed_out())     # must be False: a rank's wait never ran out
    total_sum = float(partial.item())
    if comm is not None and peer_ok:
        # the same loop with the other way of combining the partials, as an extra figure
        other = "nccl" if peer_on else "peer"
        if other == "peer":
            comm.set_overlap(False)
            comm.resume_peer_exchange()
        else:
            comm.disable_peer_exchange()
            comm.set_overlap(not args.no_overlap)
        for _ in range(2):
            step()
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for _ in range(args.steps):
            step()
        comm.wait()
        a1.record(stream)
        barrier()
        ta = torch.tensor([a0.elapsed_time(a1) / args.steps], dtype=torch.float64, device=dev)
        dist.all_reduce(ta, op=dist.ReduceOp.MAX)
        key = "peer_exchange" if other == "peer" else "nccl_overlapped"
        checks[key + "_ms_per_step"] = round(float(ta.item()), 4)
        if other == "peer":
            checks["peer_exchange_timed_out"] = bool(comm.peer_timed_out())
        # NCCL folds the ranks' doubles in its own order, the exchange in rank order: the totals agree to rounding
        checks["other_checksum_rel_diff"] = abs(float(partial.item()) - total_sum) / max(abs(total_sum), 1e-300)
        # back to the mode of the main loop for the legs that follow
        if other == "peer":
            comm.disable_peer_exchange()
            comm.set_overlap(not args.no_overlap)
        else:
            comm.set_overlap(False)
            comm.resume_peer_exchange()
    ms_per_step = ms / args.steps
    total_bytes = step_bytes(rows) * world
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # per-kernel durations (CUDA events on the launching stream), for the roofline of the dominant kernel
    def time_call(fn, reps):
        evs = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            evs.append((a, b))
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(b) for a, b in evs)
        return sum(ts) / len(ts), ts[0]

    reps = max(3, min(args.steps, 10))
    kernels = {}
    for name, fn, nbytes in (
        ("cmul contig_vec", lambda: tz.cmul(tx, ty), 12 * n),
        ("add_scalar contig_vec (in place)", lambda: tz.add(tz, 1.0), 8 * n),
        ("max+argmax dim1 row_warp", lambda: tv.max(ti, tz, 1, 1), 4 * n + 12 * rows),
        ("sumall reduce_all", lambda: tz.sumall_to_device(partial.data_ptr()), 4 * n),
    ):
        avg, best = time_call(fn, reps)
        kernels[name] = {"avg_ms": avg, "best_ms": best, "bytes": nbytes, "gbs": nbytes / (avg * 1e-3) / 1e9}
    peak, peak_src = measured_peaks()
    dom = kernels["cmul contig_vec"]
    roofline = {"bound": "hbm", "kernel": "apply_contig_vec_kernel<MUL,float,2> (THCudaTensor_cmul)",
                "achieved": dom["gbs"], "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                "frac": dom["gbs"] / peak, "frac_of_nominal_8000": dom["gbs"] / 8000.0,
                # dram__bytes_read + dram__bytes_write of this kernel from an ncu capture of a 16384-row
                # slice (11.71 B/element; traffic grows with the element count), scaled to the elements
                # of one launch here
                "traffic": int(CMUL_TRAFFIC_BYTES_PER_ELEM * n), "traffic_source": "ncu capture of a 16384-row slice, scaled by elements"}
    # flat scalar keys: per-kernel average duration and fraction of the peak for the four calls of a step
    for key, name in (("cmul", "cmul contig_vec"), ("add", "add_scalar contig_vec (in place)"),
                      ("max_dim1", "max+argmax dim1 row_warp"), ("sumall", "sumall reduce_all")):
        roofline[key + "_avg_ms"] = round(kernels[name]["avg_ms"], 4)
        roofline[key + "_frac"] = round(kernels[name]["gbs"] / peak, 4)
    roofline["kernels_sum_ms"] = round(sum(k["avg_ms"] for k in kernels.values()), 4)
    roofline["step_minus_kernels_us"] = round((ms_per_step - sum(k["avg_ms"] for k in kernels.values())) * 1e3, 2)

    # end to end: host (pinned) inputs -> device -> THC calls -> results back on the host
    e2e = None if args.no_e2e else run_e2e(args, torch, thc, state, stream, dev, rows, world, rank, comm, local)

    extra = {}
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        srows = 32768
        gbs, dt, nthreads = run_cpu(srows, 10, 1, None)
        cpu_baseline = {"value": gbs, "unit": UNIT, "cores": nthreads, "kind": "port",
                        "sample": f"{srows} of {ROWS_TOTAL} rows x {COLS} (10 steps after 1 warm-up), oracle/th_oracle.cpp with {nthreads} threads",
                        "one_thread": one_thread_baseline(), "host": host_description()}
    if rank == 0 and world == 1 and args.configs:
        from bench_configs import run_small_configs
        per_config = run_small_configs(torch, thc, state, stream, dev, peak)
        extra["per_config"] = per_config
        # the c1-c4 figures as flat scalar keys of `roofline`: fraction of the measured peak of the
        # flushed single call, its median, and the per-call time of a back-to-back train over rotating buffers
        # ... and the fractions of the rows around the path that were below 0.85 of the measured peak
        for name, short in (("f1_maskedSelect_f32_128M_half_set", "maskedSelect"), ("f2_cumsum_f32_1d_128M", "cumsum_1d_chunked"),
                            ("f2_cumsum_f32_16384x8192_dim0", "cumsum_dim0_chunked"),
                            ("a7_sum_dim0_f32_16384x8191_odd_columns", "sum_dim0_odd_width"),
                            ("a8_max_dim0_f32_16384x8191_odd_columns", "max_dim0_odd_width"),
                            ("b_template_apply2_scale_f32_contiguous_128M", "template_apply_contiguous"),
                            ("b_template_apply2_scale_f32_transposed_source_16384x8192", "template_apply_transposed"),
                            ("b_template_reduceDim_sumsq_f32_16384x8192_dim1", "template_reduce_dim1"),
                            ("b_template_reduceDim_sumsq_f32_16384x8192_dim0", "template_reduce_dim0"),
                            ("b_template_reduceAll_absmax_f32_128M_to_host", "template_reduce_all_to_host")):
            if name in per_config and "frac" in per_config[name]:
                roofline[short + "_frac"] = per_config[name]["frac"]
        for name, r in per_config.items():
            if not name.startswith(("c1_", "c2_", "c3_", "c4_")):
                continue
            short = name.replace("_f32_16M", "").replace("_f32_transposed_strided", "").replace("_128M", "").replace("_f16", "")
            roofline[short + "_frac"] = r["frac"]
            roofline[short + "_us"] = r["median_us"]
            if "back_to_back_us" in r:
                roofline[short + "_b2b_us"] = r["back_to_back_us"]
                roofline[short + "_b2b_frac"] = r["back_to_back_frac"]
    extra.update(checks)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "c5: THCudaTensor_cmul, _add(1), _max(dim 1, indices), sum-all + all-reduce of partials on fp32 "
                                   f"{ROWS_TOTAL}x{COLS} split by rows over {world} GPU(s)",
                       "rows_per_gpu": rows, "cols": COLS, "bytes_per_step": total_bytes,
                       "l2": "inputs (16 GiB per tensor at N=1) are far larger than the 126 MB L2; no flush needed",
                       "collective": ("none (one GPU)" if comm is None else
                                      "inside the reducing kernel: the finishing CTA stores the rank's accumulator into every rank's exchange "
                                      "block over NVLink (peer stores), waits with a bound for the others' and folds them in rank order "
                                      "(thcb200_sharded_reduce_all with the peer exchange on)" if peer_on else
                                      "ncclAllReduce(sum, 1 x f64) issued by thcb200_sharded_reduce_all on the slot the finishing CTA wrote, "
                                      + ("in the compute stream's order" if args.no_overlap else
                                         "on the communicator's own stream behind an event (the next step's kernels do not wait for it; "
                                         "the timed region ends after the last one)")
                                      + f" (NCCL {comm.nccl_version()} bound by libthcb200.so)"),
                       "elements_per_s": rows * COLS * world / (ms_per_step * 1e-3)},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks, "checksum": total_sum,
        }
        line.update(extra)
        print(json.dumps(line))
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def multi_gpu_checks(np, torch, thc, state, comm, dev, world, rank, stream, collective="nccl"):
    """Run before the timed region when there are two or more ranks (a one-GPU box cannot):
    copies between two GPUs of one process, and reductions along the SHARDED dim through the C
    library's communicator, each compared bit for bit with the unsharded result; then the time of the
    two sharded-dim reductions at the benchmark's shape."""
    import torch.distributed as dist
    out = {}
    T = thc.Tensor

    def wrap(t, kind):
        w = T.wrap(state, kind, t.data_ptr(), tuple(t.shape), tuple(t.stride()))
        w._owner = t
        return w

    # ---- copies from cuda:1 into cuda:0, driven by rank 0 (THCTensor_(copy) across devices) ----
    if rank == 0:
        try:
            verdict = "ok"
            if torch.cuda.device_count() < 2:
                verdict = "skipped: one visible device"
            else:
                r = np.random.default_rng(77)
                a = r.standard_normal((1024, 1536)).astype(np.float32)
                h = r.standard_normal((777, 333)).astype(np.float16)
                other = torch.device("cuda", 1 if dev.index == 0 else 0)
                src = torch.from_numpy(a).to(other)
                src_t = torch.from_numpy(np.ascontiguousarray(a.T)).to(other).t()     # a transposed view on the other GPU
                src_h = torch.from_numpy(h).to(other)
                torch.cuda.synchronize(other)
                for label, s_, kind, want in (("contiguous f32", src, "Float", a), ("transposed source f32", src_t, "Float", a),
                                              ("f16 -> f32", src_h, "Half", h.astype(np.float32))):
                    dst = torch.zeros(want.shape, dtype=torch.float32, device=dev)
                    td, ts = wrap(dst, "Float"), wrap(s_, kind)
                    if kind == "Float":
                        td.copy(ts)
                    else:
                        td.copy_from(ts)
                    torch.cuda.synchronize(dev)
                    got = dst.cpu().numpy()
                    if not np.array_equal(got.view(np.uint32), want.view(np.uint32)):
                        bad = np.argwhere(got != want)
                        verdict = f"{label}: {len(bad)} elements differ, first at {tuple(bad[0])}"
                        break
            out["xdev_check"] = verdict
        except Exception as e:   # the check reports, it does not end the benchmark
            out["xdev_check"] = f"error: {e}"
    dist.barrier()

    # ---- reductions along the sharded dim: a replicated-seed matrix split by rows ----
    try:
        rows_total, cols = 4096 + 3 * world, 2048
        r = np.random.default_rng(4242)
        full = (r.integers(-1000, 1001, (rows_total, cols)) / 8).astype(np.float32)   # exact sums, many ties
        full[rows_total // 2, 5] = np.nan
        from cutorch_b200.shard import shard_rows
        start, cnt = shard_rows(rows_total, world, rank)
        mine = torch.from_numpy(full[start:start + cnt]).to(dev)
        tm = wrap(mine, "Float")
        osum = torch.empty(1, cols, dtype=torch.float32, device=dev)
        omax = torch.empty(1, cols, dtype=torch.float32, device=dev)
        oidx = torch.empty(1, cols, dtype=torch.int64, device=dev)
        slot = torch.zeros(1, dtype=torch.float64, device=dev)
        comm.reduce_dim(wrap(osum, "Float"), tm, 0, "SUM")
        comm.reduce_dim_index(wrap(omax, "Float"), wrap(oidx, "Long"), tm, 0, start, "MAX")
        comm.reduce_all(tm, slot.data_ptr(), "MAX")     # a floating max over all ranks: the gather + fold path
        torch.cuda.synchronize(dev)
        verdict = "ok"
        if rank == 0:
            whole = torch.from_numpy(full).to(dev)
            tw = wrap(whole, "Float")
            wsum = torch.empty(1, cols, dtype=torch.float32, device=dev)
            wmax = torch.empty(1, cols, dtype=torch.float32, device=dev)
            widx = torch.empty(1, cols, dtype=torch.int64, device=dev)
            wslot = torch.zeros(1, dtype=torch.float64, device=dev)
            wrap(wsum, "Float").sum(tw, 0, 1)
            wrap(wmax, "Float").max(wrap(widx, "Long"), tw, 0, 1)
            lib = state.lib
            import ctypes as C
            from cutorch_b200 import _lib
            d = tw.descriptor()
            _lib.check(lib.thcb200_reduce_all(C.c_void_p(state.context), _lib.RED["MAX"], 0, _lib.scalar(0), C.byref(d),
                                              C.c_void_p(wslot.data_ptr()), C.c_void_p(state.stream)))
            torch.cuda.synchronize(dev)
            eq = lambda x, y: np.array_equal(x.cpu().numpy().view(np.uint8), y.cpu().numpy().view(np.uint8))
            # a column that holds the NaN sums to NaN both ways (the payload bits of a computed NaN are not
            # defined); every other sum is exact (multiples of 1/8) and has to agree bit for bit
            if not np.array_equal(osum.cpu().numpy(), wsum.cpu().numpy(), equal_nan=True):
                verdict = "sum along the sharded dim differs from the unsharded call"
            elif not eq(omax, wmax) or not eq(oidx, widx):
                verdict = "max / positions along the sharded dim differ from the unsharded call"
            elif not eq(slot, wslot):
                verdict = "sharded full max differs from the unsharded call"
        out["sharded_check"] = verdict
    except Exception as e:
        out["sharded_check"] = f"error: {e}"
    dist.barrier()

    # ---- the exchange through peer memory against NCCL's all-reduce: same data, same bits ----
    if True:
        try:
            vals = torch.from_numpy(np.nan_to_num(full[start:start + cnt])).to(dev)
            tvv = wrap(vals, "Float")
            by_nccl = torch.zeros(1, dtype=torch.float64, device=dev)
            by_peer = torch.zeros(1, dtype=torch.float64, device=dev)
            comm.reduce_all(tvv, by_nccl.data_ptr(), "SUM")
            why = comm.enable_peer_exchange()
            if why:
                out["peer_check"] = f"unavailable ({why}): the all-reduce stays with NCCL"
            else:
                for _ in range(3):       # three calls: both parities of the exchange blocks
                    comm.reduce_all(tvv, by_peer.data_ptr(), "SUM")
                torch.cuda.synchronize(dev)
                same = bool(by_nccl.item() == by_peer.item()) and not comm.peer_timed_out()
                agree = torch.tensor([1 if same else 0], device=dev)
                dist.all_reduce(agree, op=dist.ReduceOp.MIN)
                if int(agree.item()) == 1:
                    out["peer_check"] = "ok"
                else:
                    out["peer_check"] = f"differs from NCCL on some rank (here {by_peer.item()!r} vs {by_nccl.item()!r})"
                    comm.disable_peer_exchange()
        except Exception as e:
            out["peer_check"] = f"error: {e}"
        dist.barrier()

    # ---- the same two calls at the benchmark's shape: this rank's rows of 524288 x 8192 ----
    try:
        from cutorch_b200.shard import shard_rows
        start, cnt = shard_rows(ROWS_TOTAL, world, rank)
        big = torch.empty(cnt, COLS, dtype=torch.float32, device=dev).normal_()
        tb = wrap(big, "Float")
        osum = torch.empty(1, COLS, dtype=torch.float32, device=dev)
        oidx = torch.empty(1, COLS, dtype=torch.int64, device=dev)
        tsum, tidx = wrap(osum, "Float"), wrap(oidx, "Long")

        def timed(fn):
            for _ in range(2):
                fn()
            dist.barrier()
            torch.cuda.synchronize(dev)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(5):
                fn()
            b.record(stream)
            torch.cuda.synchronize(dev)
            t = torch.tensor([a.elapsed_time(b) / 5], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return round(float(t.item()), 4)

        out["sharded_sum_dim0_ms"] = timed(lambda: comm.reduce_dim(tsum, tb, 0, "SUM"))
        out["sharded_sum_dim0_local_only_ms"] = timed(lambda: tsum.sum(tb, 0, 1))
        out["sharded_max_dim0_ms"] = timed(lambda: comm.reduce_dim_index(tsum, tidx, tb, 0, start, "MAX"))
        out["sharded_max_dim0_local_only_ms"] = timed(lambda: tsum.max(tidx, tb, 0, 1))
        out["sharded_note"] = ("dim 0 of the row-sharded 524288 x 8192 tensor: local column reduction of this rank's rows, then "
                               "ncclAllReduce of 8192 floats (sum) or ncclAllGather of 8192 (value, position) pairs + combine (max)")
        del big
        torch.cuda.empty_cache()
    except Exception as e:
        out["sharded_timing_error"] = str(e)
    dist.barrier()
    return out


def run_e2e(args, torch, thc, state, stream, dev, rows, world, rank, comm, local):
    """Same step with HOST inputs: per row chunk, pinned host -> device copies, the four THC
    calls, and the row results plus the sum copied back, all inside the timed region.  The bytes
    cross through the library's own CPU <-> GPU tensor copies (THCudaTensor_copyAsyncCPU and
    TH<Type>Tensor_copyAsyncCuda, the calls under cutorch's :cuda() / :float()), issued on a copy
    stream that is made current for them; torch only allocates the buffers and records the events."""
    import torch.distributed as dist
    chunk = min(8192, rows)
    nchunks = rows // chunk
    # host side: one pinned chunk pair per slot, refilled from a host array standing for the
    # caller's data.  The host array is `host_rows` rows, cycled when the shard is larger than
    # what the box can pin.
    avail = 0
    try:
        for ln in open("/proc/meminfo"):
            if ln.startswith("MemAvailable"):
                avail = int(ln.split()[1]) * 1024
    except OSError:
        pass
    need = 2 * rows * COLS * 4
    budget = max(avail // (3 * max(world, 1)), 2 * chunk * COLS * 4)
    host_rows = rows if need <= budget else max(chunk, (budget // (2 * COLS * 4)) // chunk * chunk)
    hx = torch.empty(host_rows, COLS, dtype=torch.float32, pin_memory=True)
    hy = torch.empty(host_rows, COLS, dtype=torch.float32, pin_memory=True)
    g = torch.Generator(device=dev)
    g.manual_seed(2000 + rank)
    tmp = torch.empty(chunk, COLS, dtype=torch.float32, device=dev)
    for r0 in range(0, host_rows, chunk):
        tmp.normal_(generator=g)
        hx[r0:r0 + chunk].copy_(tmp)
        tmp.normal_(generator=g)
        hy[r0:r0 + chunk].copy_(tmp)
    hv = torch.empty(rows, 1, dtype=torch.float32, pin_memory=True)
    hi = torch.empty(rows, 1, dtype=torch.int64, pin_memory=True)
    hs = torch.empty(1, dtype=torch.float64, pin_memory=True)
    # the pinned arrays as TH CPU tensors (one per chunk of the inputs)
    cx = [thc.CpuTensor(hx[r0:r0 + chunk].numpy()) for r0 in range(0, host_rows, chunk)]
    cy = [thc.CpuTensor(hy[r0:r0 + chunk].numpy()) for r0 in range(0, host_rows, chunk)]
    chv, chi, chs = thc.CpuTensor(hv.numpy()), thc.CpuTensor(hi.numpy()), thc.CpuTensor(hs.numpy())
    nslots = 2
    dx = [torch.empty(chunk, COLS, dtype=torch.float32, device=dev) for _ in range(nslots)]
    dy = [torch.empty(chunk, COLS, dtype=torch.float32, device=dev) for _ in range(nslots)]
    dz = [torch.empty(chunk, COLS, dtype=torch.float32, device=dev) for _ in range(nslots)]
    dv = torch.empty(rows, 1, dtype=torch.float32, device=dev)
    di = torch.empty(rows, 1, dtype=torch.int64, device=dev)
    parts = torch.zeros(nchunks, dtype=torch.float64, device=dev)
    total = torch.zeros(1, dtype=torch.float64, device=dev)
    W = lambda t, kind, shape: thc.Tensor.wrap(state, kind, t.data_ptr(), shape)
    tx = [W(t, "Float", (chunk, COLS)) for t in dx]
    ty = [W(t, "Float", (chunk, COLS)) for t in dy]
    tz = [W(t, "Float", (chunk, COLS)) for t in dz]
    tvs = [W(dv[c * chunk:], "Float", (chunk, 1)) for c in range(nchunks)]
    tis = [W(di[c * chunk:], "Long", (chunk, 1)) for c in range(nchunks)]
    tdv, tdi, ttotal = W(dv, "Float", (rows, 1)), W(di, "Long", (rows, 1)), W(total, "Double", (1,))
    tparts = W(parts, "Double", (nchunks,))
    copy_stream = torch.cuda.Stream(device=dev)
    ready = [torch.cuda.Event() for _ in range(nslots)]
    freed = [torch.cuda.Event() for _ in range(nslots)]
    nhost = len(cx)

    def e2e_step():
        for c in range(nchunks):
            s = c % nslots
            if c >= nslots:
                copy_stream.wait_event(freed[s])
            # host -> device through the library, in the order of the copy stream
            state.set_stream(copy_stream.cuda_stream, local)
            tx[s].copy_async_from_cpu(cx[c % nhost])
            ty[s].copy_async_from_cpu(cy[c % nhost])
            state.set_stream(stream.cuda_stream, local)
            ready[s].record(copy_stream)
            stream.wait_event(ready[s])
            tz[s].cmul(tx[s], ty[s])
            tz[s].add(tz[s], 1.0)
            tvs[c].max(tis[c], tz[s], 1, 1)
            tz[s].sumall_to_device(parts[c:].data_ptr())
            freed[s].record(stream)
        if comm is None:
            tparts.sumall_to_device(total.data_ptr())
        else:
            comm.reduce_all(tparts, total.data_ptr(), "SUM")
            comm.wait()               # the total is read next
        # device -> host through the library, in the order of the compute stream
        tdv.copy_async_to_cpu(chv)
        tdi.copy_async_to_cpu(chi)
        ttotal.copy_async_to_cpu(chs)

    e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps = max(5, min(args.steps, 8))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(steps):
        e2e_step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    h2d = 2 * rows * COLS * 4
    d2h = rows * 12 + 8
    return {"value": step_bytes(rows) * world / (ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
            "d2h_bytes_per_step": d2h * world, "ms_per_step": ms, "steps": steps,
            "bound": f"pcie h2d, {h2d / (ms * 1e-3) / 1e9:.1f} GB/s per GPU: the step moves {h2d >> 20} MiB per GPU from host memory, "
                     "which takes longer than the kernels; the host link of the box, not the library, sets this number",
            "copies": "THCudaTensor_copyAsyncCPU / TH<Type>Tensor_copyAsyncCuda (the library's CPU <-> GPU tensor copies)",
            "host_rows_resident": host_rows, "note": "pinned host chunks of 8192 rows, double-buffered H2D overlapped with the kernels"
            + ("" if host_rows == rows else f"; host array of {host_rows} rows cycled (box cannot pin {need >> 30} GiB)")}


def only_main(args):
    """Times a subset of the c1-c4 configs on cuda:0 (the small case used for ncu captures)."""
    import torch
    from cutorch_b200 import thc
    from bench_configs import run_small_configs
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    state = thc.State()
    stream = torch.cuda.current_stream()
    state.set_stream(stream.cuda_stream, 0)
    peak, src = measured_peaks()
    res = run_small_configs(torch, thc, state, stream, dev, peak, only=set(args.only.split(",")), reps_override=args.reps or None)
    print(json.dumps({"per_config": res, "peak": peak, "peak_source": src}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU (default: 524288 / world size)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--configs", action="store_true", default=True, help="also time the c1-c4 configs at N=1")
    ap.add_argument("--no-configs", dest="configs", action="store_false")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-overlap", action="store_true", help="N > 1: run the all-reduce in the compute stream's order")
    ap.add_argument("--collective", default="nccl", choices=["peer", "nccl"],
                    help="N > 1, the timed loop: ncclAllReduce overlapped on the communicator's stream (default), or the exchange "
                         "inside the reducing kernel through peer memory (falls back to NCCL when the blocks cannot be mapped); "
                         "the other one is timed after the main loop and reported as an extra key")
    ap.add_argument("--only", default="", help="comma list of c1..c4: time just those configs on one GPU and print them")
    ap.add_argument("--reps", type=int, default=0, help="timed repetitions per entry with --only")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        return reference_main(args)
    if args.only:
        return only_main(args)
    return ours_main(args)


if __name__ == "__main__":
    sys.exit(main())
