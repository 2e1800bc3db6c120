"""Device-time measurements of the baseline configs c1-c4 (full size, one GPU), used by bench.py.

Each entry is one THC call timed with CUDA events on the launching stream; a read of a 512 MiB
buffer runs between timed iterations so that tensors that would fit the 126 MB L2 are read from
HBM (a read, not a memset: dirty lines of a written flush buffer would be written back during
the timed call).
`python bench.py --only c2,c3` runs a subset (that is also the small case the ncu captures use).
"""
from __future__ import annotations


def run_small_configs(torch, thc, state, stream, dev, peak, only=None, reps_override=None):
    def W(t, kind):
        w = thc.Tensor.wrap(state, kind, t.data_ptr(), tuple(t.shape), tuple(t.stride()))
        w._owner = t   # the wrapper holds a raw pointer: keep the torch tensor alive with it
        return w

    # The L2 is flushed by READING a buffer four times its size.  Writing one instead (a memset) leaves
    # up to 126 MB of dirty lines behind, and the timed call then pays for their write-back: measured
    # here, a 1 GiB fp64 sum-all read 175 us after a 512 MiB memset followed by a 256 MiB read, 156 us
    # after a read-only flush and 151 us in a back-to-back train.
    flush = torch.zeros(512 << 20, dtype=torch.uint8, device=dev)
    res_flush = torch.zeros(1, dtype=torch.int64, device=dev)
    tflush = W(flush, "Byte")
    torch.cuda.synchronize()

    def timed(fn, nbytes, reps=10, rot=None):
        reps = reps_override or reps
        ts = []
        for _ in range(3):
            fn()
        for _ in range(reps):
            # read 512 MiB (four times the L2) so that the operands of the timed call come from HBM
            tflush.sumall_to_device(res_flush.data_ptr())
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        med = ts[len(ts) // 2]
        gbs = nbytes / (med * 1e-3) / 1e9
        r = {"gbs": round(gbs, 1), "frac": round(gbs / peak, 4), "frac_of_nominal_8000": round(gbs / 8000.0, 4),
             "median_us": round(med * 1e3, 2), "best_us": round(ts[0] * 1e3, 2), "bytes": nbytes}
        if rot:
            # The same call back to back over rotating buffer sets (together larger than 4x the L2, so
            # every read comes from HBM), one event pair around the whole train: per-call time without
            # the cost of an event pair and an idle GPU around each launch.
            for f in rot:
                f()
            rounds = max(6, 24 // len(rot))
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record(stream)
            for _ in range(rounds):
                for f in rot:
                    f()
            b.record(stream)
            torch.cuda.synchronize()
            per = a.elapsed_time(b) / (rounds * len(rot))
            rg = nbytes / (per * 1e-3) / 1e9
            r.update({"back_to_back_gbs": round(rg, 1), "back_to_back_frac": round(rg / peak, 4),
                      "back_to_back_us": round(per * 1e3, 2), "buffer_sets": len(rot)})
            # the same train recorded once into a CUDA graph and replayed: no per-call host work
            side = torch.cuda.Stream(device=dev)
            didx = dev.index if dev.index is not None else 0
            state.set_stream(side.cuda_stream, didx)
            try:
                with torch.cuda.stream(side):
                    for f in rot:
                        f()
                    side.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        for f in rot:
                            f()
                    graph.replay()
                    side.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(side)
                    for _ in range(rounds):
                        graph.replay()
                    b.record(side)
                    side.synchronize()
                per = a.elapsed_time(b) / (rounds * len(rot))
                rg = nbytes / (per * 1e-3) / 1e9
                r.update({"graph_replay_gbs": round(rg, 1), "graph_replay_frac": round(rg / peak, 4),
                          "graph_replay_us": round(per * 1e3, 2)})
            finally:
                state.set_stream(stream.cuda_stream, didx)
        return r

    keep = []   # buffer sets of the back-to-back timings, dropped when their config is done
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    res = torch.zeros(1, dtype=torch.float64, device=dev)
    out = {}

    def c1():
        n = 16777216
        x = torch.empty(n, device=dev).uniform_(-1, 1, generator=g)
        y = torch.empty(n, device=dev).uniform_(-1, 1, generator=g)
        z = torch.empty(n, device=dev)
        tx, ty, tz = W(x, "Float"), W(y, "Float"), W(z, "Float")
        sets = [(W(x.clone(), "Float"), W(y.clone(), "Float"), W(torch.empty_like(z), "Float")) for _ in range(8)]
        keep.append(sets)
        out["c1_cadd_f32_16M"] = timed(lambda: tz.cadd(tx, 2.5, ty), 12 * n,
                                       rot=[(lambda s=s: s[2].cadd(s[0], 2.5, s[1])) for s in sets[:4]])
        out["c1_sumall_f32_16M"] = timed(lambda: tz.sumall_to_device(res.data_ptr()), 4 * n,
                                         rot=[(lambda s=s: s[0].sumall_to_device(res.data_ptr())) for s in sets])
        # the config as it is stated: z = x + 2.5 y, then the sum of that z (which the cadd has just left
        # in the L2); bytes of both calls, time of the pair
        def pair(s):
            s[2].cadd(s[0], 2.5, s[1])
            s[2].sumall_to_device(res.data_ptr())
        out["c1_chain_cadd_then_sumall"] = timed(lambda: pair((tx, ty, tz)), 16 * n, rot=[(lambda s=s: pair(s)) for s in sets[:4]])

    def c2():
        shape = (64, 256, 56, 56)
        n = 64 * 256 * 56 * 56
        x = torch.empty(shape, device=dev).normal_(generator=g)
        ybase = torch.empty(64, 56, 56, 256, device=dev).normal_(generator=g)
        yv = ybase.transpose(1, 3)
        wbase = torch.empty(64, 256, 56, 112, device=dev).normal_(generator=g)
        wv = wbase[..., ::2]
        o = torch.empty(shape, device=dev)
        to, tx, ty, tw = W(o, "Float"), W(x, "Float"), W(yv, "Float"), W(wv, "Float")
        out["c2_addcmul_f32_transposed_strided"] = timed(lambda: to.addcmul(tx, 0.5, ty, tw), 16 * n)

    def c3():
        m = (torch.randint(-1000, 1001, (32768, 8192), device=dev, generator=g).float() / 8)
        tm = W(m, "Float")
        n = m.numel()
        r1, r0 = torch.empty(32768, 1, device=dev), torch.empty(1, 8192, device=dev)
        i1 = torch.empty(32768, 1, dtype=torch.int64, device=dev)
        i0 = torch.empty(1, 8192, dtype=torch.int64, device=dev)
        tr1, tr0, ti1, ti0 = W(r1, "Float"), W(r0, "Float"), W(i1, "Long"), W(i0, "Long")
        tm2 = W(m.clone(), "Float")    # second buffer set of the back-to-back trains (2 GiB together)
        both = (tm, tm2)
        out["c3_sum_dim1"] = timed(lambda: tr1.sum(tm, 1, 1), 4 * n + 4 * 32768, rot=[(lambda t=t: tr1.sum(t, 1, 1)) for t in both])
        out["c3_sum_dim0"] = timed(lambda: tr0.sum(tm, 0, 1), 4 * n + 4 * 8192, rot=[(lambda t=t: tr0.sum(t, 0, 1)) for t in both])
        out["c3_max_dim1"] = timed(lambda: tr1.max(ti1, tm, 1, 1), 4 * n + 12 * 32768, rot=[(lambda t=t: tr1.max(ti1, t, 1, 1)) for t in both])
        out["c3_max_dim0"] = timed(lambda: tr0.max(ti0, tm, 0, 1), 4 * n + 12 * 8192, rot=[(lambda t=t: tr0.max(ti0, t, 0, 1)) for t in both])

    def c4():
        h = (torch.empty(8192, 8192, device=dev).normal_(0, 2, generator=g)).half()
        h2 = torch.empty_like(h)
        rh = torch.empty(1, 8192, dtype=torch.float16, device=dev)
        th, th2, trh = W(h, "Half"), W(h2, "Half"), W(rh, "Half")
        n = h.numel()
        hs = [(W(h.clone(), "Half"), W(torch.empty_like(h), "Half")) for _ in range(4)]
        keep.append(hs)
        out["c4_sigmoid_f16"] = timed(lambda: th2.sigmoid(th), 4 * n, rot=[(lambda s=s: s[1].sigmoid(s[0])) for s in hs])
        out["c4_mean_dim0_f16"] = timed(lambda: trh.mean(th2, 0, 1), 2 * n + 2 * 8192,
                                        rot=[(lambda s=s: trh.mean(s[0], 0, 1)) for s in hs])
        out["c4_norm2_dim0_f16"] = timed(lambda: trh.norm(th2, 2, 0, 1), 2 * n + 2 * 8192,
                                         rot=[(lambda s=s: trh.norm(s[0], 2, 0, 1)) for s in hs])
        # the config as it is stated: sigmoid, then mean and 2-norm along dim 0 of its result
        def chain(s):
            s[1].sigmoid(s[0])
            trh.mean(s[1], 0, 1)
            trh.norm(s[1], 2, 0, 1)
        out["c4_chain_sigmoid_mean_norm_f16"] = timed(lambda: chain((th, th2)), 4 * n + 2 * (2 * n + 2 * 8192),
                                                      rot=[(lambda s=s: chain(s)) for s in hs])
        keep.clear()
        del h, h2, hs
        n = 134217728
        a = torch.randint(-2**20, 2**20 + 1, (n,), dtype=torch.int32, device=dev, generator=g)
        b = torch.randint(-7, 8, (n,), dtype=torch.int32, device=dev, generator=g)
        c = torch.empty_like(a)
        ta, tb, tc = W(a, "Int"), W(b, "Int"), W(c, "Int")
        out["c4_cmul_i32_128M"] = timed(lambda: tc.cmul(ta, tb), 12 * n, reps=5)
        # the three 512 MiB tensors serve as the rotating sets of the back-to-back train (1.5 GiB together)
        out["c4_sumall_i32_128M"] = timed(lambda: tc.sumall_to_device(res.data_ptr()), 4 * n, reps=5,
                                          rot=[(lambda t=t: t.sumall_to_device(res.data_ptr())) for t in (tc, ta, tb)])
        del a, b, c, ta, tb, tc
        d = torch.empty(n, dtype=torch.float64, device=dev).uniform_(0, 1, generator=g)
        td, td2 = W(d, "Double"), W(d.clone(), "Double")
        out["c4_sumall_f64_128M"] = timed(lambda: td.sumall_to_device(res.data_ptr()), 8 * n, reps=5,
                                          rot=[(lambda t=t: t.sumall_to_device(res.data_ptr())) for t in (td, td2)])

    def nxt():
        """The callers either side of the path (comparisons into bytes, masks, scans, indexed moves,
        triangles, renorm), each on a tensor far larger than the L2.  Bytes are the compulsory
        reads and writes of the call; extra passes an implementation makes do not count."""
        n = 134217728
        x = torch.empty(n, device=dev).normal_(generator=g)
        tx = W(x, "Float")
        m = torch.empty(n, dtype=torch.uint8, device=dev)
        tm = W(m, "Byte")
        out["f1_gtValue_f32_to_byte_128M"] = timed(lambda: tx.call("gtValue", tm, tx, 0.0), 5 * n, reps=5)
        cnt = int(m.sum().item())
        y = x.clone()
        ty = W(y, "Float")
        out["f1_maskedFill_f32_128M_half_set"] = timed(lambda: ty.maskedFill(tm, 0.0), 9 * n, reps=5)
        sel = thc.Tensor.new(state, "Float")
        out["f1_maskedSelect_f32_128M_half_set"] = timed(lambda: sel.maskedSelect(tx, tm), 5 * n + 4 * cnt, reps=5)
        out["f2_cumsum_f32_1d_128M"] = timed(lambda: ty.cumsum(tx, 0), 8 * n, reps=5)
        del y, m
        mat = x.view(16384, 8192)
        mo = torch.empty_like(mat)
        tmat, tmo = W(mat, "Float"), W(mo, "Float")
        out["f2_cumsum_f32_16384x8192_dim1"] = timed(lambda: tmo.cumsum(tmat, 1), 8 * n, reps=5)
        out["f2_cumsum_f32_16384x8192_dim0"] = timed(lambda: tmo.cumsum(tmat, 0), 8 * n, reps=5)
        odd, oddo = x[: 16384 * 8191].view(16384, 8191), mo.view(-1)[: 16384 * 8191].view(16384, 8191)
        todd, toddo = W(odd, "Float"), W(oddo, "Float")
        out["f2_cumsum_f32_16384x8191_dim1_odd_rows"] = timed(lambda: toddo.cumsum(todd, 1), 8 * 16384 * 8191, reps=5)
        sq = x.view(-1)[: 11584 * 11584].view(11584, 11584)
        so = torch.empty_like(sq)
        tsq, tso = W(sq, "Float"), W(so, "Float")
        nsq = 11584 * 11584
        out["a5_tril_f32_11584x11584"] = timed(lambda: tso.tril(tsq, 0), 6 * nsq, reps=5)
        emb = x.view(524288, 256)
        eo = torch.empty_like(emb)
        temb, teo = W(emb, "Float"), W(eo, "Float")
        out["f2_renorm_f32_524288x256_dim0"] = timed(lambda: teo.renorm(temb, 2, 0, 15.0), 8 * n, reps=5)
        idx = torch.randint(1, 524288 + 1, (524288,), dtype=torch.int64, device=dev, generator=g)
        tidx = W(idx, "Long")
        out["f4_indexSelect_f32_524288_rows_of_256"] = timed(lambda: teo.indexSelect(temb, 0, tidx), 8 * n + 8 * 524288, reps=5)
        gi = torch.randint(1, 256 + 1, (524288, 256), dtype=torch.int64, device=dev, generator=g)
        tgi = W(gi, "Long")
        out["f4_gather_f32_524288x256_dim1"] = timed(lambda: teo.gather(temb, 1, tgi), (8 + 8) * n, reps=5)

    def generic():
        """Layouts that only the generic strided walk can take: rows of an odd length with an odd
        pitch (no 16-byte alignment from row to row), and three operands permuted three different ways."""
        R, Cc, pitch = 16384, 8191, 8195
        bufs = [torch.empty(R, pitch, device=dev).normal_(generator=g) for _ in range(3)]
        a, b, o = (t[:, :Cc] for t in bufs)
        ta, tb, to_ = W(a, "Float"), W(b, "Float"), W(o, "Float")
        n = R * Cc
        out["a4_cadd_f32_odd_rows_16384x8191_pitch_8195"] = timed(lambda: to_.cadd(ta, 2.5, tb), 12 * n, reps=5)
        base = [torch.empty(256, 512, 1024, device=dev).normal_(generator=g) for _ in range(3)]
        p0 = base[0]                                  # (256, 512, 1024) contiguous
        p1 = base[1].view(512, 256, 1024).transpose(0, 1)   # dims 0 and 1 swapped in memory
        p2 = base[2].view(256, 1024, 512).transpose(1, 2)   # dims 1 and 2 swapped in memory
        t0, t1, t2 = W(p0, "Float"), W(p1, "Float"), W(p2, "Float")
        n = p0.numel()
        out["a4_cmul_f32_three_permutations_256x512x1024"] = timed(lambda: t0.cmul(t1, t2), 12 * n, reps=5)
        del base, p0, p1, p2, t0, t1, t2
        # a window cut out of three larger 3-D tensors: three dims, none of them collapsible
        big = [torch.empty(258, 514, 1004, device=dev).normal_(generator=g) for _ in range(3)]
        w0, w1, w2 = (t[1:257, 1:513, 2:1002] for t in big)
        tw0, tw1, tw2 = W(w0, "Float"), W(w1, "Float"), W(w2, "Float")
        n = 256 * 512 * 1000
        out["a4_cmul_f32_window_256x512x1000_of_258x514x1004"] = timed(lambda: tw0.cmul(tw1, tw2), 12 * n, reps=5)
        # dimension reductions of a matrix with an odd number of columns (rows start at every alignment)
        om = bufs[0].view(-1)[: 16384 * 8191].view(16384, 8191)
        tom = W(om, "Float")
        oc, orow = torch.empty(1, 8191, device=dev), torch.empty(16384, 1, device=dev)
        oci = torch.empty(1, 8191, dtype=torch.int64, device=dev)
        toc, torow, toci = W(oc, "Float"), W(orow, "Float"), W(oci, "Long")
        no = 16384 * 8191
        out["a7_sum_dim0_f32_16384x8191_odd_columns"] = timed(lambda: toc.sum(tom, 0, 1), 4 * no, reps=5)
        out["a8_max_dim0_f32_16384x8191_odd_columns"] = timed(lambda: toc.max(toci, tom, 0, 1), 4 * no, reps=5)
        out["a7_sum_dim1_f32_16384x8191_odd_columns"] = timed(lambda: torow.sum(tom, 1, 1), 4 * no, reps=5)
        # dense 1-D runs that start one element past a 16-byte boundary
        flat = [t.view(-1)[1:1 + (1 << 27)] for t in big]
        tf0, tf1, tf2 = (W(t, "Float") for t in flat)
        out["a4_cadd_f32_1d_2p27_misaligned_by_one"] = timed(lambda: tf0.cadd(tf1, 2.5, tf2), 12 * (1 << 27), reps=5)
        out["a9_sumall_f32_1d_2p27_misaligned_by_one"] = timed(lambda: tf1.sumall_to_device(res.data_ptr()), 4 * (1 << 27), reps=5)
        # full reductions of views that are not one dense run
        out["a9_sumall_f32_window_256x512x1000"] = timed(lambda: tw0.sumall_to_device(res.data_ptr()), 4 * n, reps=5)
        tr = big[1].view(258 * 514, 1004).t()
        ttr = W(tr, "Float")
        out["a9_sumall_f32_transposed_1004x132612"] = timed(lambda: ttr.sumall_to_device(res.data_ptr()), 4 * tr.numel(), reps=5)
        rowsum = torch.empty(256, 512, 1, device=dev)
        trs = W(rowsum, "Float")
        out["a7_sum_dim2_f32_window_256x512x1000"] = timed(lambda: trs.sum(tw0, 2, 1), 4 * n, reps=5)
        colsum = torch.empty(1, 512, 1000, device=dev)
        tcs = W(colsum, "Float")
        out["a7_sum_dim0_f32_window_256x512x1000"] = timed(lambda: tcs.sum(tw0, 0, 1), 4 * n, reps=5)

    def xdev():
        """Copies from GPU 1 to GPU 0 over NVLink, driven from this process (needs two visible
        devices): a contiguous tensor (cudaMemcpyPeerAsync), a transposed source and a converting
        copy (the copy kernels run on the source GPU and store into the peer's memory).  Bytes are
        those that have to cross the link; the reference for the link is 770 GB/s per direction."""
        if torch.cuda.device_count() < 2:
            out["xdev"] = {"skipped": "needs two visible GPUs"}
            return
        n = 1 << 28
        dst = torch.empty(n, device=dev)
        torch.cuda.set_device(1)
        src = torch.empty(n, device="cuda:1").normal_()
        src_t = src.view(16384, 16384).t()
        src_h = src.half()
        torch.cuda.synchronize()
        torch.cuda.set_device(dev)
        tdst, tsrc = W(dst, "Float"), W(src, "Float")
        tdst2, tsrc_t, tsrc_h = W(dst.view(16384, 16384), "Float"), W(src_t, "Float"), W(src_h, "Half")
        link = 770.0

        def timed_x(fn, nbytes):
            ts = []
            for _ in range(2):
                fn()
            for _ in range(5):
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)      # the destination's stream waits for the copy, so its events bracket it
                fn()
                b.record(stream)
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            ts.sort()
            med = ts[len(ts) // 2]
            gbs = nbytes / (med * 1e-3) / 1e9
            return {"gbs": round(gbs, 1), "frac_of_nvlink_770": round(gbs / link, 4), "median_us": round(med * 1e3, 2), "bytes": nbytes}

        out["xdev_copy_f32_contiguous_1GiB"] = timed_x(lambda: tdst.copy(tsrc), 4 * n)
        out["xdev_copy_f32_transposed_source_1GiB"] = timed_x(lambda: tdst2.copy(tsrc_t), 4 * n)
        out["xdev_copy_f16_to_f32_2pow28"] = timed_x(lambda: tdst.copy_from(tsrc_h), 4 * n)

    def host():
        """Copies between CPU and GPU tensors (wall-clock: the calls block).  The CPU side is pinned
        memory (what cutorch's pinned host allocator gives); bytes = what crosses the bus."""
        import time
        import numpy as np
        n = 1 << 28
        hp = torch.empty(n, dtype=torch.float32).pin_memory()
        hp.uniform_(-1, 1)
        host32 = hp.numpy()
        host_t = host32.reshape(16384, 16384).T              # a transposed CPU view: packed on the host
        g32 = torch.empty(n, device=dev)
        g16t = torch.empty(16384, 16384, dtype=torch.float16, device=dev).t()
        t32, t16t = W(g32, "Float"), W(g16t, "Half")
        c32, ct = thc.CpuTensor(host32), thc.CpuTensor(host_t)

        def wall(fn, nbytes, reps=3):
            fn()
            ts = []
            for _ in range(reps):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn()
                ts.append(time.perf_counter() - t0)
            ts.sort()
            med = ts[len(ts) // 2]
            return {"gbs": round(nbytes / med / 1e9, 1), "median_ms": round(med * 1e3, 2), "bytes": nbytes}

        out["host_to_gpu_f32_dense_1GiB"] = wall(lambda: t32.copy_from_cpu(c32), 4 * n)
        out["host_to_gpu_f32_dense_into_f16_transposed"] = wall(lambda: t16t.copy_from_cpu(c32), 4 * n)
        out["gpu_to_host_f32_dense_1GiB"] = wall(lambda: t32.copy_to_cpu(c32), 4 * n)
        out["gpu_f16_transposed_to_host_f32_dense"] = wall(lambda: t16t.copy_to_cpu(c32), 4 * n)
        out["host_f32_transposed_view_to_gpu_dense"] = wall(lambda: t32.copy_from_cpu(ct), 4 * n, reps=1)

    def template():
        """The C++ template face (include/THC/THCApply.cuh, THCReduce.cuh) with user functors, through
        the test library built from tests/csrc/user_apply_test.cu: a scale functor on a contiguous and
        on a transposed 2^27-element fp32 tensor, and a user sum along each dim."""
        import ctypes as C
        from cutorch_b200.build import USERTEST_LIB
        if not USERTEST_LIB.exists():
            out["template"] = {"skipped": "the user-functor test library is not built"}
            return
        ulib = C.CDLL(str(USERTEST_LIB))
        ulib.usertest_scale.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float]
        ulib.usertest_scale.restype = C.c_int
        n = 1 << 27
        x = torch.empty(n, device=dev).normal_(generator=g)
        y = torch.empty(n, device=dev)
        tx, ty = W(x, "Float"), W(y, "Float")
        out["b_template_apply2_scale_f32_contiguous_128M"] = timed(
            lambda: ulib.usertest_scale(state.ptr, ty.ptr, tx.ptr, 1.5), 8 * n, reps=5)
        xt = x.view(8192, 16384).t()
        yt = y.view(16384, 8192)
        txt, tyt = W(xt, "Float"), W(yt, "Float")
        out["b_template_apply2_scale_f32_transposed_source_16384x8192"] = timed(
            lambda: ulib.usertest_scale(state.ptr, tyt.ptr, txt.ptr, 1.5), 8 * n, reps=5)
        # user reductions through THC_reduceDim / THC_reduceAll: a sum of squares along each dim, an absolute maximum
        ulib.usertest_sumsq_dim.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        ulib.usertest_sumsq_dim.restype = C.c_int
        ulib.usertest_absmax_all.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]
        ulib.usertest_absmax_all.restype = C.c_int
        m = x.view(16384, 8192)
        tm = W(m, "Float")
        r1, r0 = torch.empty(16384, 1, device=dev), torch.empty(1, 8192, device=dev)
        tr1, tr0 = W(r1, "Float"), W(r0, "Float")
        out["b_template_reduceDim_sumsq_f32_16384x8192_dim1"] = timed(lambda: ulib.usertest_sumsq_dim(state.ptr, tr1.ptr, tm.ptr, 1, 1), 4 * n, reps=5)
        out["b_template_reduceDim_sumsq_f32_16384x8192_dim0"] = timed(lambda: ulib.usertest_sumsq_dim(state.ptr, tr0.ptr, tm.ptr, 0, 1), 4 * n, reps=5)
        host_max = C.c_float(0)
        out["b_template_reduceAll_absmax_f32_128M_to_host"] = timed(lambda: ulib.usertest_absmax_all(state.ptr, tx.ptr, C.byref(host_max)), 4 * n, reps=5)

    # c1-c4 come last so that they are the end of the printed line
    for name, fn in (("next", nxt), ("generic", generic), ("xdev", xdev), ("host", host), ("template", template),
                     ("c1", c1), ("c2", c2), ("c3", c3), ("c4", c4)):
        if name in ("xdev", "host") and (only is None or name not in only):
            continue
        if only is None or name in only:
            fn()
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
    return out
