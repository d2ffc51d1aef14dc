"""Benchmark of the legacy-op hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is the elementwise chain on float32 [16384, 4096]:
    execBroadcast Add of a [4096] row vector  ->  execTransform Tanh  ->  execPairwiseTransform Multiply
(x ~ N(0,1) seed 1, b ~ N(0,1) seed 2, y ~ U(0,1) seed 3). The headline value is array elements
pushed through the chain per second, summed over all GPUs (each rank owns its own arrays: weak
scaling, no data-path collective). Besides the contract keys the JSON line carries the roofline
of the dominant kernel, a CPU baseline (the reference's own OpenMP loops on a bounded sample),
the end-to-end number through host buffers, and a `families` table with the achieved HBM GB/s of
the other op families at their configured sizes.

With --impl reference the reference's CPU implementation (oracle/_ref) is timed instead.
Under torchrun every rank runs the GPU arm; rank 0 prints the line.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS = 16384, 4096
ELEMS = ROWS * COLS
# algorithmic bytes per launch: operands read once + result written once
BYTES = {"broadcast_add": 2 * ELEMS * 4 + COLS * 4, "transform_tanh": 2 * ELEMS * 4, "pairwise_mul": 3 * ELEMS * 4}
METRIC = "elementwise chain throughput (broadcast Add -> Tanh -> pairwise Multiply, f32 [16384,4096])"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs", 6650.0), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback 6.65 TB/s"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the benchmark's kernels run: through NVML
    (read-only queries every ~2 ms from a thread) when the bindings are importable, else by
    parsing `nvidia-smi -lms`."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []        # (arrival time, sm MHz, max sm MHz, set of reasons)
        self.proc = None
        self.thread = None
        self.running = False
        self.source = None
        self.window = [None, None]

    def _visible_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._visible_index())
            self.source = "nvml"
            self.running = True
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
        except Exception:
            self._start_smi()
        t0 = time.monotonic()
        while not self.samples and time.monotonic() - t0 < 3.0:
            time.sleep(0.01)

    def _poll_nvml(self):
        n = self.nvml
        mx = float(n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM))
        bits = (("hw_slowdown", n.nvmlClocksThrottleReasonHwSlowdown),
                ("hw_thermal_slowdown", n.nvmlClocksThrottleReasonHwThermalSlowdown),
                ("sw_thermal_slowdown", n.nvmlClocksThrottleReasonSwThermalSlowdown),
                ("sw_power_cap", n.nvmlClocksThrottleReasonSwPowerCap))
        while self.running:
            try:
                sm = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((time.monotonic(), sm, mx, {name for name, bit in bits if mask & bit}))
            except Exception:
                pass
            time.sleep(0.002)

    def _start_smi(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self._visible_index()), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
            threading.Thread(target=self._pump_smi, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump_smi(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.strip().split(",")]
            if len(parts) < 9:
                continue
            try:
                sm, mx = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            self.samples.append((time.monotonic(), sm, mx,
                                 {n for n, v in zip(names, parts[5:9]) if v.lower().startswith("active")}))

    def mark_begin(self):
        self.window[0] = time.monotonic()

    def mark_end(self):
        self.window[1] = time.monotonic()

    def stop(self):
        """Summary over the samples taken between mark_begin() and mark_end() (the timed region);
        when the region was too short to catch one, over all samples taken while this benchmark's
        kernels ran (warm-up through the per-kernel timings), and `scope` says which."""
        self.running = False
        if self.thread is not None:
            self.thread.join(timeout=1.0)
        if self.proc is not None:
            time.sleep(0.05)
            self.proc.terminate()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock samples"], "samples": 0}
        w0, w1 = self.window
        inside = [s for s in self.samples if w0 is not None and w1 is not None and w0 <= s[0] <= w1]
        use = inside if inside else self.samples
        reasons = set()
        for s in use:
            reasons |= s[3]
        return {"sm_mhz": float(np.median([s[1] for s in use])), "sm_max_mhz": max(s[2] for s in use),
                "reasons": sorted(reasons), "samples": len(use), "scope": "timed region" if inside else "whole run",
                "source": self.source}


def host_threads():
    """Threads for the CPU arms: the physical cores this process may run on (hyper-threads add nothing to
    these streaming loops). Set explicitly because launchers such as torchrun export OMP_NUM_THREADS=1."""
    allowed = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        import psutil
        physical = psutil.cpu_count(logical=False) or allowed
    except Exception:
        physical = allowed
    return max(1, min(allowed, physical))


def make_inputs(rows):
    x = np.random.default_rng(1).standard_normal((rows, COLS), dtype=np.float32)
    b = np.random.default_rng(2).standard_normal(COLS, dtype=np.float32)
    y = np.random.default_rng(3).random((rows, COLS), dtype=np.float32)
    return x, b, y


# ------------------------------------------------------------------------------------------------
def cpu_reference_chain(rows, repeats, threads=None, use_port=False):
    """Times the reference's CPU loops (or, with use_port, the oracle's C restatement of them) on `rows` rows of
    the workload. Returns (Gelem/s, cores, seconds of the best pass)."""
    from libnd4j_b200 import shape as S
    if use_port:
        from oracle import port
        ref = port.Port()
    else:
        from oracle import reference
        ref = reference.Reference()
    if threads:
        ref.set_threads(threads)
    cores = ref.threads()
    x, b, y = make_inputs(rows)
    xi, bi = S.shape_info([rows, COLS]), S.shape_info([1, COLS])
    xf, yf = x.ravel(), y.ravel()
    t1, t2, t3 = (np.empty(rows * COLS, np.float32) for _ in range(3))
    best = None
    for _ in range(repeats + 1):   # first pass warms pages and the OpenMP pool
        t0 = time.perf_counter()
        ref.broadcast(0, xf, xi, b, bi, t1, xi, [1])
        ref.transform(15, t1, xi, t2, xi)
        ref.pairwise(6, t2, xi, yf, xi, t3, xi)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return rows * COLS / best / 1e9, cores, best


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import reference
    from libnd4j_b200 import shape as S
    if reference.available():
        rows = ROWS   # the whole configured array: about 0.1 s per step on a multi-core host
        ref, kind = reference.Reference(), "reference"
        what = "reference CPU loops (OpenMP)"
    else:
        # the reference's own build is absent: time the oracle's scalar C restatement of the same loops on a
        # bounded sample instead
        rows = 2048
        from oracle import port
        ref, kind = port.Port(), "port"
        what = "oracle port of the reference CPU loops"
    ref.set_threads(host_threads())
    cores = ref.threads()
    x, b, y = make_inputs(rows)
    xi, bi = S.shape_info([rows, COLS]), S.shape_info([1, COLS])
    xf, yf = x.ravel(), y.ravel()
    t1, t2, t3 = (np.empty(rows * COLS, np.float32) for _ in range(3))

    def step():
        ref.broadcast(0, xf, xi, b, bi, t1, xi, [1])
        ref.transform(15, t1, xi, t2, xi)
        ref.pairwise(6, t2, xi, yf, xi, t3, xi)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = rows * COLS / dt / 1e9
    sample = "%d of %d rows per step, %s, %d threads" % (rows, ROWS, what, cores)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "Gelem/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "elementwise chain f32 [16384,4096]: execBroadcast Add(dim 1) -> execTransform Tanh -> "
                               "execPairwiseTransform Multiply" + ("" if rows == ROWS else " (sampled: %d rows)" % rows)},
        "cpu_baseline": {"value": value, "unit": "Gelem/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "Gelem/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------
class Calls:
    """Pre-marshalled C-ABI calls so that the per-launch host cost is one ctypes call."""

    def __init__(self, ops, stream):
        self.lib = ops.lib
        self.stream = ctypes.c_void_p(stream)
        self.keep = []

    def longs(self, a):
        arr = np.ascontiguousarray(a, dtype=np.int64)
        self.keep.append(arr)
        return arr.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))

    def ints(self, a):
        arr = np.ascontiguousarray(a, dtype=np.int32)
        self.keep.append(arr)
        return arr.ctypes.data_as(ctypes.POINTER(ctypes.c_int))

    @staticmethod
    def p(t):
        return ctypes.c_void_p(t.data_ptr()) if t is not None else None

    def check(self, code):
        if code != 0:
            raise RuntimeError(self.lib.nd4jb200_last_error().decode())


def time_loop(torch, stream, fn, iters):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(iters):
        fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop) / iters


def time_graph(torch, stream, fn, iters, replays=5):
    """Average duration of one launch with the launches captured into a CUDA graph, so that the
    host's per-call cost and most of the inter-kernel gap stay out of the measurement. Only for
    calls that neither synchronise nor allocate (the workspace is warm by then)."""
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(replays):
            graph.replay()
        stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop) / (iters * replays)


def family_table(torch, ops, calls, stream, peak, quick, only=None, profile=False):
    """Achieved HBM GB/s of the other op families at their configured sizes (algorithmic bytes /
    CUDA-event time, inputs larger than L2 or L2 flushed by the rotation of buffers)."""
    from libnd4j_b200 import shape as S
    lib, st, P = calls.lib, calls.stream, calls.p
    out = {}
    dev = torch.device("cuda")

    def record(name, nbytes, elems, fn, iters=20, graph=True):
        if only and not any(part in name for part in only.split(",")):
            return
        if profile:
            iters = min(iters, 3)
        for _ in range(3):
            fn()
        ms = time_graph(torch, stream, fn, iters) if (graph and not profile) else time_loop(torch, stream, fn, iters)
        out[name] = {"ms": round(ms, 5), "GBps": round(nbytes / ms / 1e6, 1), "frac_of_measured_peak": round(nbytes / ms / 1e6 / peak, 3),
                     "Gelem_s": round(elems / ms / 1e6, 2)}

    g = torch.Generator(device=dev)
    g.manual_seed(0)
    # reduce Sum along dimension 1, [8192,4096]; several input copies rotate so L2 never holds the input
    xs = [torch.empty(8192, 4096, device=dev).uniform_(-1, 1, generator=g) for _ in range(3)]
    z = torch.zeros(8192, device=dev)
    xi, zi, d1 = calls.longs(S.shape_info([8192, 4096])), calls.longs(S.shape_info([8192, 1])), calls.ints([1])
    k = [0]

    def f():
        k[0] = (k[0] + 1) % 3
        calls.check(lib.nd4jb200_exec_reduce(st, 0, 1, P(xs[k[0]]), xi, None, P(z), zi, d1, 1))
    record("reduce_sum_dim1_8192x4096", 134250496, 8192 * 4096, f)
    z0 = torch.zeros(4096, device=dev)
    zi0, d0 = calls.longs(S.shape_info([1, 4096])), calls.ints([0])

    def f():
        k[0] = (k[0] + 1) % 3
        calls.check(lib.nd4jb200_exec_reduce(st, 0, 1, P(xs[k[0]]), xi, None, P(z0), zi0, d0, 1))
    record("reduce_sum_dim0_8192x4096", 134234112, 8192 * 4096, f)
    del xs
    # index reduce IMax dim 1 and summary-stats variance dim 0 on [65536,1024] with 16 levels; two input copies
    # (2 x 268 MB) rotate so that no part of a launch's input is left in the 126 MB L2 by the launch before it
    lvs = [torch.randint(0, 16, (65536, 1024), device=dev, generator=g).float() / 8 - 1 for _ in range(2)]
    xi3 = calls.longs(S.shape_info([65536, 1024]))
    zr, zc = torch.zeros(65536, device=dev), torch.zeros(1024, device=dev)
    zir, zic = calls.longs(S.shape_info([65536, 1])), calls.longs(S.shape_info([1, 1024]))

    def f():
        k[0] = (k[0] + 1) % 2
        calls.check(lib.nd4jb200_exec_index_reduce(st, 0, 0, P(lvs[k[0]]), xi3, None, P(zr), zir, d1, 1))
    record("indexreduce_imax_dim1_65536x1024", 268697600, 65536 * 1024, f)

    def f():
        k[0] = (k[0] + 1) % 2
        calls.check(lib.nd4jb200_exec_summary_stats(st, 0, 0, P(lvs[k[0]]), xi3, None, P(zc), zic, d0, 1, 1))
    record("summarystats_variance_dim0_65536x1024", 268439552, 65536 * 1024, f)
    del lvs
    # reduce3 cosine / euclidean on [32768,512] pairs, c-order and stride-2 f-order column views, f32 and f16
    for dt, code, name in ((torch.float32, 0, "f32"), (torch.float16, 2, "f16")):
        es = 4 if code == 0 else 2
        nb = 2 * 32768 * 512 * es + 32768 * es
        xa = [torch.randn(32768, 1024, device=dev, generator=g).to(dt) for _ in range(4)]
        ya = [torch.randn(32768, 1024, device=dev, generator=g).to(dt) for _ in range(4)]
        zz = torch.zeros(32768, device=dev, dtype=dt)
        ci = calls.longs(S.shape_info([32768, 512]))
        vi = calls.longs(S.shape_info([32768, 512], "f", [1, 65536], ews=-1))
        zi4 = calls.longs(S.shape_info([32768, 1]))
        for op, opname in ((2, "cosine"), (1, "euclidean")):
            for info, lay in ((ci, "corder"), (vi, "fview")):
                def f(op=op, info=info):
                    k[0] = (k[0] + 1) % 4
                    calls.check(lib.nd4jb200_exec_reduce3(st, code, op, P(xa[k[0]]), info, None, P(ya[k[0]]), info, P(zz), zi4, d1, 1))
                record("reduce3_%s_%s_%s_32768x512" % (opname, lay, name), nb, 32768 * 512, f)
        del xa, ya
    # reduce3 over all TAD pairs: every row of x [4096,512] against every row of y [4096,512]. The work is
    # 4096 * 4096 * 512 pair operations over 16 MB of input: bound by the FP32 pipes, not by HBM, so the
    # entry reports pair operations per second instead of a bandwidth fraction.
    xa_, ya_ = torch.randn(4096, 512, device=dev, generator=g), torch.randn(4096, 512, device=dev, generator=g)
    za_ = torch.zeros(4096 * 4096, device=dev)
    ai, azi = calls.longs(S.shape_info([4096, 512])), calls.longs(S.shape_info([4096, 4096]))
    for op, opname in ((2, "cosine"), (1, "euclidean")):
        name = "reduce3_all_%s_f32_4096x4096x512" % opname
        record(name, 2 * 4096 * 512 * 4 + 4096 * 4096 * 4, 4096 * 4096,
               lambda op=op: calls.check(lib.nd4jb200_exec_reduce3_all(st, 0, op, P(xa_), ai, None, P(ya_), ai, P(za_), azi, d1, 1)),
               iters=5)
        if name in out:
            out[name]["bound"] = "fp32 pipes (all-pairs work, inputs stay in L2)"
            out[name]["Gpairops_s"] = round(4096 * 4096 * 512 / out[name]["ms"] / 1e6, 1)
            del out[name]["frac_of_measured_peak"]
    del xa_, ya_, za_
    # fused row softmax (special transform 38): one read + one write per element; the reference runs it as
    # max / subtract / exp / sum / divide passes (about 10 array sweeps)
    for rows_, cols_ in ((65536, 1000), (16384, 4096)):
        xs_m = [torch.randn(rows_, cols_, device=dev, generator=g) for _ in range(2)]
        zs_m = torch.empty(rows_, cols_, device=dev)
        mi = calls.longs(S.shape_info([rows_, cols_]))

        def f(mi=mi, xs_m=xs_m, zs_m=zs_m):
            k[0] = (k[0] + 1) % 2
            calls.check(lib.nd4jb200_exec_transform(st, 0, 38, P(xs_m[k[0]]), mi, P(zs_m), mi, None))
        record("softmax_rows_f32_%dx%d" % (rows_, cols_), 2 * rows_ * cols_ * 4, rows_ * cols_, f, iters=10)
        del xs_m, zs_m
    # memory-movement utilities: pullRows of 32768 random rows out of [65536,1024] f32, concat of four
    # [4096,4096] blocks along dimension 0, average of 8 parameter vectors of 2^24 floats
    src_ = torch.randn(65536, 1024, device=dev, generator=g)
    pick_ = torch.randint(0, 65536, (32768,), device=dev, generator=g, dtype=torch.int64)
    out_ = torch.empty(32768, 1024, device=dev)
    tinfo_, toffs_ = ops.tadOnlyShapeInfo(S.shape_info([65536, 1024]), [1], 1)
    zinfo_, zoffs_ = ops.tadOnlyShapeInfo(S.shape_info([32768, 1024]), [1], 1)
    toffs_d, zoffs_d = torch.from_numpy(toffs_).cuda(), torch.from_numpy(zoffs_).cuda()
    ti_, zi_ = calls.longs(tinfo_), calls.longs(zinfo_)
    record("pull_rows_f32_32768_of_65536x1024", 2 * 32768 * 1024 * 4, 32768 * 1024,
           lambda: calls.check(lib.nd4jb200_pull_rows(st, 0, P(src_), P(out_), 32768, P(pick_), ti_, P(toffs_d), zi_, P(zoffs_d))))
    # shuffle: the 32768 row pairs of [65536,1024] change places (every element read and written once); tear: the
    # 65536 rows go to 65536 separate arrays. Both upload an index / pointer list per call, so they are timed as
    # plain back-to-back calls, not as a graph.
    half_ = np.full(65536, -1, np.int32)
    half_[:32768] = 32768 + np.random.default_rng(0).permutation(32768)
    xp_ = (ctypes.c_void_p * 1)(src_.data_ptr())
    xinfo_ = calls.longs(S.shape_info([65536, 1024]))
    xinfos_ = (ctypes.c_void_p * 1)(ctypes.cast(xinfo_, ctypes.c_void_p).value)
    tinfos_ = (ctypes.c_void_p * 1)(ctypes.cast(ti_, ctypes.c_void_p).value)
    offp_ = (ctypes.c_void_p * 1)(toffs_d.data_ptr())
    map_ = calls.ints(half_)
    record("shuffle_f32_65536x1024", 2 * 65536 * 1024 * 4, 65536 * 1024,
           lambda: calls.check(lib.nd4jb200_shuffle(st, 0, 1, xp_, xinfos_, map_, tinfos_, offp_)), graph=False)
    pieces_ = torch.empty(65536, 1024, device=dev)
    tp_ = (ctypes.c_void_p * 65536)(*[pieces_.data_ptr() + 4096 * r_ for r_ in range(65536)])
    pinfo_ = calls.longs(S.shape_info([1, 1024]))
    record("tear_f32_65536x1024", 2 * 65536 * 1024 * 4, 65536 * 1024,
           lambda: calls.check(lib.nd4jb200_tear(st, 0, P(src_), xinfo_, tp_, pinfo_, ti_, P(toffs_d))), graph=False)
    del src_, out_, pieces_
    # sort: every row of [65536,1024] (one pass through shared memory) and a whole array of 2^24 floats (12 stages
    # beyond the shared-memory chunks). Each timed call first refills the array from an unsorted copy (a device
    # copy inside the timed region), because sorted input would skip the network's stores.
    with torch.cuda.stream(stream):
        unsorted_ = torch.randn(65536, 1024, device=dev, generator=g)
        work_ = torch.empty_like(unsorted_)
    winfo_ = calls.longs(S.shape_info([65536, 1024]))
    flat_ = calls.longs(S.shape_info([1, 1 << 24]))

    def f_rows():
        with torch.cuda.stream(stream):
            work_.copy_(unsorted_)
        calls.check(lib.nd4jb200_sort_tad(st, 0, P(work_), winfo_, d1, 1, 0))

    def f_all():
        with torch.cuda.stream(stream):
            work_[:16384].copy_(unsorted_[:16384])
        calls.check(lib.nd4jb200_sort(st, 0, P(work_), flat_, 0))
    def refill_rows():
        with torch.cuda.stream(stream):
            work_.copy_(unsorted_)

    def refill_all():
        with torch.cuda.stream(stream):
            work_[:16384].copy_(unsorted_[:16384])
    record("sort_rows_f32_65536x1024_incl_refill", 4 * 65536 * 1024 * 4, 65536 * 1024, f_rows, iters=10, graph=False)
    record("sort_f32_2p24_incl_refill", 4 * (1 << 24) * 4, 1 << 24, f_all, iters=5, graph=False)
    # the refill alone, so that the sort's own time can be read off: sort = incl_refill - refill
    record("sort_refill_only_65536x1024", 2 * 65536 * 1024 * 4, 65536 * 1024, refill_rows, iters=10, graph=False)
    record("sort_refill_only_2p24", 2 * (1 << 24) * 4, 1 << 24, refill_all, iters=5, graph=False)
    for incl, refill, elems in (("sort_rows_f32_65536x1024_incl_refill", "sort_refill_only_65536x1024", 65536 * 1024),
                                ("sort_f32_2p24_incl_refill", "sort_refill_only_2p24", 1 << 24)):
        if incl in out and refill in out:
            ms_ = out[incl]["ms"] - out[refill]["ms"]
            out[incl]["sort_only_ms"] = round(ms_, 5)
            out[incl]["sort_only_Gelem_s"] = round(elems / ms_ / 1e6, 2)
            out[incl]["sort_only_frac_of_measured_peak"] = round(2 * elems * 4 / ms_ / 1e6 / peak, 3)
    del unsorted_, work_
    # whole-array transforms through execTransform: Im2col / Col2Im (3x3, stride 1, padding 1 on [32,64,56,56]), max
    # Pooling2D 2x2 stride 2 on [64,64,112,112], Reverse and Histogram (256 bins) of 2^26 floats
    img_ = torch.randn(32, 64, 56, 56, device=dev, generator=g)
    col_ = torch.empty(32, 64, 3, 3, 56, 56, device=dev)
    imgi_, coli_ = calls.longs(S.shape_info([32, 64, 56, 56])), calls.longs(S.shape_info([32, 64, 3, 3, 56, 56]))
    e_i2c = torch.tensor([3, 3, 1, 1, 1, 1, 1, 1, 0, 0], dtype=torch.float32, device=dev)
    e_c2i = torch.tensor([1, 1, 1, 1, 56, 56, 1, 1, 0], dtype=torch.float32, device=dev)
    record("im2col_f32_32x64x56x56_k3", (col_.numel() + img_.numel()) * 4, col_.numel(),
           lambda: calls.check(lib.nd4jb200_exec_transform(st, 0, 37, P(img_), imgi_, P(col_), coli_, P(e_i2c))))
    record("col2im_f32_32x64x56x56_k3", (col_.numel() + img_.numel()) * 4, col_.numel(),
           lambda: calls.check(lib.nd4jb200_exec_transform(st, 0, 36, P(col_), coli_, P(img_), imgi_, P(e_c2i))))
    del img_, col_
    # the 7x7 stride-2 kernel of an image network's first layer: [32,3,224,224] -> [32,3,7,7,112,112]
    img_ = torch.randn(32, 3, 224, 224, device=dev, generator=g)
    col_ = torch.empty(32, 3, 7, 7, 112, 112, device=dev)
    imgi_, coli_ = calls.longs(S.shape_info([32, 3, 224, 224])), calls.longs(S.shape_info([32, 3, 7, 7, 112, 112]))
    e_i2c7 = torch.tensor([7, 7, 2, 2, 3, 3, 1, 1, 0, 0], dtype=torch.float32, device=dev)
    record("im2col_f32_32x3x224x224_k7s2", (col_.numel() + img_.numel()) * 4, col_.numel(),
           lambda: calls.check(lib.nd4jb200_exec_transform(st, 0, 37, P(img_), imgi_, P(col_), coli_, P(e_i2c7))))
    del img_, col_
    pin_ = torch.randn(64, 64, 112, 112, device=dev, generator=g)
    pout_ = torch.empty(64, 64, 56, 56, device=dev)
    pini_, pouti_ = calls.longs(S.shape_info([64, 64, 112, 112])), calls.longs(S.shape_info([64, 64, 56, 56]))
    e_pool = torch.tensor([2, 2, 2, 2, 0, 0, 1, 1, 0, 0, 0], dtype=torch.float32, device=dev)
    record("pooling2d_max_f32_64x64x112x112_k2s2", (pin_.numel() + pout_.numel()) * 4, pin_.numel(),
           lambda: calls.check(lib.nd4jb200_exec_transform(st, 0, 71, P(pin_), pini_, P(pout_), pouti_, P(e_pool))))
    del pin_, pout_
    rv_ = torch.randn(1 << 26, device=dev, generator=g)
    rvo_ = torch.empty_like(rv_)
    rvi_ = calls.longs(S.shape_info([1, 1 << 26]))
    record("reverse_f32_2p26", 2 * (1 << 26) * 4, 1 << 26,
           lambda: calls.check(lib.nd4jb200_exec_transform(st, 0, 70, P(rv_), rvi_, P(rvo_), rvi_, None)))
    hz_ = torch.zeros(256, device=dev)
    e_hist = torch.tensor([256, -4, 4], dtype=torch.float32, device=dev)
    record("histogram_f32_2p26_256bins", (1 << 26) * 4, 1 << 26,
           lambda: calls.check(lib.nd4jb200_exec_transform(st, 0, 48, P(rv_), rvi_, P(hz_), calls.longs(S.shape_info([1, 256])), P(e_hist))))
    del rv_, rvo_
    blocks_ = [torch.randn(4096, 4096, device=dev, generator=g) for _ in range(4)]
    cat_ = torch.empty(16384, 4096, device=dev)
    ptrs_ = (ctypes.c_void_p * 4)(*[b_.data_ptr() for b_ in blocks_])
    binfo_ = calls.longs(S.shape_info([4096, 4096]))
    infos_ = (ctypes.c_void_p * 4)(*[ctypes.cast(binfo_, ctypes.c_void_p).value] * 4)
    cinfo_ = calls.longs(S.shape_info([16384, 4096]))
    record("concat_dim0_f32_4x4096x4096", 2 * 16384 * 4096 * 4, 16384 * 4096,
           lambda: calls.check(lib.nd4jb200_concat(st, 0, 0, 4, ptrs_, infos_, P(cat_), cinfo_)))
    del blocks_, cat_
    params_ = [torch.randn(1 << 24, device=dev, generator=g) for _ in range(8)]
    avg_ = torch.empty(1 << 24, device=dev)
    pp_ = (ctypes.c_void_p * 8)(*[p_.data_ptr() for p_ in params_])
    record("average_f32_8x2p24", 9 * (1 << 24) * 4, 1 << 24,
           lambda: calls.check(lib.nd4jb200_average(st, 0, pp_, P(avg_), 8, 1 << 24, 0)))
    del params_, avg_
    # The member nd4j's JNI glue binds (NativeOps::execReduceFloat, called through its mangled symbol with the
    # reference's CUDA-build conventions: device shapeInfo / dimension, host copies in extraPointers[0], [8], [9])
    # beside the C entry point it forwards to, on an array small enough that the call's host cost is what is timed.
    if not only or "member_path" in only:
        xm = torch.randn(256, 128, device=dev, generator=g)
        zm = torch.zeros(256, device=dev)
        h_xi, h_zi = S.shape_info([256, 128]), S.shape_info([256, 1])
        h_tad, _ = ops.tadOnlyShapeInfo(h_xi, [1], 1)
        h_tad = np.ascontiguousarray(h_tad, dtype=np.int64)
        d_xi, d_zi = torch.from_numpy(h_xi).cuda(), torch.from_numpy(h_zi).cuda()
        d_dim = torch.tensor([1], dtype=torch.int32, device=dev)
        c_xi, c_zi, c_d1 = calls.longs(h_xi), calls.longs(h_zi), calls.ints([1])
        extras = (ctypes.c_void_p * 16)()
        extras[0], extras[1], extras[8], extras[9] = h_xi.ctypes.data, stream.cuda_stream, h_zi.ctypes.data, h_tad.ctypes.data
        member = getattr(lib, "_ZN9NativeOps15execReduceFloatEPPviPfPxS2_S2_S3_Pii")
        member.restype = None
        member.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6 + [ctypes.c_int]
        this = ctypes.create_string_buffer(8)
        lib.nd4jb200_metadata_reads.restype = ctypes.c_ulonglong

        def via_member():
            member(this, extras, 1, P(xm), P(d_xi), None, P(zm), P(d_zi), P(d_dim), 1)

        def via_c():
            calls.check(lib.nd4jb200_exec_reduce(st, 0, 1, P(xm), c_xi, None, P(zm), c_zi, c_d1, 1))

        def host_us(fn, n=3000):
            for _ in range(200):
                fn()
            stream.synchronize()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            stream.synchronize()
            return (time.perf_counter() - t0) / n * 1e6
        reads0 = lib.nd4jb200_metadata_reads()
        us_c, us_m = host_us(via_c), host_us(via_member)
        out["member_path_execReduceFloat_256x128"] = {
            "c_abi_us_per_call": round(us_c, 2), "member_us_per_call": round(us_m, 2),
            "device_metadata_reads": int(lib.nd4jb200_metadata_reads() - reads0),
            "note": "wall time per asynchronous call incl. the Python/ctypes overhead both paths share"}
        del xm, zm
    # scalar family: x * 1.5 on the chain-sized array
    xs_ = torch.randn(ELEMS, device=dev, generator=g)
    zs_ = torch.empty_like(xs_)
    si = calls.longs(S.shape_info([ROWS, COLS]))
    record("scalar_mul_16384x4096", 2 * ELEMS * 4, ELEMS,
           lambda: calls.check(lib.nd4jb200_exec_scalar(st, 0, 2, P(xs_), si, P(zs_), si, ctypes.c_double(1.5), None)))
    del xs_, zs_
    # random family: 2^30 outputs (2^26 when quick), table of 100000 words, seed 119
    n = 1 << (26 if quick else 30)
    state = ops.initRandom([None, stream.cuda_stream], 119, 100000, None)
    zbuf = torch.empty(n, device=dev)
    zin = calls.longs(S.shape_info([1, n]))
    e01 = torch.tensor([0.0, 1.0], device=dev)
    e03 = torch.tensor([0.3], device=dev)
    e05 = torch.tensor([0.5], device=dev)
    xr = torch.ones(n, device=dev)
    sp = ctypes.c_void_p(state)
    record("random_uniform_2p%d" % (26 if quick else 30), 4 * n, n,
           lambda: calls.check(lib.nd4jb200_exec_random(st, 0, 0, sp, P(zbuf), zin, P(e01))), iters=3)
    record("random_gaussian_2p%d" % (26 if quick else 30), 4 * n, n,
           lambda: calls.check(lib.nd4jb200_exec_random_xy(st, 0, 6, sp, P(zbuf), zin, P(zbuf), zin, P(zbuf), zin, P(e01))), iters=3)
    record("random_bernoulli_2p%d" % (26 if quick else 30), 4 * n, n,
           lambda: calls.check(lib.nd4jb200_exec_random(st, 0, 7, sp, P(zbuf), zin, P(e03))), iters=3)
    record("random_dropout_inverted_2p%d" % (26 if quick else 30), 8 * n, n,
           lambda: calls.check(lib.nd4jb200_exec_random_x(st, 0, 2, sp, P(xr), zin, P(zbuf), zin, P(e05))), iters=3)
    del xr
    # The random family is bound by instruction issue on the integer pipes, not by HBM (the reference's hash is
    # 64-bit integer work): its yardstick is the issue rate, 148 SMs x 4 schedulers x 32 lanes x the SM clock.
    # Thread instructions per draw are the ncu counts of profiles/random_uniform_gaussian_2p26.md (the other two
    # ops run the Uniform kernel's hash plus a compare / a multiply).
    issue_peak = 148 * 4 * 32 * 1.965e9
    for name_, per_draw in (("random_uniform", 139), ("random_gaussian", 189), ("random_bernoulli", 139), ("random_dropout_inverted", 142)):
        key_ = "%s_2p%d" % (name_, 26 if quick else 30)
        if key_ in out:
            rate = out[key_]["Gelem_s"] * 1e9 * per_draw
            out[key_].update({"bound": "int-alu", "thread_instr_per_draw": per_draw,
                              "achieved_Tinstr_s": round(rate / 1e12, 2), "peak_Tinstr_s": round(issue_peak / 1e12, 2),
                              "frac_of_issue_peak": round(rate / issue_peak, 3)})
    # whole-array Sum of 2^31 (2^27 when quick) floats drawn U(-1,1) on the device: element e is draw e of a fresh
    # seed-119 state, which is also what the ranks of a multi-GPU run generate for their shards
    n2 = 1 << (27 if quick else 31)
    big = torch.empty(n2, device=dev)
    chunk = 1 << 26
    em1 = torch.tensor([-1.0, 1.0], device=dev)
    fresh = ops.initRandom([None, stream.cuda_stream], 119, 100000, None)
    for off in range(0, n2, chunk):
        calls.check(lib.nd4jb200_exec_random_range(st, 0, 0, 0, ctypes.c_void_p(fresh), None, None, P(big[off:off + chunk]),
                                                   P(em1), off, chunk, n2))
    ops.destroyRandom(fresh)
    bi2 = calls.longs(S.shape_info([1, n2]))
    res = ctypes.c_double()
    record("reduce_scalar_sum_2p%d" % (27 if quick else 31), 4 * n2, n2,
           lambda: calls.check(lib.nd4jb200_exec_reduce_scalar(st, 0, 1, P(big), bi2, None, ctypes.byref(res))), iters=5,
           graph=False)   # the scalar form synchronises the stream: timed as a plain loop
    # the same sum through the sharded entry point (a communicator of one rank, grid of 8 shards, result left on
    # the device): the value a 2-, 4- or 8-GPU run of this benchmark must reproduce bit for bit
    if not only or "sharded" in only:
        ops.commInit(None, 0, 1)
        zdev = torch.zeros(1, device=dev)
        record("reduce_scalar_sum_sharded_allgather", 4 * n2, n2,
               lambda: calls.check(lib.nd4jb200_exec_reduce_scalar_sharded(st, 0, 1, P(big), n2, None, 8, n2, P(zdev), None)),
               iters=10, graph=False)
        stream.synchronize()
        if "reduce_scalar_sum_sharded_allgather" in out:
            out["reduce_scalar_sum_sharded_allgather"].update({"shard_grid": 8, "sum": float(zdev.item())})
        ops.commDestroy()
    ops.destroyRandom(state)
    return out


def run_ours(args):
    import torch
    from libnd4j_b200 import shape as S
    from libnd4j_b200.native_ops import NativeOps

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ops = NativeOps()
    stream = torch.cuda.Stream()
    calls = Calls(ops, stream.cuda_stream)
    lib, st, P = calls.lib, calls.stream, calls.p
    for kv in args.tune:
        key, value = kv.split("=")
        calls.check(lib.nd4jb200_set_tuning(int(key), ctypes.c_longlong(int(value))))
    peak, peak_src = measured_peaks()

    if world > 1 and hasattr(os, "sched_setaffinity"):
        # every rank keeps to its own slice of the host cores, so that its copy threads and the pages of its
        # pinned buffers (first touched below) stay together
        cores = sorted(os.sched_getaffinity(0))
        share = max(1, len(cores) // world)
        mine = cores[local * share:(local + 1) * share] or cores
        try:
            os.sched_setaffinity(0, mine)
        except OSError:
            pass
    x, b, y = make_inputs(ROWS)
    hx, hb, hy = (torch.from_numpy(a).pin_memory() for a in (x, b, y))
    hz = torch.empty(ELEMS, dtype=torch.float32).pin_memory()
    with torch.cuda.stream(stream):
        dx, db, dy = hx.cuda(non_blocking=True), hb.cuda(non_blocking=True), hy.cuda(non_blocking=True)
        t1, t2, dz = (torch.empty(ROWS, COLS, device="cuda") for _ in range(3))
    stream.synchronize()
    xi, bi, d1 = calls.longs(S.shape_info([ROWS, COLS])), calls.longs(S.shape_info([1, COLS])), calls.ints([1])

    def k_broadcast():
        calls.check(lib.nd4jb200_exec_broadcast(st, 0, 0, P(dx), xi, P(db), bi, P(t1), xi, d1, 1))

    def k_tanh():
        calls.check(lib.nd4jb200_exec_transform(st, 0, 15, P(t1), xi, P(t2), xi, None))

    def k_mul():
        calls.check(lib.nd4jb200_exec_pairwise(st, 0, 6, P(t2), xi, P(dy), xi, P(dz), xi, None))

    def step():
        k_broadcast()
        k_tanh()
        k_mul()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler.mark_begin()
    launches0 = ops.launchCount()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(args.steps):
        step()
    stop.record(stream)
    barrier()
    sampler.mark_end()
    launches = ops.launchCount() - launches0
    ms_step = start.elapsed_time(stop) / args.steps
    if dist is not None:
        t = torch.tensor([ms_step], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item())
    value = world * ELEMS / ms_step / 1e6   # Gelem/s over all ranks

    # Per-kernel durations, each kernel timed alone on the launch stream. Consecutive launches alternate between
    # two complete sets of buffers, so that nothing a launch touches is left in the 126 MB L2 by the launch before
    # it (a kernel replayed on one set finds the tail of its own previous output there and reads above the DRAM
    # peak).
    with torch.cuda.stream(stream):
        dx2, dy2 = dx.clone(), dy.clone()
        t1b, t2b, dzb = (torch.empty(ROWS, COLS, device="cuda") for _ in range(3))
        t1b.copy_(t1); t2b.copy_(t2)
    sets = ((dx, t1, t2, dy, dz), (dx2, t1b, t2b, dy2, dzb))
    flip = [0]

    def alt(kind):
        def fn():
            flip[0] ^= 1
            ax, a1, a2, ay, az = sets[flip[0]]
            if kind == 0:
                calls.check(lib.nd4jb200_exec_broadcast(st, 0, 0, P(ax), xi, P(db), bi, P(a1), xi, d1, 1))
            elif kind == 1:
                calls.check(lib.nd4jb200_exec_transform(st, 0, 15, P(a1), xi, P(a2), xi, None))
            elif kind == 2:
                calls.check(lib.nd4jb200_exec_pairwise(st, 0, 6, P(a2), xi, P(ay), xi, P(az), xi, None))
            else:
                calls.check(lib.nd4jb200_exec_chain(st, 0, 0, P(ax), xi, P(db), bi, d1, 1, 15, None, 6, P(ay), xi, None, P(az), xi))
        return fn
    per = {}
    for kind, name in enumerate(("broadcast_add", "transform_tanh", "pairwise_mul")):
        fn = alt(kind)
        for _ in range(4):
            fn()
        per[name] = time_graph(torch, stream, fn, 20)
    # the same chain as ONE fused pass (nd4jb200_exec_chain): x and y read once, z written once
    fused_bytes = 3 * ELEMS * 4 + COLS * 4

    k_fused = alt(3)
    for _ in range(4):
        k_fused()
    fused_ms = time_graph(torch, stream, k_fused, 20)
    del dx2, dy2, t1b, t2b, dzb, sets
    fused = {"ms_per_step": round(fused_ms, 5), "Gelem_s": round(ELEMS / fused_ms / 1e6, 2),
             "GBps": round(fused_bytes / fused_ms / 1e6, 1), "frac_of_measured_peak": round(fused_bytes / fused_ms / 1e6 / peak, 4),
             "algorithmic_bytes": fused_bytes,
             "note": "one launch instead of three; bit-identical result; the headline value keeps the three exec* calls the metric names"}
    clocks = sampler.stop()
    dom = max(per, key=lambda n: per[n])
    achieved = BYTES[dom] / per[dom] / 1e6
    roofline = {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "traffic": None, "peak_source": peak_src,
                "per_kernel_ms": {k: round(v, 5) for k, v in per.items()},
                "per_kernel_GBps": {k: round(BYTES[k] / v / 1e6, 1) for k, v in per.items()},
                "frac_of_nominal_8TBps": round(achieved / 8000.0, 4),
                "note": "consecutive timed launches alternate between two buffer sets (no L2 residue); the peak is a "
                        "one-read-one-write copy, which a two-reads-one-write kernel can exceed slightly"}
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(traffic_file):
        with open(traffic_file) as f:
            roofline["traffic"] = json.load(f).get(dom)

    # End to end through host buffers: H2D of x, b, y, the chain, D2H of the result, every step. The arrays are
    # cut into row blocks; block k's chain runs while block k+1 is copied in and block k-1 is copied out (three
    # streams, the same exec* calls on [rows/blocks, COLS] shapeInfos), so a step costs about max(H2D, D2H) on a
    # full-duplex link instead of their sum. Consecutive steps are chained by their data dependencies only, block
    # by block (a block's inputs may be overwritten once the previous step's chain has read them, its result once
    # the previous result has left the device; the vector b alternates between two device copies), so the copy-in
    # of step n+1 starts while step n is still draining, as in any loop over batches.
    NBLK = args.e2e_blocks
    brow = ROWS // NBLK
    bbytes = brow * COLS * 4
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    h_in, h_cmp, h_out = (ctypes.c_void_p(q.cuda_stream) for q in (s_in, stream, s_out))
    ev_in = [torch.cuda.Event() for _ in range(NBLK)]
    ev_cmp = [torch.cuda.Event() for _ in range(NBLK)]
    ev_out = [torch.cuda.Event() for _ in range(NBLK)]
    ev_step = [torch.cuda.Event(), torch.cuda.Event()]
    ev_end = torch.cuda.Event()
    with torch.cuda.stream(stream):
        dbs = (db, db.clone())
    xib = calls.longs(S.shape_info([brow, COLS]))
    cp = lib.nd4jb200_memcpy_async
    V = ctypes.c_void_p
    step_no = [0]

    def e2e_step():
        n = step_no[0]
        step_no[0] += 1
        dbn = dbs[n % 2]
        if n >= 2:
            s_in.wait_event(ev_step[n % 2])          # the chain of step n-2 has finished with this copy of b
        calls.check(cp(V(dbn.data_ptr()), V(hb.data_ptr()), COLS * 4, 1, h_in))
        for k in range(NBLK):
            off = k * bbytes
            if n >= 1:
                s_in.wait_event(ev_cmp[k])           # the previous step's chain has read block k of x and y
            calls.check(cp(V(dx.data_ptr() + off), V(hx.data_ptr() + off), bbytes, 1, h_in))
            calls.check(cp(V(dy.data_ptr() + off), V(hy.data_ptr() + off), bbytes, 1, h_in))
            ev_in[k].record(s_in)
            stream.wait_event(ev_in[k])
            if n >= 1:
                stream.wait_event(ev_out[k])         # the previous result of block k has left the device
            calls.check(lib.nd4jb200_exec_broadcast(h_cmp, 0, 0, V(dx.data_ptr() + off), xib, P(dbn), bi,
                                                    V(t1.data_ptr() + off), xib, d1, 1))
            calls.check(lib.nd4jb200_exec_transform(h_cmp, 0, 15, V(t1.data_ptr() + off), xib, V(t2.data_ptr() + off), xib, None))
            calls.check(lib.nd4jb200_exec_pairwise(h_cmp, 0, 6, V(t2.data_ptr() + off), xib, V(dy.data_ptr() + off), xib,
                                                   V(dz.data_ptr() + off), xib, None))
            ev_cmp[k].record(stream)
            s_out.wait_event(ev_cmp[k])
            calls.check(cp(V(hz.data_ptr() + off), V(dz.data_ptr() + off), bbytes, 2, h_out))
            ev_out[k].record(s_out)
        ev_step[n % 2].record(stream)

    def e2e_drain():
        ev_end.record(s_out)
        stream.wait_event(ev_end)                    # the last block of the last step is back on the host

    e2e_step()
    e2e_drain()
    barrier()
    e2e_iters = max(4, min(args.steps, 10))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(e2e_iters):
        e2e_step()
    e2e_drain()
    stop.record(stream)
    stop.synchronize()
    e2e_ms = start.elapsed_time(stop) / e2e_iters
    # the chain's result of the last step, as it arrived in host memory, against the device's copy
    torch.cuda.synchronize()
    if not torch.equal(hz.view(ROWS, COLS)[-brow:], dz[-brow:].cpu()):
        raise SystemExit("end-to-end step: the result read back differs from the device's")
    if dist is not None:
        t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": round(world * ELEMS / e2e_ms / 1e6, 3), "unit": "Gelem/s", "ms_per_step": round(e2e_ms, 3),
           "h2d_bytes_per_step": 2 * ELEMS * 4 + COLS * 4, "d2h_bytes_per_step": ELEMS * 4,
           "pipeline": "%d row blocks; H2D, chain and D2H on three streams; consecutive steps chained block by block" % NBLK,
           "per_rank_h2d_GBps": round((2 * ELEMS * 4 + COLS * 4) / e2e_ms / 1e6, 1),
           "per_rank_d2h_GBps": round(ELEMS * 4 / e2e_ms / 1e6, 1)}

    families = None
    if world == 1 and not args.no_families:
        with torch.cuda.stream(stream):
            del dx, dy, t1, t2, dz
            torch.cuda.empty_cache()
            families = family_table(torch, ops, calls, stream, peak, args.quick, args.only, args.profile)
    elif world > 1:
        families = sharded_families(torch, dist, ops, calls, stream, world, rank, args.quick)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import reference
        if reference.available():
            rows = ROWS
            gel, cores, secs = cpu_reference_chain(rows, repeats=3, threads=host_threads())
            cpu = {"value": round(gel, 4), "unit": "Gelem/s", "cores": cores, "kind": "reference",
                   "sample": "all %d rows, best of 3 after one warm-up pass, %.1f ms" % (rows, secs * 1e3)}
        else:
            rows = 512      # the scalar port: a smaller sample keeps this leg at a few seconds
            gel, cores, secs = cpu_reference_chain(rows, repeats=1, threads=host_threads(), use_port=True)
            cpu = {"value": round(gel, 4), "unit": "Gelem/s", "cores": cores, "kind": "port",
                   "sample": "%d of %d rows (same row width), oracle port, best of 1 after one warm-up pass, %.1f ms" % (rows, ROWS, secs * 1e3)}

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": round(value, 3), "unit": "Gelem/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "elementwise chain f32 [16384,4096]: execBroadcast Add(dim 1) -> execTransform Tanh -> "
                                   "execPairwiseTransform Multiply", "l2": "inputs larger than L2 (3 x 268 MB streamed per step); per-kernel timings alternate two buffer sets",
                       "sharding": "one independent chain per GPU"},
            "roofline": roofline, "fused_chain": fused, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks,
            "families": families,
        }))
    if dist is not None:
        dist.destroy_process_group()


def sharded_families(torch, dist, ops, calls, stream, world, rank, quick):
    """N > 1: every family of the configurations, sharded the way it shards naturally. Random generation is
    offset-sharded with global indices; reductions along a dimension are row- or column-sharded (disjoint result
    slices); neither needs an exchange. The whole-array Sum reduces each shard locally and combines accumulator
    states through the library's own communicator (one ncclAllGather on the launch stream, then the same
    fixed-order fold on every rank): the only collective on this path. Times are CUDA-event times on the launch
    stream, max over ranks; Gelem/s counts the elements of all ranks."""
    from libnd4j_b200 import shape as S
    lib, st, P = calls.lib, calls.stream, calls.p
    dev = torch.device("cuda")
    out = {}
    uid = [ops.commUniqueId() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    # NCCL announces its version on stdout when a process creates its first communicator of its own; stdout
    # carries the one JSON line, so the announcement is sent to stderr
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        ops.commInit(uid[0], rank, world)
    finally:
        os.dup2(saved, 1)
        os.close(saved)

    def over_ranks(ms):
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, iters, graph=False, batches=1):
        """Max over ranks of the device time per call; with several batches, the median batch (a collective's
        occasional slow call - one in a few hundred on these boxes - then does not decide the number)."""
        for _ in range(3):
            fn()
        got = []
        for _ in range(batches):
            dist.barrier()
            torch.cuda.synchronize()
            ms = time_graph(torch, stream, fn, iters) if graph else time_loop(torch, stream, fn, iters)
            got.append(over_ranks(ms))
        return sorted(got)[len(got) // 2]

    # ---- C5a: 2^30 draws, rank g produces global indices [g * n / G, (g + 1) * n / G) ----
    n = 1 << (26 if quick else 30)
    per = n // world
    state = ops.initRandom([None, stream.cuda_stream], 119, 100000, None)
    sp = ctypes.c_void_p(state)
    z = torch.empty(per, device=dev)
    ones = torch.ones(per, device=dev)
    for name, op, arity, extra, bytes_per in (("uniform", 0, 0, [0.0, 1.0], 4), ("gaussian", 6, 2, [0.0, 1.0], 4),
                                              ("bernoulli", 7, 0, [0.3], 4), ("dropout_inverted", 2, 1, [0.5], 8)):
        ex = torch.tensor(extra, device=dev)
        xa = ones if arity == 1 else (z if arity == 2 else None)
        ya = z if arity == 2 else None
        ms = timed(lambda: calls.check(lib.nd4jb200_exec_random_range(st, 0, op, arity, sp, P(xa), P(ya), P(z), P(ex),
                                                                      rank * per, per, n)), 3)
        out["random_%s_sharded" % name] = {"ms": round(ms, 4), "Gelem_s": round(n / ms / 1e6, 2),
                                           "GBps": round(bytes_per * n / ms / 1e6, 1), "elements": n}
    del ones
    # ---- C5b: whole-array Sum of 2^31 floats over a fixed grid of 8 shards ----
    n2 = 1 << (27 if quick else 31)
    per2 = n2 // world
    big = torch.empty(per2, device=dev)
    chunk = min(per2, 1 << 26)
    em1 = torch.tensor([-1.0, 1.0], device=dev)
    for off in range(0, per2, chunk):
        calls.check(lib.nd4jb200_exec_random_range(st, 0, 0, 0, sp, None, None, P(big[off:off + chunk]), P(em1),
                                                   rank * per2 + off, chunk, n2))
    grid_shards = max(8, world)
    zdev = torch.zeros(1, device=dev)
    ms = timed(lambda: calls.check(lib.nd4jb200_exec_reduce_scalar_sharded(st, 0, 1, P(big), per2, None, grid_shards // world,
                                                                           n2, P(zdev), None)), 10, batches=5)
    stream.synchronize()
    out["reduce_scalar_sum_sharded_allgather"] = {"ms": round(ms, 4), "Gelem_s": round(n2 / ms / 1e6, 2),
                                                  "GBps": round(4 * n2 / ms / 1e6, 1), "elements": n2,
                                                  "shard_grid": grid_shards, "sum": float(zdev.item()),
                                                  "timing": "median of 5 batches of 10 calls, max over ranks",
                                                  "note": "same shard grid at every N: the sum's bits must not change with N"}
    ops.destroyRandom(state)
    del big
    # ---- C1 / C3 / C4: the along-dimension reductions with their TADs split over the ranks ----
    g = torch.Generator(device=dev)
    g.manual_seed(100 + rank)
    d1, d0 = calls.ints([1]), calls.ints([0])
    k = [0]

    def rotating(make, count):
        return [make() for _ in range(count)]
    r1 = 8192 // world
    xs = rotating(lambda: torch.empty(r1, 4096, device=dev).uniform_(-1, 1, generator=g), 3)
    zz = torch.zeros(r1, device=dev)
    xi, zi = calls.longs(S.shape_info([r1, 4096])), calls.longs(S.shape_info([r1, 1]))

    def f():
        k[0] = (k[0] + 1) % 3
        calls.check(lib.nd4jb200_exec_reduce(st, 0, 1, P(xs[k[0]]), xi, None, P(zz), zi, d1, 1))
    ms = timed(f, 20, graph=True)
    out["reduce_sum_dim1_8192x4096_row_sharded"] = {"ms": round(ms, 5), "Gelem_s": round(8192 * 4096 / ms / 1e6, 1),
                                                    "GBps": round(134250496 / ms / 1e6, 1)}
    del xs
    r3 = 65536 // world
    lv = rotating(lambda: torch.randint(0, 16, (r3, 1024), device=dev, generator=g).float() / 8 - 1, 2)
    zr = torch.zeros(r3, device=dev)
    xi3, zi3 = calls.longs(S.shape_info([r3, 1024])), calls.longs(S.shape_info([r3, 1]))

    def f():
        k[0] = (k[0] + 1) % 2
        calls.check(lib.nd4jb200_exec_index_reduce(st, 0, 0, P(lv[k[0]]), xi3, None, P(zr), zi3, d1, 1))
    ms = timed(f, 20, graph=True)
    out["indexreduce_imax_dim1_65536x1024_row_sharded"] = {"ms": round(ms, 5), "Gelem_s": round(65536 * 1024 / ms / 1e6, 1),
                                                           "GBps": round(268697600 / ms / 1e6, 1)}
    del lv
    # variance along dimension 0: every rank owns 1024 / G columns of all 65536 rows (a strided view of the array)
    c3 = 1024 // world
    full = rotating(lambda: torch.randint(0, 16, (65536, 1024), device=dev, generator=g).float() / 8 - 1, 2)
    zc = torch.zeros(c3, device=dev)
    vi3 = calls.longs(S.shape_info([65536, c3], "c", [1024, 1]))
    zic = calls.longs(S.shape_info([1, c3]))

    def f():
        k[0] = (k[0] + 1) % 2
        calls.check(lib.nd4jb200_exec_summary_stats(st, 0, 0, ctypes.c_void_p(full[k[0]].data_ptr() + 4 * rank * c3), vi3, None,
                                                    P(zc), zic, d0, 1, 1))
    ms = timed(f, 20, graph=True)
    out["summarystats_variance_dim0_65536x1024_column_sharded"] = {"ms": round(ms, 5), "Gelem_s": round(65536 * 1024 / ms / 1e6, 1),
                                                                   "GBps": round(268439552 / ms / 1e6, 1)}
    del full
    r4 = 32768 // world
    for dt, code, name in ((torch.float32, 0, "f32"), (torch.float16, 2, "f16")):
        es = 4 if code == 0 else 2
        xa = rotating(lambda: torch.randn(r4, 512, device=dev, generator=g).to(dt), 4)
        ya = rotating(lambda: torch.randn(r4, 512, device=dev, generator=g).to(dt), 4)
        z4 = torch.zeros(r4, device=dev, dtype=dt)
        ci, zi4 = calls.longs(S.shape_info([r4, 512])), calls.longs(S.shape_info([r4, 1]))
        for op, opname in ((2, "cosine"), (1, "euclidean")):
            def f(op=op):
                k[0] = (k[0] + 1) % 4
                calls.check(lib.nd4jb200_exec_reduce3(st, code, op, P(xa[k[0]]), ci, None, P(ya[k[0]]), ci, P(z4), zi4, d1, 1))
            ms = timed(f, 20, graph=True)
            out["reduce3_%s_%s_32768x512_row_sharded" % (opname, name)] = {
                "ms": round(ms, 5), "Gelem_s": round(32768 * 512 / ms / 1e6, 1),
                "GBps": round((2 * 32768 * 512 * es + 32768 * es) / ms / 1e6, 1)}
        del xa, ya
    ops.commDestroy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--quick", action="store_true", help="smaller sizes for the families table")
    ap.add_argument("--no-families", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--e2e-blocks", type=int, default=4, help="row blocks of the pipelined end-to-end step (divides 16384)")
    ap.add_argument("--only", default=None, help="run only the families whose name contains one of these comma-separated texts")
    ap.add_argument("--profile", action="store_true", help="profiling aid: three plain timed launches per family, no graph")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="override a launch heuristic through nd4jb200_set_tuning (repeatable)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
