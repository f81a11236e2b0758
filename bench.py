#!/usr/bin/env python
"""Benchmark of the linear-recurrence scan hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--regions R] [--impl reference]

Prints ONE JSON line.  A "step" is one forward plus one backward pass of the scan over one batch
of synthetic input.  Workload of the headline: the autograd configuration of the task definition --
x ~ N(0,1), c ~ U(0.9, 1), dy ~ N(0,1), fp32, shape (16, 2048, 8192), scanning the last dimension --
per GPU; with N GPUs every rank holds its own batch of that shape (channel sharding of a
(16*N, 2048, 8192) batch, no collective on the data path), i.e. weak scaling.

metric   linrec fwd+bwd achieved HBM GB/s: algorithmic bytes (12 B/element forward + 20 B/element
         backward for fp32, the byte model of the reference's eval/utils.py:48-60) of all ranks
         divided by the slowest rank's device time for the K steps.
value    inputs AND results resident in HBM (allocated once, before the warm-up; the timed region
         makes no allocation, which the line proves with the allocator's counters), operators called
         through the C ABI.  R regions of exactly K steps are timed back to back, each bracketed by a
         barrier and a device synchronisation; `value` and `ms_per_step` are the MEDIAN region, all R
         are listed.
e2e      the same step through the public host API starting from pinned HOST buffers: host->device
         copies of x, c, dy and device->host copies of y, dx, dc are inside the timed region; beside
         it the same copies with no kernel at all (the ceiling the link sets).
roofline the backward operator (the larger of the two kernels of a step): algorithmic bytes per
         launch / mean CUDA-event duration of the launches inside the median region, against the
         measured copy bandwidth of MEASURED_PEAKS.json (fallback 6650 GB/s).
regimes  (one GPU) every other configuration of the task definition, device resident, event timed:
         (512, 4096) forward, (512, 65536) forward in both directions, and 2^28 elements at
         L = 2^8 ... 2^20 in fp32 and bf16 storage, forward and backward.
cfg5     the multi-GPU configuration, fp32 (8192, 2^20), c ~ U(0.99, 1), forward + backward, split by
         rows (`channel`) and by columns (`seq`: local scan, one exchange of per-row records, fix-up),
         each with sampled rows compared against the unsharded single-device operator.
cpu_baseline  the reference's CPU path (a torch restatement of its Python loop, oracle.pyloop_*)
         timed on this machine's host cores on a bounded sample of the same workload.

--impl reference times that CPU path alone, with all host threads, and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "linrec fwd+bwd achieved HBM GB/s"
SHAPE = (16, 2048, 8192)          # per GPU
C_RANGE = (0.9, 1.0)
BYTES_PER_ELEM_FWD, BYTES_PER_ELEM_BWD = 12, 20
SEED = 12334567890
FALLBACK_PEAK_GBS = 6650.0
RTOL, ATOL = 1e-4, 1e-5           # fp32 tolerance of the task definition

# DRAM traffic of the backward kernel measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum
# per launch, divided by the elements of the captured launch); the capture and its command are in
# profiles/.
NCU_DRAM_BYTES_PER_ELEM_BWD = 5.32e9 / 268435456   # full-size capture, profiles/linrec_tma_kernel_bwd_f32_4096x8192.md


def _peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed regions run on the device.

    NVML is initialised and a first query is made BEFORE the timed regions: attaching a monitoring
    client to the GPU (which is what starting `nvidia-smi` does) stalls kernel launches for tens of
    milliseconds, which must not land inside the measurement.  The samples themselves are taken by the
    benchmarking thread after it has queued the last launch of a region (see sample_while_busy), every
    few milliseconds until the device has finished that region."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period_s: float = float(os.environ.get("LINREC_BENCH_CLOCK_PERIOD", "0.01"))):
        self.index, self.period, self.rows = index, period_s, []
        self.nvml = None
        self.handle = None

    def _sample(self):
        n = self.nvml
        sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        return sm, mx, int(get(self.handle))

    def prepare(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip().isdigit()]
            phys = int(ids[self.index]) if self.index < len(ids) else self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self._sample()
        except Exception:
            self.nvml = None

    def sample_while_busy(self, finished):
        """Samples from the CALLING thread until `finished()` is true; at least once.  Called right
        after the last launch of a timed region has been queued: the host runs far ahead of the
        device, so the GPU is under that load for the whole time and no launch can be held up by a
        query."""
        if self.nvml is None:
            return
        while True:
            try:
                self.rows.append(self._sample())
            except Exception:
                pass
            if finished():
                return
            time.sleep(self.period)
            if finished():
                return

    def summary(self):
        if self.nvml is None or not self.rows:
            return None
        sm = [r[0] for r in self.rows]
        mask = 0
        for r in self.rows:
            mask |= r[2]
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": max(r[1] for r in self.rows),
                "reasons": sorted(v for k, v in self.REASONS.items() if mask & k), "samples": len(sm)}


# ======================================================================================================
#  CPU path of the reference (the `cpu_baseline` leg and `--impl reference`)
# ======================================================================================================
def _host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def _cpu_reference_run(steps: int, warmup: int, rows: int, with_c_port: bool = True):
    """The reference's CPU path on `rows` rows of the workload; returns (seconds per step, info)."""
    import torch

    import oracle
    # launchers (torchrun) pin OMP_NUM_THREADS to 1: this leg is meant to use the host's cores
    torch.set_num_threads(_host_threads())
    L = SHAPE[-1]
    g = torch.Generator(device="cpu").manual_seed(SEED)
    x = torch.randn((rows, L), generator=g)
    c = C_RANGE[0] + (C_RANGE[1] - C_RANGE[0]) * torch.rand((rows, L), generator=g)
    dy = torch.randn((rows, L), generator=g)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        y = oracle.pyloop_fwd(x, c)
        dx, dc = oracle.pyloop_bwd(dy, c, y)
        t1 = time.perf_counter()
        if i >= warmup:
            times.append(t1 - t0)
    sec = statistics.median(times)
    info = {"rows": rows, "seqlen": L, "torch_threads": torch.get_num_threads(), "os_cpu_count": os.cpu_count()}
    if with_c_port:
        # the C restatement with OpenMP over the rows, for context (a far tighter CPU loop than the
        # reference has)
        oracle.set_threads(_host_threads())
        xn, cn, dyn = x.numpy(), c.numpy(), dy.numpy()
        t0 = time.perf_counter()
        yn = oracle.fwd_f32(xn, cn)
        oracle.bwd_f32(dyn, cn, yn)
        c_sec = time.perf_counter() - t0
        info.update({"c_port_openmp_gbs": rows * L * 32 / c_sec / 1e9, "c_port_threads": oracle.threads()})
    return sec, info


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1024
    sec, info = _cpu_reference_run(args.steps, max(args.warmup, 1), rows)
    gbs = rows * SHAPE[-1] * (BYTES_PER_ELEM_FWD + BYTES_PER_ELEM_BWD) / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "autograd fwd+bwd, x~N(0,1), c~U(0.9,1), fp32, (16,2048,8192) per GPU",
                   "timing": "host wall clock, CPU path, median step"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": info["torch_threads"], "kind": "port",
                         "sample": f"{rows} of 32768 rows x {SHAPE[-1]} (fwd+bwd) per step, torch restatement of the "
                                   "reference's Python loop; its throughput does not grow with the number of rows "
                                   "(see cpu_baseline.more_rows of the other arm)", **info},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ======================================================================================================
#  helpers of the GPU arm
# ======================================================================================================
class Ctx:
    """What every leg of the GPU arm needs: device, ranks, barrier, max over ranks."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU implementation of the product path)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def all_true(self, flag: bool) -> bool:
        if self.world == 1:
            return bool(flag)
        t = self.torch.tensor([1 if flag else 0], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(int(t.item()))

    def event(self):
        return self.torch.cuda.Event(enable_timing=True)

    def alloc_counters(self):
        st = self.torch.cuda.memory_stats(self.dev)
        return {"device_allocs": int(st.get("num_device_alloc", st.get("segment.all.allocated", 0))),
                "alloc_retries": int(st.get("num_alloc_retries", 0))}

    def timed(self, fn, n, warm=3):
        """Mean device milliseconds of `fn` over n back-to-back calls on this rank (single-GPU side measurements)."""
        for _ in range(warm):
            fn()
        self.torch.cuda.synchronize()
        a, b = self.event(), self.event()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        self.torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    def region(self, fn, steps, warm=3):
        """One region of exactly `steps` calls of `fn` between barriers: milliseconds, max over ranks."""
        for _ in range(warm):
            fn()
        self.barrier()
        a, b = self.event(), self.event()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        self.barrier()
        return self.max_over_ranks([a.elapsed_time(b)])[0]


def _judge(torch, ours, seq32, truth64, scale=1.0):
    """Acceptance for slowly decaying coefficients (c close to 1), where two valid fp32 evaluation
    orders already differ by more than rtol 1e-4 / atol 1e-5 near zero crossings: the error against
    the fp64 evaluation may be at most twice the sequential fp32 operator's own error against it
    (plus atol), and the share of elements outside the nominal tolerance at most twice the sequential
    operator's own share (or 1e-4 of the elements).  Returns (ok, max error, share outside)."""
    o, s, t = ours.double() / scale, seq32.double() / scale, truth64 / scale
    err, err_seq = float((o - t).abs().max()), float((s - t).abs().max())
    tol = ATOL + RTOL * t.abs()
    miss, miss_seq = float(((o - t).abs() > tol).double().mean()), float(((s - t).abs() > tol).double().mean())
    ok = err <= 2.0 * err_seq + ATOL and miss <= max(1e-4, 2.0 * miss_seq)
    return ok, err, miss


# ======================================================================================================
#  the GPU arm
# ======================================================================================================
def run_ours(args):
    ctx = Ctx()
    torch, dist, dev, rank, world = ctx.torch, ctx.dist, ctx.dev, ctx.rank, ctx.world

    import linrec_b200
    from linrec_b200 import _capi
    from linrec_b200 import ops as lr_ops
    C = linrec_b200._C
    PIPE = _capi.KIND_PIPE

    def fwd(x, c, y, rev=False, **kw):
        lr_ops._launch(PIPE, False, (x, c), rev, kw, outs=(y,))

    def bwd(dy, c, y, dx, dc, rev=False, **kw):
        lr_ops._launch(PIPE, True, (dy, c, y), rev, kw, outs=(dx, dc))

    peak, peak_kind = _peak()
    steps, warmup, regions = args.steps, max(args.warmup, 3), max(args.regions, 1)

    # ---- headline: device resident, inputs and results allocated once ----------------------------------
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    x = torch.randn(SHAPE, device=dev, generator=g)
    c = torch.empty(SHAPE, device=dev).uniform_(C_RANGE[0], C_RANGE[1], generator=g)
    dy = torch.randn(SHAPE, device=dev, generator=g)
    y, dx, dc = (torch.empty(SHAPE, device=dev) for _ in range(3))
    n_elem = x.numel()
    step_bytes = n_elem * (BYTES_PER_ELEM_FWD + BYTES_PER_ELEM_BWD)

    def step():
        fwd(x, c, y)
        bwd(dy, c, y, dx, dc)

    sampler = ClockSampler(ctx.local) if rank == 0 else None
    if sampler:
        sampler.prepare()
    ev = [[[ctx.event() for _ in range(3)] for _ in range(steps)] for _ in range(regions)]
    marks = [(ctx.event(), ctx.event()) for _ in range(regions)]
    for _ in range(warmup):
        step()
    linrec_b200.check_status()
    ctx.barrier()
    alloc0 = ctx.alloc_counters()
    launches0 = C.launch_count()
    for r in range(regions):
        ctx.barrier()
        marks[r][0].record()
        for i in range(steps):
            ev[r][i][0].record()
            fwd(x, c, y)
            ev[r][i][1].record()
            bwd(dy, c, y, dx, dc)
            ev[r][i][2].record()
        marks[r][1].record()
        if sampler:
            sampler.sample_while_busy(marks[r][1].query)
        ctx.barrier()
    launches = (C.launch_count() - launches0) // regions
    alloc1 = ctx.alloc_counters()
    region_ms_local = [a.elapsed_time(b) for a, b in marks]
    region_ms = ctx.max_over_ranks(region_ms_local)
    order = sorted(range(regions), key=lambda r: region_ms[r])
    med = order[(regions - 1) // 2]            # the median region (lower median for an even count)
    total_ms = region_ms[med]
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev[med])
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev[med])
    step_ms = [e[0].elapsed_time(e[2]) for e in ev[med]]
    all_step_ms = [e[0].elapsed_time(e[2]) for r in range(regions) for e in ev[r]]
    clocks = sampler.summary() if sampler else None
    linrec_b200.check_status()
    value = world * step_bytes * steps / (total_ms * 1e-3) / 1e9
    no_alloc = alloc1 == alloc0
    del ev, marks

    # ---- one GPU: side measurements and the other configurations ----------------------------------------
    ceiling = axis = regimes = None
    if world == 1:
        tmp = torch.empty_like(x)
        ms = ctx.timed(lambda: torch.mul(x, c, out=tmp), 20)
        ceiling = {"op": "torch.mul(x, c, out=y), 12 B per element", "ms": ms, "gbps": n_elem * 12 / (ms * 1e-3) / 1e9}
        del tmp
        # the same problem laid out (batch, sequence, channel) and scanned along the middle axis where it lies
        xa, ca, dya = (t.view(SHAPE[0], SHAPE[2], SHAPE[1]) for t in (x, c, dy))
        ya = lr_ops.linrec_dim_fwd(xa, ca, 1, False)
        f_ms = ctx.timed(lambda: lr_ops.linrec_dim_fwd(xa, ca, 1, False), 10, warm=1)
        b_ms = ctx.timed(lambda: lr_ops.linrec_dim_bwd(dya, ca, ya, 1, False), 10, warm=1)
        linrec_b200.check_status()
        axis = {"workload": "(16, 8192, 2048) fp32, scan along the middle axis, no transposed copies",
                "fwd_gbps": n_elem * BYTES_PER_ELEM_FWD / (f_ms * 1e-3) / 1e9,
                "bwd_gbps": n_elem * BYTES_PER_ELEM_BWD / (b_ms * 1e-3) / 1e9,
                "value": step_bytes / ((f_ms + b_ms) * 1e-3) / 1e9, "unit": "GB/s"}
        del ya, xa, ca, dya
        if not args.no_regimes:
            regimes = _regimes(ctx, fwd, bwd, x, c, dy, y, dx, dc, peak)
            c.uniform_(C_RANGE[0], C_RANGE[1], generator=g)     # the sweep redrew the coefficients from U[0,1)

    # ---- end to end from pinned host buffers through the public API -----------------------------------
    fwd(x, c, y)
    e2e = _e2e(ctx, linrec_b200, x, c, dy, y, step_bytes, n_elem, steps)
    del x, c, dy, y, dx, dc
    torch.cuda.empty_cache()

    # ---- the multi-GPU configuration: (8192, 2^20), split by rows and by columns ------------------------
    cfg5 = None if args.no_cfg5 else _cfg5(ctx, linrec_b200, fwd, bwd, peak, steps)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    achieved = n_elem * BYTES_PER_ELEM_BWD / (bwd_ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": "linrec_tma_kernel<float,16,512,1,1,BWD> (backward operator; 8192-element tiles, one row per tile)",
            "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
            "traffic": (NCU_DRAM_BYTES_PER_ELEM_BWD * n_elem) if NCU_DRAM_BYTES_PER_ELEM_BWD else None,
            "algorithmic_bytes_per_launch": n_elem * BYTES_PER_ELEM_BWD, "ms_per_launch": bwd_ms,
            "frac_of_nominal_8TBs": achieved / 8000.0, "elementwise_ceiling": ceiling,
            "forward": {"achieved": n_elem * BYTES_PER_ELEM_FWD / (fwd_ms * 1e-3) / 1e9, "ms_per_launch": fwd_ms,
                        "frac": n_elem * BYTES_PER_ELEM_FWD / (fwd_ms * 1e-3) / 1e9 / peak}}

    cpu = None
    if world == 1 and not args.no_cpu:
        rows = 1024
        sec, info = _cpu_reference_run(3, 1, rows)
        more = 4096
        sec_more, _ = _cpu_reference_run(1, 0, more, with_c_port=False)
        cpu = {"value": rows * SHAPE[-1] * 32 / sec / 1e9, "unit": "GB/s", "cores": info["torch_threads"],
               "kind": "port",
               "sample": f"{rows} of 32768 rows x {SHAPE[-1]} (fwd+bwd), torch restatement of the reference's "
                         "Python loop on the host cores", **info,
               "more_rows": {"rows": more, "value": more * SHAPE[-1] * 32 / sec_more / 1e9,
                             "note": "the loop walks columns of a row-major tensor: more rows per step do not raise its throughput"}}

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": total_ms / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "autograd fwd+bwd, x~N(0,1), c~U(0.9,1), fp32, (16,2048,8192) per GPU "
                               "(numseq 32768, seqlen 8192)",
                   "sharding": "channel (rows) sharded, no data-path collective",
                   "l2": "inputs larger than L2 (1 GiB per tensor, 6 tensors)",
                   "elements_per_gpu": n_elem, "bytes_per_element": 32,
                   "timing": f"{regions} regions of {steps} steps, each between barriers; value = median region"},
        "regions_ms": region_ms, "regions_value": [world * step_bytes * steps / (m * 1e-3) / 1e9 for m in region_ms],
        "median_region": med,
        "step_ms_median": statistics.median(step_ms), "step_ms_max": max(step_ms),
        "step_ms_argmax": step_ms.index(max(step_ms)),
        "all_regions_step_ms_max": max(all_step_ms), "all_regions_step_ms_median": statistics.median(all_step_ms),
        "allocator": {"before": alloc0, "after": alloc1, "no_allocation_in_timed_regions": no_alloc},
        "gelem_per_s": world * n_elem * steps / (total_ms * 1e-3) / 1e9,
        "frac_of_measured_peak": value / (world * peak),
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "cfg5": cfg5,
        "regimes": regimes,
        "axis_scan": axis,
        "roofline": roof,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------
def _regimes(ctx, fwd, bwd, x, c, dy, y, dx, dc, peak):
    """Configurations 1, 2 and 4 of the task definition on one GPU, device resident, event timed, 20
    launches each after 3 warm-up launches.  The buffers of the headline are reused as flat storage
    (timing does not depend on the values; the coefficients are redrawn from U[0,1) as those
    configurations name them)."""
    torch = ctx.torch
    N = 1 << 28
    flat = [t.view(-1) for t in (x, c, dy, y, dx, dc)]
    flat[1].uniform_(0.0, 1.0)
    half = [torch.empty(N, dtype=torch.bfloat16, device=ctx.dev) for _ in range(3)]   # x, c, dy in bf16 storage
    for h, f in zip(half, flat[:3]):
        h.copy_(f)
    half_out = [f.view(torch.bfloat16)[:N] for f in flat[3:]]

    def views(rows, L, dtype):
        src = (flat[:3] + flat[3:]) if dtype == "f32" else (half + half_out)
        return [t[:rows * L].view(rows, L) for t in src]

    def one(rows, L, dtype, which, rev=False, n=20):
        vx, vc, vdy, vy, vdx, vdc = views(rows, L, dtype)
        size = 4 if dtype == "f32" else 2
        if which == "fwd":
            ms = ctx.timed(lambda: fwd(vx, vc, vy, rev), n)
            nbytes = rows * L * 3 * size
        else:
            fwd(vx, vc, vy, rev)
            ms = ctx.timed(lambda: bwd(vdy, vc, vy, vdx, vdc, rev), n)
            nbytes = rows * L * 5 * size
        gbps = nbytes / (ms * 1e-3) / 1e9
        return {"rows": rows, "seqlen": L, "dtype": dtype, "pass": which, "reverse": rev, "us_per_launch": ms * 1e3,
                "gbps": gbps, "frac_of_measured_peak": gbps / peak, "gelem_per_s": rows * L / (ms * 1e-3) / 1e9}

    out = {"launches_per_entry": 20, "note": "GB/s at 12 / 20 B per fp32 element (6 / 10 B per bf16 element), forward / backward"}
    # configuration 1: (512, 4096) forward -- 24 MiB in all, L2 resident, launch-latency bound
    e = one(512, 4096, "f32", "fwd")
    vx, vc, _, vy, _, _ = views(512, 4096, "f32")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(200):
        fwd(vx, vc, vy)
    host_us = (time.perf_counter() - t0) / 200 * 1e6
    torch.cuda.synchronize()
    e.update({"l2_resident": True, "host_us_per_call": host_us})
    # the host call takes longer than the kernel: the same 20 launches captured in a CUDA graph and
    # replayed show the device side alone
    try:
        side = torch.cuda.Stream(device=ctx.dev)
        side.wait_stream(torch.cuda.current_stream(ctx.dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fwd(vx, vc, vy)                       # the workspace of this stream exists before the capture
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(20):
                fwd(vx, vc, vy)
        for _ in range(3):
            graph.replay()
        ms = ctx.timed(graph.replay, 5) / 20
        e["graph_replay_us_per_launch"] = ms * 1e3
        e["graph_replay_gbps"] = 512 * 4096 * 12 / (ms * 1e-3) / 1e9
        del graph
    except Exception as exc:                       # the figure is a side note: never fail the bench for it
        e["graph_replay_us_per_launch"] = None
        e["graph_replay_error"] = str(exc)[:200]
    out["cfg1"] = e
    # configuration 2: (512, 65536) forward in both directions
    out["cfg2"] = [one(512, 65536, "f32", "fwd", rev) for rev in (False, True)]
    # configuration 4: 2^28 elements, L = 2^8 ... 2^20, fp32 and bf16 storage, forward and backward
    sweep = []
    for log2l in range(8, 21, 2):
        L = 1 << log2l
        for dtype in ("f32", "bf16"):
            for which in ("fwd", "bwd"):
                sweep.append(one(N // L, L, dtype, which))
    out["cfg4"] = sweep
    out["cfg4_min_frac_f32"] = min(e["frac_of_measured_peak"] for e in sweep if e["dtype"] == "f32")
    out["cfg4_min_frac_bf16"] = min(e["frac_of_measured_peak"] for e in sweep if e["dtype"] == "bf16")
    # rows that are not whole 16-byte chunks (any-alignment kernel) and rows of 16-byte chunks that are not
    # whole 128-byte lines (cp.async kernel)
    out["odd_lengths"] = [one(N // L, L, "f32", w) for L in (1001, 10001, 1000, 10000) for w in ("fwd", "bwd")]
    # a handful of very long rows
    out["few_long_rows"] = [one(r, L, "f32", w) for (r, L) in ((8, 1 << 25), (1, 1 << 28)) for w in ("fwd", "bwd")]
    import linrec_b200
    linrec_b200.check_status()
    return out


# ------------------------------------------------------------------------------------------------------
def _numa_of_gpu(torch, index):
    try:
        import pynvml
        pynvml.nvmlInit()
        vis = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip().isdigit()]
        phys = int(vis[index]) if index < len(vis) else index
        info = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(phys))
        bus_id = info.busId.decode() if isinstance(info.busId, bytes) else str(info.busId)
        path = f"/sys/bus/pci/devices/{bus_id[-12:].lower()}/numa_node"
        with open(path) as f:
            return int(f.read().strip())
    except Exception:
        return None


def _e2e(ctx, linrec_b200, x, c, dy, y, step_bytes, n_elem, steps):
    """The step through `linrec_b200.host.linrec_fwd_bwd_host` from pinned host buffers (row slabs; copy-in
    of slab i+1, the two scans of slab i and copy-out of slab i-1 overlap on three streams), the same
    copies with no kernel at all, and the step through autograd on whole tensors."""
    torch, dev, world = ctx.torch, ctx.dev, ctx.world
    from linrec_b200 import host as lr_host
    k = max(1, min(steps, 3))
    hx, hc, hdy = (torch.empty(SHAPE, pin_memory=True) for _ in range(3))
    hy, hdx, hdc = (torch.empty(SHAPE, pin_memory=True) for _ in range(3))
    hx.copy_(x); hc.copy_(c); hdy.copy_(dy)
    fwd_y = y.cpu()     # the forward result of the device-resident run, same inputs

    def e2e_step():
        lr_host.linrec_fwd_bwd_host(hx, hc, hdy, reverse=False, out=(hy, hdx, hdc), device=dev)

    ms = ctx.region(e2e_step, k, warm=1)
    value = world * step_bytes * k / (ms * 1e-3) / 1e9
    ok = bool(torch.equal(hy, fwd_y))
    del fwd_y

    # the ceiling: the same bytes in the same 64 MiB pieces, both directions at once, no kernels
    rows = SHAPE[0] * SHAPE[1]
    piece = max(1, (64 << 20) // (SHAPE[2] * 4))
    dbuf = [torch.empty((piece, SHAPE[2]), device=dev) for _ in range(6)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    hin = [t.view(rows, SHAPE[2]) for t in (hx, hc, hdy)]
    hout = [t.view(rows, SHAPE[2]) for t in (hy, hdx, hdc)]

    def copy_only():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur); s_out.wait_stream(cur)
        for r0 in range(0, rows, piece):
            n = min(piece, rows - r0)
            with torch.cuda.stream(s_in):
                for j in range(3):
                    dbuf[j][:n].copy_(hin[j][r0:r0 + n], non_blocking=True)
            with torch.cuda.stream(s_out):
                for j in range(3):
                    hout[j][r0:r0 + n].copy_(dbuf[3 + j][:n], non_blocking=True)
        cur.wait_stream(s_in); cur.wait_stream(s_out)

    copy_ms = ctx.region(copy_only, k, warm=1)
    del dbuf

    # the same through autograd on whole tensors (copy in, scan, copy out, nothing overlapped)
    def autograd_step():
        xd = hx.to(dev, non_blocking=True).requires_grad_(True)
        cd = hc.to(dev, non_blocking=True).requires_grad_(True)
        dyd = hdy.to(dev, non_blocking=True)
        yd = linrec_b200.linrec(xd, cd, reverse=False)
        gx, gc = torch.autograd.grad(yd, (xd, cd), dyd)
        hy.copy_(yd.detach(), non_blocking=True)
        hdx.copy_(gx, non_blocking=True)
        hdc.copy_(gc, non_blocking=True)

    auto_ms = ctx.region(autograd_step, k, warm=1)
    numa = _numa_of_gpu(torch, ctx.local)
    return {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 3 * n_elem * 4, "d2h_bytes_per_step": 3 * n_elem * 4,
            "steps": k, "ms_per_step": ms / k,
            "api": "linrec_b200.host.linrec_fwd_bwd_host (row slabs, copies and scans overlapped)",
            "matches_device_run": ok,
            "copy_only": {"ms_per_step": copy_ms / k,
                          "gb_per_s_each_direction": world * 3 * n_elem * 4 * k / (copy_ms * 1e-3) / 1e9,
                          "what": "the same 3 GiB in + 3 GiB out per rank in 64 MiB pieces on two streams, no kernels, "
                                  "all ranks at once"},
            "frac_of_copy_ceiling": copy_ms / ms,
            "host": {"gpu_numa_node_rank0": numa, "cpus_visible": _host_threads(),
                     "note": "pinned buffers are allocated by the rank's own process; no NUMA binding is applied"},
            "autograd_whole_tensor": {"value": world * step_bytes * k / (auto_ms * 1e-3) / 1e9, "ms_per_step": auto_ms / k,
                                      "api": "linrec_b200.linrec + torch.autograd.grad"}}


# ------------------------------------------------------------------------------------------------------
def _cfg5(ctx, linrec_b200, fwd, bwd, peak, steps):
    """fp32 (8192, 2^20), x ~ N(0,1), c ~ U(0.99, 1), dy ~ N(0,1), forward + backward: 2^33 elements,
    32 GiB per tensor, 275 GB algorithmic per step, over all ranks (strong scaling).

    channel  every rank scans its 8192/N rows; no communication.
    seq      every rank holds the columns [rank*L/N, (rank+1)*L/N) of all 8192 rows: local scan, one
             all-gather of the per-row records, fused fix-up (and the same with the records read from
             the peers' memory by the fix-up kernel instead of the all-gather).

    One GPU cannot hold the six tensors (192 GiB): there the problem is worked through in eight row
    slabs of (1024, 2^20) on one fixed set of device buffers, the same bytes per element through the
    same kernels; with two or more ranks each rank holds its whole share.  Both layouts use the same
    storage, read as (rows/N, 2^20) or as (8192, 2^20/N).

    Parity bit: eight sampled rows of y, dx and dc are compared with the unsharded single-device
    operator on the gathered full rows, and judged -- like the full-size test of this configuration --
    against a double-precision evaluation on the device (the sequential operator in fp64) relative to
    the sequential fp32 operator's own error."""
    torch, dist, dev, world, rank = ctx.torch, ctx.dist, ctx.dev, ctx.world, ctx.rank
    from linrec_b200 import _capi, sharded
    C = linrec_b200._C
    ROWS, L = 8192, 1 << 20
    if ROWS % world or L % world:
        return {"skipped": f"{world} ranks do not divide (8192, 2^20)"}
    slabs = 8 if world == 1 else 1
    n_local = ROWS * L // world // slabs          # elements per tensor held on this rank
    k = max(1, min(steps, 5))
    g = torch.Generator(device=dev).manual_seed(SEED + 500 + rank)
    store = [torch.empty(n_local, device=dev) for _ in range(6)]
    store[0].normal_(generator=g)
    store[1].uniform_(0.99, 1.0, generator=g)
    store[2].normal_(generator=g)
    total_bytes = ROWS * L * 32

    def block(ms_per_step, extra):
        gbps = total_bytes / (ms_per_step * 1e-3) / 1e9
        return {"value": gbps, "unit": "GB/s", "ms_per_step": ms_per_step, "steps": k, "scaling": "strong",
                "frac_of_measured_peak": gbps / (world * peak), **extra}

    def sample_rows(n):
        return torch.tensor(sorted({0, n - 1, *[(i * 2654435761) % n for i in range(1, 7)]}), device=dev)

    def judge_rows(xr, cr, dyr, ours):
        """`ours` = (y, dx, dc) of the sampled full rows as computed by the sharded run."""
        y1, dx1, dc1 = (torch.empty_like(xr) for _ in range(3))
        fwd(xr, cr, y1); bwd(dyr, cr, y1, dx1, dc1)
        ys = C.linrec_ref_fwd(inputs=xr, coeffs=cr)
        dxs, dcs = C.linrec_ref_bwd(d_outputs=dyr, coeffs=cr, outputs=ys)
        y64 = C.linrec_ref_fwd(inputs=xr.double(), coeffs=cr.double())
        dx64, dc64 = C.linrec_ref_bwd(d_outputs=dyr.double(), coeffs=cr.double(), outputs=y64)
        scale = max(1.0, float(y64.abs().max()))
        res = {}
        ok = True
        for name, o, s32, t64, single, sc in (("y", ours[0], ys, y64, y1, 1.0), ("dx", ours[1], dxs, dx64, dx1, 1.0),
                                               ("dc", ours[2], dcs, dc64, dc1, scale)):
            good, err, miss = _judge(torch, o, s32, t64, sc)
            ok = ok and good and bool(torch.isfinite(o).all())
            res[name] = {"max_err_vs_fp64": err, "share_outside_nominal_tolerance": miss,
                         "max_abs_diff_vs_single_device": float((o - single).abs().max())}
        return ok, res

    out = {"workload": "fwd+bwd, fp32 (8192, 2^20) global, x~N(0,1), c~U(0.99,1), dy~N(0,1); 2^33 elements, 32 B each",
           "layout": f"{slabs} row slabs of ({ROWS // world // slabs}, 2^20) per step on one set of device buffers (six tensors "
                     "of the whole problem are 192 GiB)" if slabs > 1 else "each rank holds its whole share of the six tensors"}

    # ---- channel (row) sharding ---------------------------------------------------------------------
    rows_c = ROWS // world // slabs
    X, Cc, DY, Y, DX, DC = (t.view(rows_c, L) for t in store)

    def chan_step():
        for _ in range(slabs):
            fwd(X, Cc, Y)
            bwd(DY, Cc, Y, DX, DC)

    ms = ctx.region(chan_step, k, warm=2) / k
    rs = sample_rows(rows_c)
    ok, detail = judge_rows(X[rs].contiguous(), Cc[rs].contiguous(), DY[rs].contiguous(), (Y[rs], DX[rs], DC[rs]))
    linrec_b200.check_status()
    out["channel"] = block(ms, {"collective": "none", "rows_per_rank": ROWS // world,
                                "matches_single_device": ctx.all_true(ok), "parity_rank0": detail})

    # ---- sequence (column) sharding ----------------------------------------------------------------------
    Ls = L // world
    rows_s = ROWS // slabs
    X, Cc, DY, Y, DX, DC = (t.view(rows_s, Ls) for t in store)
    exchange = None
    if world > 1:
        try:
            exchange = sharded.PeerExchange(rows_s)
        except Exception as exc:      # symmetric memory unavailable: the all-gather path still runs
            print(f"rank {rank}: peer exchange unavailable: {exc}", file=sys.stderr)
        if not ctx.all_true(exchange is not None):   # the exchange is collective: every rank or none
            exchange = None

    def seq_step(ex=None):
        for _ in range(slabs):
            if world == 1:
                fwd(X, Cc, Y)
                bwd(DY, Cc, Y, DX, DC)
            else:
                sharded.seq_sharded_fwd(X, Cc, False, exchange=ex, out=Y)
                sharded.seq_sharded_bwd(DY, Cc, Y, False, exchange=ex, out=(DX, DC))

    def gather_cols(t):
        """Sampled rows of a column-sharded tensor, all columns, on every rank."""
        part = t[rs].contiguous()
        if world == 1:
            return part
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        return torch.cat(parts, dim=1)

    rs = sample_rows(rows_s)
    ms = ctx.region(seq_step, k, warm=2) / k
    ok, detail = judge_rows(gather_cols(X), gather_cols(Cc), gather_cols(DY), tuple(gather_cols(t) for t in (Y, DX, DC)))
    linrec_b200.check_status()
    seq = block(ms, {"collective": "one all-gather of 8 B (fwd) / 16 B (bwd) per row and rank" if world > 1 else "none (one rank)",
                     "columns_per_rank": Ls, "matches_single_device": ctx.all_true(ok), "parity_rank0": detail})
    if world > 1:
        # device time of the three phases, measured in a separate instrumented pass
        kern = sharded.CudaShardKernels()
        ph = {n: [] for n in ("fwd_scan", "fwd_gather", "fwd_fixup", "bwd_scan", "bwd_gather", "bwd_fixup")}
        for _ in range(3):
            e = [ctx.event() for _ in range(7)]
            ctx.barrier()
            e[0].record()
            _, rec = kern.fwd_carry(X, Cc, False, rank, world, out=Y)
            e[1].record()
            gathered = sharded._gather(rec, None)
            e[2].record()
            kern.fwd_fixup(X, Y, Cc, gathered, False, rank, world)
            e[3].record()
            _, _, rec, _, _, _ = kern.bwd_carry(DY, Cc, Y, False, rank, world, out=(DX, DC))
            e[4].record()
            gathered = sharded._gather(rec, None)
            e[5].record()
            kern.bwd_fixup(DY, DX, DC, Cc, Y, gathered, False, rank, world)
            e[6].record()
            ctx.barrier()
            for i, n in enumerate(ph):
                ph[n].append(e[i].elapsed_time(e[i + 1]))
        seq["phases_ms_max_over_ranks"] = dict(zip(ph, ctx.max_over_ranks([statistics.median(v) for v in ph.values()])))
        if exchange is not None:
            ms_p = ctx.region(lambda: seq_step(exchange), k, warm=2) / k
            okp, detail_p = judge_rows(gather_cols(X), gather_cols(Cc), gather_cols(DY), tuple(gather_cols(t) for t in (Y, DX, DC)))
            exchange.poll(wait=True)
            linrec_b200.check_status()
            seq["peer_memory_exchange"] = block(ms_p, {"collective": "none: records read from the peers' memory by the fix-up kernel",
                                                      "matches_single_device": ctx.all_true(okp), "parity_rank0": detail_p})
    out["seq"] = seq
    del store, X, Cc, DY, Y, DX, DC
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps each; the median one is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cfg5", action="store_true", help="skip the (8192, 2^20) row- and column-sharded measurements")
    ap.add_argument("--no-regimes", action="store_true", help="skip configurations 1, 2 and 4 (one GPU only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
