#!/usr/bin/env python
"""Benchmark of the advantage hot path: elements/s and achieved HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

A step is one pass of the path over one `[segments, horizon]` fp32 buffer that
is already resident in HBM: the advantage kernel with its fused per-segment
|advantage| sums, the priority weights, (N > 1) the exchange of the weight
total between the GPUs, and the sampling probabilities.  The small launches of
step i run on a side stream while the advantage kernel of step i+1 runs; all K
steps finish inside the timed region.

With N GPUs (one process per GPU) the headline is weak scaling: every rank owns
its own `segments x horizon` buffer.  Every N > 1 line also carries
`strong_scaling`: ONE buffer of that size split by rows over the ranks, with
the kernel-only and the kernel + exchange times of a step.  The weight total
crosses GPUs inside the priority kernels (stores into peer-mapped mailboxes);
`--exchange nccl` uses a torch.distributed all-reduce instead.

One JSON line is printed by rank 0.  `value` is the whole-job rate with
device-resident inputs, `e2e` the same metric through the host-buffer C-ABI
entry point with pinned host inputs and outputs (copies inside the timed
region) beside the time of its bare copies, `roofline` the advantage kernel's
algorithmic bytes over its CUDA-event duration against the measured HBM copy
peak, `small_workloads` (N = 1) the steady-state kernel time of the other
configurations with a parity bit each, `neighbour_kernels` (N = 1) the sampler
prologue, the minibatch gather and the rollout writer on the headline's buffer
shape, and `cpu_baseline` the reference CPU op timed on this machine's cores.

`--impl reference` times only the reference's own CPU implementation (the
build under oracle/_ref/ when present, else the oracle port) and prints the
same line shape.
"""
import argparse
import collections
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from pufferlib_b200.workloads import WORKLOADS, make_inputs  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
BYTES_PER_ELEMENT = 20          # 4 fp32 inputs read + 1 fp32 output written
PRIO_ALPHA = 0.8                # config/default.ini:60
DEPTH = int(os.environ.get("PUFF_BENCH_DEPTH", "3"))   # steps whose side-stream work may be outstanding
FALLBACK_HBM_GBS = 6650.0


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi in loop mode, read-only; samples are matched to the timed
    windows by wall-clock time."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        self.path = None
        try:
            fd, self.path = tempfile.mkstemp(prefix="puff_clocks_", suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, windows):
        """windows: list of (t0, t1) wall-clock spans; returns the clocks dict."""
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        rows = []
        try:
            import datetime
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(parts[1]), float(parts[2]), parts[3], parts[5:9]))
                except Exception:
                    continue
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        if not rows:
            return None
        inside = [r for r in rows if any(t0 <= r[0] <= t1 for t0, t1 in windows)]
        scope = "timed region"
        if not inside:
            inside, scope = rows, "whole run (timed region shorter than the sampling period)"
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in inside for n, v in zip(names, r[4]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": inside[0][2],
                "reasons": reasons, "samples": len(inside), "scope": scope}


# ---------------------------------------------------------------------------
# reference / CPU arm
# ---------------------------------------------------------------------------
def cpu_reference_rate(wl, seconds_budget, want_single=True):
    """Elements/s of the reference CPU op on this machine: as shipped (one
    thread) and from a thread pool over contiguous row slices on all physical
    cores (the op has no internal parallelism; torch releases the GIL)."""
    import numpy as np
    import psutil
    from concurrent.futures import ThreadPoolExecutor
    from oracle import puff_oracle

    ref = puff_oracle.load_reference()
    kind = "reference" if ref is not None else "port"
    inputs = make_inputs(wl)
    adv = torch.zeros_like(inputs[0])
    hyper = wl.hyper()
    S, H = wl.segments, wl.horizon
    torch.set_num_threads(1)

    if ref is not None:
        def run_rows(lo, hi):
            ref(*[t[lo:hi] for t in inputs], adv[lo:hi], *hyper)
    else:
        np_in = [t.numpy() for t in inputs]
        np_adv = adv.numpy()

        def run_rows(lo, hi):
            puff_oracle.advantage(*[a[lo:hi] for a in np_in], np_adv[lo:hi], *hyper)

    # one thread, a slice worth ~0.25 s
    single = None
    if want_single:
        rows1 = max(1, min(S, int(30e6) // H))
        run_rows(0, min(rows1, 1024))
        t0 = time.perf_counter()
        run_rows(0, rows1)
        single = rows1 * H / (time.perf_counter() - t0)

    cores = psutil.cpu_count(logical=False) or os.cpu_count() or 1
    try:
        cores = min(cores, len(os.sched_getaffinity(0)))
    except Exception:
        pass
    bounds = [((i * S) // cores, ((i + 1) * S) // cores) for i in range(cores)]
    times = []
    with ThreadPoolExecutor(max_workers=cores) as pool:
        list(pool.map(lambda b: run_rows(*b), bounds))   # warm
        t_end = time.perf_counter() + seconds_budget
        while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
            t0 = time.perf_counter()
            list(pool.map(lambda b: run_rows(*b), bounds))
            times.append(time.perf_counter() - t0)
    pooled = S * H / statistics.median(times)
    return {"kind": kind, "cores": cores, "pooled": pooled, "single": single, "passes": len(times),
            "sample": f"{len(times)} full passes over {S}x{H} from {cores} threads over row slices"
                      + (f"; 1 thread on {rows1}x{H}" if want_single else "")}


def run_reference_arm(args, wl, rank, world):
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    # bound the whole run: every step is one pooled pass over a sample of the workload
    import psutil
    from concurrent.futures import ThreadPoolExecutor
    from oracle import puff_oracle
    ref = puff_oracle.load_reference()
    kind = "reference" if ref is not None else "port"
    cores = psutil.cpu_count(logical=False) or os.cpu_count() or 1
    try:
        cores = min(cores, len(os.sched_getaffinity(0)))
    except Exception:
        pass
    torch.set_num_threads(1)
    budget = 90.0 / (steps + warmup)
    rows = int(min(wl.segments, max(cores * 8, budget * 100e6 * max(1, cores // 2) / wl.horizon)))
    sample = wl.with_segments(rows)
    inputs = make_inputs(sample)
    adv = torch.zeros_like(inputs[0])
    hyper = wl.hyper()
    if ref is not None:
        def run_rows(b):
            ref(*[t[b[0]:b[1]] for t in inputs], adv[b[0]:b[1]], *hyper)
    else:
        np_in = [t.numpy() for t in inputs]
        np_adv = adv.numpy()

        def run_rows(b):
            puff_oracle.advantage(*[a[b[0]:b[1]] for a in np_in], np_adv[b[0]:b[1]], *hyper)
    bounds = [((i * rows) // cores, ((i + 1) * rows) // cores) for i in range(cores)]
    with ThreadPoolExecutor(max_workers=cores) as pool:
        for _ in range(warmup):
            list(pool.map(run_rows, bounds))
        t0 = time.perf_counter()
        for _ in range(steps):
            list(pool.map(run_rows, bounds))
        dt = time.perf_counter() - t0
    t1 = time.perf_counter()
    run_rows((0, max(1, rows // cores)))
    single = max(1, rows // cores) * wl.horizon / (time.perf_counter() - t1)
    value = rows * wl.horizon * steps / dt
    line = {
        "impl": "reference", "metric": "advantage elements/sec", "value": value, "unit": "elements/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": 1e3 * dt / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(wl, args.gpus),
        "cpu_baseline": {"value": value, "unit": "elements/s", "cores": cores, "kind": kind,
                         "sample": f"each step: one pass over the first {rows} of {wl.segments} segments x {wl.horizon}, "
                                   f"row slices on {cores} threads (the op itself is single-threaded)",
                         "single_thread_value": single},
        "e2e": {"value": value, "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "achieved_gbs": value * BYTES_PER_ELEMENT / 1e9,
    }
    print(json.dumps(line), flush=True)


def workload_config(wl, n_gpus):
    """The `config` object, identical in the B200 arm and the reference arm."""
    set_bytes = BYTES_PER_ELEMENT * wl.elements
    n_sets = rotation_sets(set_bytes)
    return {"workload": f"{wl.name}: {wl.segments}x{wl.horizon} fp32 per GPU",
            "segments_per_gpu": wl.segments, "horizon": wl.horizon,
            "global_segments": wl.segments * n_gpus,
            "gamma": wl.gamma, "lambda": wl.lam, "rho_clip": wl.rho_clip, "c_clip": wl.c_clip,
            "parallelism": f"segments sharded over {n_gpus} GPU(s), one fp64 scalar exchanged per step"
                           if n_gpus > 1 else "single GPU",
            "l2": "inputs larger than L2" if n_sets == 1 else
                  f"rotating over {n_sets} buffer sets ({n_sets * set_bytes >> 20} MiB > 2x L2)"}


def rotation_sets(set_bytes):
    """Buffer sets to rotate over so that consecutive launches never find their inputs in L2."""
    return 1 if set_bytes >= 2 * L2_BYTES else -(-2 * L2_BYTES // set_bytes)


# ---------------------------------------------------------------------------
# the B200 arm
# ---------------------------------------------------------------------------
MAX_GRAPH_STEPS = 500


class PathTimer:
    """Times the hot path over one rank's buffers.

    step(i): advantage kernel (+ fused sums) on the current stream; priority
    weights, the cross-GPU exchange of their total and the probabilities behind
    it on a side stream, overlapping the advantage kernel of step i+1.  The
    loops are captured into CUDA graphs (all steps in one graph, up to
    MAX_GRAPH_STEPS per graph) and replayed: the per-step host work -- operator
    calls on every rank -- is otherwise comparable to the kernel time.  The
    side stream joins the main one once per graph, inside the timed region."""

    def __init__(self, wl_local, host_inputs, dev, sharded, hyper, world, fence):
        self.S, self.H = wl_local.segments, wl_local.horizon
        self.elems = self.S * self.H
        self.hyper, self.sharded, self.world, self.fence = hyper, sharded, world, fence
        self.n_sets = rotation_sets(BYTES_PER_ELEMENT * self.elems)
        self.sets = []
        for i in range(self.n_sets):
            ins = [t.to(dev) for t in host_inputs] if i == 0 else [t.clone() for t in self.sets[0][:4]]
            # DEPTH sum buffers per set: the priority launches of step i read one on the side
            # stream while the advantage kernels of the following steps fill the others
            self.sets.append(ins + [torch.zeros((self.S, self.H), device=dev),
                                    tuple(torch.empty(self.S, device=dev) for _ in range(DEPTH))])
        self.side_stream = torch.cuda.Stream(priority=-1)
        self.capture_stream = torch.cuda.Stream()
        self.pending = collections.deque()
        self.last = {}
        self.windows = []
        self.status_errors = []

    # -- one step in its three forms -------------------------------------------
    def step(self, i):
        v, r, d, w, adv, abs2 = self.sets[i % self.n_sets]
        main = torch.cuda.current_stream()
        while len(self.pending) >= DEPTH:      # the sum buffer of step i-DEPTH is free again
            main.wait_event(self.pending.popleft())
        probs, total, done = self.sharded.step_overlapped(v, r, d, w, adv, abs2[i % DEPTH], self.side_stream)
        self.pending.append(done)
        self.last["probs"], self.last["total"] = probs, total

    def step_serial(self, i):
        """Everything on one stream: kernel, then weights, exchange, probabilities."""
        v, r, d, w, adv, abs2 = self.sets[i % self.n_sets]
        self.sharded.kernels.advantage_prio(v, r, d, w, adv, abs2[i % DEPTH], self.hyper)
        self.last["probs"], self.last["total"] = self.sharded.priorities(abs2[i % DEPTH])

    def adv_only(self, i):
        v, r, d, w, adv, abs2 = self.sets[i % self.n_sets]
        self.sharded.kernels.advantage_prio(v, r, d, w, adv, abs2[i % DEPTH], self.hyper)

    def drain(self):
        main = torch.cuda.current_stream()
        while self.pending:
            main.wait_event(self.pending.popleft())

    # -- timing -----------------------------------------------------------------
    def _capture(self, fn, count):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.capture_stream):
            for i in range(count):
                fn(i)
            self.drain()          # join the side stream back into the capture
        return g

    def warm(self, fn, count):
        with torch.cuda.stream(self.capture_stream):
            for i in range(count):
                fn(i)
            self.drain()
        self.fence()

    def timed_graph(self, fn, total_steps):
        """ms for `total_steps` steps of fn, replayed from graphs; every launch of every step
        (side stream included) ends inside the timed region."""
        from pufferlib_b200 import cabi
        per = max(min(total_steps, MAX_GRAPH_STEPS), min(self.n_sets, total_steps))
        full, rem = divmod(total_steps, per)
        g_full = self._capture(fn, per)
        g_rem = self._capture(fn, rem) if rem else None
        g_full.replay()
        self.fence()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        t0.record()
        for _ in range(full):
            g_full.replay()
        if g_rem is not None:
            g_rem.replay()
        t1.record()
        self.fence()
        self.windows.append((w0, time.time()))
        self._check_status()
        return t0.elapsed_time(t1), per

    def timed_eager(self, fn, total_steps):
        from pufferlib_b200 import cabi
        self.fence()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        t0.record()
        for i in range(total_steps):
            fn(i)
        self.drain()                 # every step's side-stream work ends inside the timed region
        t1.record()
        self.fence()
        self.windows.append((w0, time.time()))
        self._check_status()
        return t0.elapsed_time(t1), 1

    def _check_status(self):
        """A bounded wait that gave up inside a kernel invalidates the timed region.  It is
        recorded and reported in the JSON line (`device_status`) rather than raised: one rank
        leaving early would strand the others in their next collective."""
        from pufferlib_b200 import cabi
        status = cabi.device_status()
        if status != 0:
            self.status_errors.append(f"{status}: {cabi.strerror(status)}")


def max_over_ranks(values, dev, world):
    if world == 1:
        return [float(v) for v in values]
    import torch.distributed as dist
    t = torch.tensor(list(values), device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def numa_bind(local_rank):
    """Run this process (and so place its pinned buffers, first touch) on the CPUs of the NUMA
    node its GPU hangs off, when the machine says which that is.  Returns what was done."""
    try:
        props = torch.cuda.get_device_properties(local_rank)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return {"node": None, "why": "the GPU reports no NUMA node"}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return {"node": node, "why": "none of the node's CPUs is in this process's affinity mask"}
        os.sched_setaffinity(0, cpus)
        return {"node": node, "cpus": len(cpus)}
    except Exception as exc:
        return {"node": None, "why": str(exc)[:120]}


def run_b200_arm(args, wl, rank, local_rank, world):
    import torch.distributed as dist
    import pufferlib_b200
    from pufferlib_b200 import cabi
    from pufferlib_b200.sharded import ShardedAdvantage
    from pufferlib_b200.workloads import shard_rows

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = numa_bind(local_rank) if world > 1 else None    # before any pinned allocation
    exchange, exchange_kind = None, "none (single GPU)"
    if world > 1:
        # the collective fallback's kernel has to slip in beside persistent advantage kernels
        # that fill every SM: give NCCL's stream (and the side stream) high priority
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
        exchange_kind = "torch.distributed all-reduce (NCCL)"
        if args.exchange == "p2p":
            try:
                from pufferlib_b200.exchange import PeerExchange
                exchange = PeerExchange.for_process_group()
                exchange_kind = "peer stores inside the priority kernels (puff_exchange, CUDA IPC mailboxes)"
            except Exception as exc:
                exchange_kind += f"; peer exchange unavailable: {str(exc)[:120]}"
            # all ranks must agree, or half of them would wait for pushes that never come
            ok = torch.tensor([1 if exchange is not None else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok) == 0 and exchange is not None:
                exchange.close()
                exchange = None
                exchange_kind = "torch.distributed all-reduce (NCCL); peer exchange unavailable on another rank"
    elif os.environ.get("PUFF_BENCH_EXCHANGE_WORLD1") == "1":
        # diagnosis: the exchange kernels (push into the own mailbox, gather from it) on one GPU
        from pufferlib_b200.exchange import PeerExchange
        exchange = PeerExchange(0, 1, want_handle=False)
        exchange_kind = "peer-exchange kernels with a world of one (diagnosis)"
    if args.reserve_sms > 0:
        cabi.set_tuning(reserve_sms=args.reserve_sms)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    S, H = wl.segments, wl.horizon
    hyper = wl.hyper()
    elems = S * H
    variant = args.variant
    pufferlib_b200.set_variant(variant)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    # ---- headline: every rank owns its own S x H buffer (weak scaling) ------------
    host = make_inputs(wl.with_segments(S, seed=wl.seed + rank), pin=True)
    sharded = ShardedAdvantage(S * world, H, hyper, PRIO_ALPHA, rank=rank, world=world, exchange=exchange)
    timer = PathTimer(wl, host, dev, sharded, hyper, world, fence)
    timer.warm(timer.step, max(warmup, timer.n_sets))
    kernel_name = cabi.last_kernel()
    sampler = ClockSampler(local_rank) if rank == 0 else None

    lc0 = cabi.launch_count()
    timer.step(0)
    timer.drain()
    launches_per_step = cabi.launch_count() - lc0
    fence()
    timed = timer.timed_eager if args.no_graph else timer.timed_graph
    ms_total, per_graph = timed(timer.step, steps)
    ko_total, _ = timed(timer.adv_only, steps)
    launches = launches_per_step * steps          # graph replays re-run the captured launches
    ms_total, ko_total = max_over_ranks([ms_total, ko_total], dev, world)
    kernel_ms = ko_total / steps                   # back-to-back advantage launches alone, launch gaps included
    value = elems * world * steps / (ms_total * 1e-3)
    timing = ("eager launches" if args.no_graph else
              f"CUDA graphs of {per_graph} steps replayed, side stream joined once per graph") + \
             "; kernel time = the same loop with the advantage launches only (launch gaps included)"

    # ---- the contract's split: ONE S x H buffer sharded over the ranks (strong scaling) ----
    strong = None
    if world > 1 and not args.no_strong:
        lo, hi = shard_rows(S, rank, world)
        full = make_inputs(wl)                     # the same global buffer on every rank
        local = [t[lo:hi].contiguous() for t in full]
        del full
        wl_local = wl.with_segments(hi - lo)
        sh = ShardedAdvantage(S, H, hyper, PRIO_ALPHA, rank=rank, world=world, exchange=exchange)
        st = PathTimer(wl_local, local, dev, sh, hyper, world, fence)
        st.warm(st.step, max(warmup, st.n_sets))
        n = max(steps, 200)                        # short steps: time enough of them
        a, _ = st.timed_graph(st.step, n)
        b, _ = st.timed_graph(st.adv_only, n)
        c, _ = st.timed_graph(st.step_serial, n)
        a, b, c = max_over_ranks([a, b, c], dev, world)
        strong = {"scaling": "strong", "global_segments": S, "segments_per_gpu": hi - lo, "steps": n,
                  "value": elems * n / (a * 1e-3), "unit": "elements/s", "ms_per_step": a / n,
                  "kernel_only_us": 1e3 * b / n, "kernel_plus_exchange_serial_us": 1e3 * c / n,
                  "exchange_serial_us": 1e3 * (c - b) / n,
                  "l2": f"rotating over {st.n_sets} buffer sets" if st.n_sets > 1 else "inputs larger than L2",
                  "what": "ms_per_step: exchange overlapped with the next step's kernel (as the headline); "
                          "kernel_plus_exchange_serial_us: kernel, weights, exchange, probabilities on one stream"}
        timer.windows += st.windows
        timer.status_errors += st.status_errors
        del st, local

    # ---- small and odd workloads: steady-state kernel time (single GPU only) -------
    small = neighbours = None
    if world == 1 and not args.no_small and args.workload == "cfg2" and args.segments == 0:
        small = time_small_workloads(dev, fence)
        neighbours = time_neighbour_kernels(dev, fence)

    # ---- the reference's own CUDA kernel on this GPU (secondary baseline) -----
    ref_cuda = None
    if rank == 0 and not args.no_ref_cuda:
        ref_cuda = time_reference_cuda_kernel(timer.sets, timer.n_sets, hyper, elems)

    # ---- the 9-argument torch op, eager, launch cost included ----------------
    op_call = time_torch_op(timer.sets, timer.n_sets, hyper, elems) if rank == 0 else None

    # ---- CPU baseline (and the parity bits of the small workloads: the oracle as checker) ----
    cpu_line = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_reference_rate(wl, seconds_budget=6.0)
        cpu_line = {"value": cpu["pooled"], "unit": "elements/s", "cores": cpu["cores"],
                    "kind": cpu["kind"], "sample": cpu["sample"], "single_thread_value": cpu["single"]}
        if small is not None:
            check_small_workloads(small)
    if small is not None:
        for row in small:
            row.pop("_got", None)

    # ---- end to end through the host-buffer C ABI ----------------------------
    e2e = None
    if args.e2e_steps > 0:
        e2e_steps = max(2, min(steps, args.e2e_steps))
        h_adv = torch.zeros((S, H)).pin_memory()
        h_abs = torch.zeros(S).pin_memory()
        lib = cabi.load()

        def host_call():
            pufferlib_b200.compute_puff_advantage_host(*host, h_adv, *hyper, seg_abs_sum=h_abs,
                                                       variant=variant, device=local_rank)

        def copies_only():
            cabi.check(lib.puff_advantage_sm100_host_copies_only(*[t.data_ptr() for t in host], h_adv.data_ptr(),
                                                                 h_abs.data_ptr(), S, H, local_rank))

        def wall(fn, n):
            for _ in range(2):
                fn()
            fence()
            w0 = time.time()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            fence()
            timer.windows.append((w0, time.time()))
            return max_over_ranks([dt], dev, world)[0]

        ceil_s = wall(copies_only, e2e_steps)      # first: it leaves garbage in h_adv, the real run overwrites it
        e2e_s = wall(host_call, e2e_steps)
        e2e = {"value": elems * world * e2e_steps / e2e_s, "unit": "elements/s",
               "h2d_bytes_per_step": 16 * elems * world,
               "d2h_bytes_per_step": (4 * S * (H - 1) + 4 * S) * world, "steps": e2e_steps,
               "ms_per_step": 1e3 * e2e_s / e2e_steps,
               "copy_ceiling_ms": 1e3 * ceil_s / e2e_steps,
               "frac_of_copy_ceiling": ceil_s / e2e_s,
               "copy_ceiling": "the same blocks, streams and bytes with no kernel between the copies "
                               "(puff_advantage_sm100_host_copies_only), all ranks at once",
               "numa": numa,
               "api": "puff_advantage_sm100_host (C ABI, pinned host buffers)"}

    clocks = sampler.stop(timer.windows) if sampler is not None else None
    final_status = cabi.device_status()
    if final_status != 0:
        timer.status_errors.append(f"{final_status}: {cabi.strerror(final_status)}")
    n_bad = max_over_ranks([len(timer.status_errors)], dev, world)[0]

    if rank == 0:
        peak, peak_kind = hbm_peak()
        achieved = BYTES_PER_ELEMENT * elems / (kernel_ms * 1e-3) / 1e9
        traffic = TRAFFIC.get((wl.name, kernel_name)) if wl.segments == WORKLOADS[wl.name].segments else None
        line = {
            "metric": "advantage elements/sec", "value": value, "unit": "elements/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_total / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": workload_config(wl, world),
            "variant": variant, "kernel": kernel_name, "exchange": exchange_kind,
            "achieved_gbs": value * BYTES_PER_ELEMENT / 1e9,
            "kernel_only": {"ms_per_launch": kernel_ms, "elements_per_s": elems * world / (kernel_ms * 1e-3),
                            "gbs_per_gpu": BYTES_PER_ELEMENT * elems / (kernel_ms * 1e-3) / 1e9},
            "timing": timing,
            "reference_cuda_kernel": ref_cuda,
            "torch_op_eager": op_call,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": None if traffic is None else traffic["read"] + traffic["write"],
                         "traffic_read": None if traffic is None else traffic["read"],
                         "traffic_write": None if traffic is None else traffic["write"],
                         "traffic_source": None if traffic is None else traffic["source"],
                         "kernel": kernel_name, "kernel_ms": kernel_ms, "peak_kind": f"of {peak_kind}",
                         "algorithmic_bytes": BYTES_PER_ELEMENT * elems},
            "e2e": e2e,
            "gpu_launches": launches,
            "clocks": clocks,
            # 0 on every rank, or this run's numbers are void: a kernel gave up a bounded wait
            "device_status": "ok" if n_bad == 0 else {"ranks_max_errors": int(n_bad), "rank0": timer.status_errors},
        }
        if strong is not None:
            line["strong_scaling"] = strong
        if small is not None:
            line["small_workloads"] = small
        if neighbours is not None:
            line["neighbour_kernels"] = neighbours
        if cpu_line is not None:
            line["cpu_baseline"] = cpu_line
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        if exchange is not None:
            exchange.close()
        dist.destroy_process_group()


# Workloads that are too small (or too odd) for the headline, measured as steady state:
# back-to-back launches rotating over buffer sets larger than 2x L2.
def small_workload_list():
    from pufferlib_b200.workloads import Workload
    return [WORKLOADS["cfg0"], WORKLOADS["cfg1"], WORKLOADS["cfg3"], WORKLOADS["cfg4"],
            # the shipped odd horizon: config/ocean/drive.ini:36-39 (745472 // 91 = 8192 segments)
            Workload("drive", 8192, 91, gamma=0.98, lam=0.95, seed=7, epilogue=True),
            # an odd horizon at the headline's scale
            Workload("odd_large", 131072, 127, seed=8, epilogue=True)]


def time_small_workloads(dev, fence):
    from pufferlib_b200 import cabi
    from pufferlib_b200.advantage import launch_raw
    peak, _ = hbm_peak()
    rows = []
    stream = torch.cuda.Stream()
    for wl in small_workload_list():
        S, H = wl.segments, wl.horizon
        hyper = wl.hyper()
        set_bytes = BYTES_PER_ELEMENT * S * H
        n_sets = rotation_sets(set_bytes)
        host = make_inputs(wl)
        first = [t.to(dev) for t in host]
        sets = [first + [torch.zeros((S, H), device=dev), torch.empty(S, device=dev)]]
        for _ in range(n_sets - 1):
            sets.append([t.clone() for t in first] + [torch.zeros((S, H), device=dev), torch.empty(S, device=dev)])

        def launch(i):
            v, r, d, w, adv, sums = sets[i % n_sets]
            launch_raw(v, r, d, w, adv, *hyper, seg_abs_sum=sums, variant=wl.variant)

        n = max(n_sets, 200)
        with torch.cuda.stream(stream):
            for i in range(min(n, 2 * n_sets)):
                launch(i)
        kernel = cabi.last_kernel()
        fence()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(n):
                launch(i)
        g.replay()
        fence()
        times = []
        for _ in range(5):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            g.replay()
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1) / n)
        us = 1e3 * statistics.median(times)
        gbs = set_bytes / (us * 1e-6) / 1e9
        rows.append({"workload": f"{wl.name}: {S}x{H}", "kernel": kernel, "variant": wl.variant,
                     "us_per_launch": us, "gbs": gbs, "frac": gbs / peak,
                     "traffic_floor_us": 1e6 * set_bytes / (peak * 1e9), "buffer_sets": n_sets,
                     "_got": (wl, sets[0][4].cpu(), sets[0][5].cpu())})
        del sets, first
    # what a launch costs before it moves a byte: an empty-handed kernel, same graph structure
    x = torch.zeros(1, device=dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for _ in range(200):
            x.add_(1.0)
    g.replay()
    fence()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    g.replay()
    t1.record()
    torch.cuda.synchronize()
    floor = 1e3 * t0.elapsed_time(t1) / 200
    for row in rows:
        row["launch_floor_us"] = floor
    return rows


def time_neighbour_kernels(dev, fence):
    """Steady-state device time of the kernels either side of the advantage op, on cfg2's
    buffer shape: the sampler prologue (priority weights + probabilities, pufferl.py:359-361),
    the minibatch gather with its normalisation (:363-375, 408-409; 8192 sampled segments)
    and the rollout writer (:275, 294-296).  Each is a CUDA graph of back-to-back calls
    through the C ABI, rotating over buffer sets that together exceed 2x L2."""
    from pufferlib_b200 import cabi
    lib = cabi.load()
    peak, _ = hbm_peak()
    S, H, M = 131072, 256, 8192
    gen = torch.Generator(device="cpu").manual_seed(11)
    stream = torch.cuda.Stream()

    def timed(launch, n):
        with torch.cuda.stream(stream):
            for i in range(min(n, 8)):
                launch(i)
        fence()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(n):
                launch(i)
        g.replay()
        fence()
        times = []
        for _ in range(5):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            g.replay()
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1) / n)
        return 1e3 * statistics.median(times)

    def st():
        return torch.cuda.current_stream().cuda_stream

    rows = []
    # --- minibatch gather + normalisation ---
    adv = torch.randn((S, H), generator=gen).to(dev)
    val = torch.randn((S, H), generator=gen).to(dev)
    probs = torch.rand(S, generator=gen).to(dev)
    probs /= probs.sum()
    n_sets = rotation_sets(7 * 4 * M * H)
    idx = [torch.randint(0, S, (M,), generator=gen).to(dev) for _ in range(n_sets)]
    outs = [[torch.empty((M, H), device=dev) for _ in range(4)] + [torch.empty(M, device=dev)] for _ in range(n_sets)]
    mb_scratch = torch.empty(lib.puff_minibatch_sm100_scratch_bytes(M) // 8 + 1, dtype=torch.float64, device=dev)

    def gather(i):
        o = outs[i % n_sets]
        cabi.check(lib.puff_minibatch_sm100_gather_ex(
            adv.data_ptr(), val.data_ptr(), probs.data_ptr(), idx[i % n_sets].data_ptr(), o[0].data_ptr(),
            o[1].data_ptr(), o[2].data_ptr(), o[3].data_ptr(), o[4].data_ptr(), 0.5, S, S, H, M,
            mb_scratch.data_ptr(), mb_scratch.numel() * 8, st()))

    us = timed(gather, max(n_sets, 100))
    mb_bytes = 7 * 4 * M * H
    rows.append({"kernels": "puff_mb_gather_kernel + puff_mb_normalize_kernel",
                 "what": f"minibatch gather + normalisation, {M} of {S} segments x {H}",
                 "us_per_call": us, "algorithmic_bytes": mb_bytes, "gbs": mb_bytes / (us * 1e-6) / 1e9,
                 "frac": mb_bytes / (us * 1e-6) / 1e9 / peak,
                 "bytes": "28 B per gathered element: 8 read + 12 written by the gather, 4 read + 4 written "
                          "by the normalisation", "buffer_sets": n_sets})
    del outs, idx

    # --- sampler prologue: weights, total, probabilities ---
    sums = torch.rand(S, generator=gen).to(dev)
    n_sets = rotation_sets(16 * S)
    n_sets = min(n_sets, 64)   # 2 MB per call: L2-resident in any trainer, so no attempt to defeat L2 beyond this
    wts = [torch.empty(S, device=dev) for _ in range(n_sets)]
    prb = [torch.empty(S, device=dev) for _ in range(n_sets)]
    total = torch.empty(1, dtype=torch.float64, device=dev)
    pr_scratch = torch.empty(lib.puff_priorities_sm100_scratch_bytes(S) // 8 + 1, dtype=torch.float64, device=dev)

    def prologue(i):
        cabi.check(lib.puff_priorities_sm100_weights(sums.data_ptr(), wts[i % n_sets].data_ptr(), total.data_ptr(), 0.6, S,
                                                     pr_scratch.data_ptr(), pr_scratch.numel() * 8, st()))
        cabi.check(lib.puff_priorities_sm100_probs(wts[i % n_sets].data_ptr(), total.data_ptr(), prb[i % n_sets].data_ptr(),
                                                   S, st()))

    us = timed(prologue, 200)
    rows.append({"kernels": "puff_prio_weights_kernel + puff_prio_total_kernel + puff_prio_probs_kernel",
                 "what": f"sampler prologue: weights, their total, probabilities over {S} segments",
                 "us_per_call": us, "algorithmic_bytes": 16 * S, "gbs": 16 * S / (us * 1e-6) / 1e9,
                 "frac": 16 * S / (us * 1e-6) / 1e9 / peak,
                 "bytes": "16 B per segment; three dependent launches, latency-bound"})

    # --- rollout writer: one environment step into one column ---
    rew, ter = torch.zeros((S, H), device=dev), torch.zeros((S, H), device=dev)
    s_r, s_v = torch.randn(S, generator=gen).to(dev), torch.randn(S, generator=gen).to(dev)
    s_d = (torch.rand(S, generator=gen) < 0.01).to(dev)

    def rollout(i):
        cabi.check(lib.puff_rollout_sm100_write(rew.data_ptr(), ter.data_ptr(), val.data_ptr(), s_r.data_ptr(),
                                                s_d.data_ptr(), s_v.data_ptr(), 0, S, i % H, S, H, 1.0, st()))

    us = timed(rollout, 256)
    ro_bytes = S * (9 + 12)
    rows.append({"kernels": "puff_rollout_write_kernel",
                 "what": f"rollout writer: one step of {S} environments into one column of three [S, {H}] buffers",
                 "us_per_call": us, "algorithmic_bytes": ro_bytes, "gbs": ro_bytes / (us * 1e-6) / 1e9,
                 "frac": ro_bytes / (us * 1e-6) / 1e9 / peak,
                 "bytes": "9 B read + 12 B written per environment; the writes are 4-byte column elements of "
                          "1 KB rows, one 32-byte sector each"})
    assert cabi.device_status() == 0
    return rows


def check_small_workloads(rows):
    """Parity bit per small workload: this run's output against the CPU oracle (bitwise for
    the serial kernels, |a-b| <= max(1e-6, 1e-5|b|) for the scan kernel)."""
    import numpy as np
    from oracle import puff_oracle
    for row in rows:
        wl, got, sums = row["_got"]
        inputs = [t.numpy() for t in make_inputs(wl)]
        want = np.zeros(inputs[0].shape, dtype=np.float32)
        puff_oracle.advantage(*inputs, want, *wl.hyper())
        got = got.numpy()
        if row["kernel"] == "scan":
            ok = bool(np.all(np.abs(got - want) <= np.maximum(1e-6, 1e-5 * np.abs(want))))
            row["parity"] = "within 1e-5 rel / 1e-6 abs of the oracle" if ok else "FAILED"
        else:
            ok = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
            row["parity"] = "bitwise equal to the oracle" if ok else "FAILED"
        exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
        row["sums_ok"] = bool(np.allclose(sums.numpy(), exact, rtol=1e-5, atol=1e-6))


def time_reference_cuda_kernel(sets, n_sets, hyper, elems):
    """The reference's cuda/pufferlib.cu (one thread per segment), compiled
    unchanged for sm_100a into oracle/_ref/, on the same buffers.  It launches
    on the legacy default stream, so it is timed eagerly with events there."""
    try:
        from oracle import puff_oracle
        ref = puff_oracle.load_reference(cuda=True)
        if ref is None or not puff_oracle.reference_has_cuda():
            return None
        n = max(20, min(200, 2 * n_sets))
        for i in range(3):
            v, r, d, w, adv = sets[i % n_sets][:5]
            ref(v, r, d, w, adv, *hyper)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            v, r, d, w, adv = sets[i % n_sets][:5]
            ref(v, r, d, w, adv, *hyper)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        return {"ms_per_launch": ms, "elements_per_s": elems / (ms * 1e-3),
                "gbs": BYTES_PER_ELEMENT * elems / (ms * 1e-3) / 1e9, "launches": n}
    except Exception as exc:   # the secondary baseline must never break the benchmark
        return {"error": str(exc)[:200]}


def time_torch_op(sets, n_sets, hyper, elems):
    """torch.ops.pufferlib.compute_puff_advantage called eagerly on device
    tensors (the call of pufferl.py:674): wall clock per call with the Python
    and dispatcher cost included, device drained before and after the loop."""
    from pufferlib_b200 import _C  # noqa: F401  (registers the op)
    op = torch.ops.pufferlib.compute_puff_advantage
    n = max(50, min(400, 4 * n_sets))
    for i in range(5):
        op(*sets[i % n_sets][:5], *hyper)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n):
        op(*sets[i % n_sets][:5], *hyper)
    issue_s = time.perf_counter() - t0
    torch.cuda.synchronize()
    wall_s = time.perf_counter() - t0
    return {"us_per_call": 1e6 * wall_s / n, "host_issue_us_per_call": 1e6 * issue_s / n,
            "elements_per_s": elems * n / wall_s, "calls": n}


def run_sequence_arm(args, wl):
    """--sequence: the trainer's per-minibatch sequence around the op
    (pufferl.py:346-375, 408-409) as the reference writes it -- eager torch
    kernels around the 9-argument op -- against the same sequence on the fused
    entry points, both eager on one GPU, same buffers, same sampled indices."""
    import pufferlib_b200
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    S, H = wl.segments, wl.horizon
    hyper = wl.hyper()
    values, rewards, terminals, ratio = [t.to(dev) for t in make_inputs(wl)]
    M = max(1, S // 16)                      # nmmo3.ini: 32768 / 64 = 512 of 8192 segments
    a, beta = PRIO_ALPHA, 0.6
    gen = torch.Generator(device=dev)

    def reference_style():
        advantages = torch.zeros((S, H), device=dev)
        pufferlib_b200.compute_puff_advantage(values, rewards, terminals, ratio, advantages, *hyper)
        adv = advantages.abs().sum(axis=1)
        prio_weights = torch.nan_to_num(adv ** a, 0, 0, 0)
        prio_probs = (prio_weights + 1e-6) / (prio_weights.sum() + 1e-6)
        idx = torch.multinomial(prio_probs, M, generator=gen)
        mb_prio = (S * prio_probs[idx, None]) ** -beta
        mb_values = values[idx]
        mb_returns = advantages[idx] + mb_values
        mb_advantages = advantages[idx]
        adv_n = mb_prio * (mb_advantages - mb_advantages.mean()) / (mb_advantages.std() + 1e-8)
        return idx, mb_values, mb_returns, adv_n

    sums = torch.empty(S, device=dev)
    advantages = torch.empty((S, H), device=dev)

    def fused():
        pufferlib_b200.compute_puff_advantage_fill(values, rewards, terminals, ratio, *hyper,
                                                   advantages=advantages, seg_abs_sum=sums)
        weights, total = pufferlib_b200.priority_weights(sums, a)
        prio_probs = pufferlib_b200.priority_probs(weights, total)
        idx = torch.multinomial(prio_probs, M, generator=gen)
        mb_values, mb_returns, _, adv_n, _ = pufferlib_b200.minibatch_gather(advantages, values, prio_probs, idx, beta)
        return idx, mb_values, mb_returns, adv_n

    # same sampled indices -> same results
    gen.manual_seed(1)
    r1 = reference_style()
    gen.manual_seed(1)
    r2 = fused()
    same_idx = bool(torch.equal(r1[0], r2[0]))
    max_err = float((r1[3] - r2[3]).abs().max()) if same_idx else None

    def timeit(fn, n):
        for _ in range(10):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / n

    n = max(20, args.steps if args.steps < 2000 else 500)
    t_ref = timeit(reference_style, n)
    t_fused = timeit(fused, n)
    print(json.dumps({
        "mode": "sequence", "workload": f"{wl.name}: {S}x{H}, minibatch {M} segments",
        "reference_style_us": 1e6 * t_ref, "fused_us": 1e6 * t_fused, "ratio": t_ref / t_fused,
        "same_sampled_indices": same_idx, "max_abs_diff_normalised_advantages": max_err,
        "what": "eager launches, wall clock per minibatch sequence (pufferl.py:352-375, 408-409); "
                "reference_style = torch.zeros + this repo's 9-argument op + the reference's eager torch lines"}), flush=True)


# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum, dram__bytes_write.sum)
# from the ncu capture summarised under profiles/ (see `source`), keyed by workload and kernel.
TRAFFIC = {
    ("cfg2", "tma2d"): {"read": 553692928, "write": 115028992,
                        "source": "profiles/tma2d_ws_kernel_cfg2_131072x256_dram_traffic.md: one full-size launch; "
                                  "about 20 MB of the 134 MB output is still dirty in L2 when the kernel ends, "
                                  "so writes read below the algorithmic 134.2 MB"},
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--variant", default="auto", choices=["auto", "serial", "scan", "generic"])
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--sequence", action="store_true",
                    help="time the trainer's per-minibatch sequence (eager reference lines vs fused entry points)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: how the weight total crosses GPUs (peer stores inside the priority kernels, "
                         "or a torch.distributed all-reduce between them)")
    ap.add_argument("--reserve-sms", type=int, default=0,
                    help="SMs the persistent advantage grid leaves free for side-stream kernels")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the strong-scaling leg")
    ap.add_argument("--no-small", action="store_true", help="N = 1: skip the small-workload table")
    ap.add_argument("--no-graph", action="store_true", help="never capture the timed loop into CUDA graphs")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip timing the reference CUDA kernel")
    ap.add_argument("--segments", type=int, default=0,
                    help="override the workload's segment count (small cases for profiler captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        args.gpus = world
    wl = WORKLOADS[args.workload]
    if args.segments > 0:
        wl = wl.with_segments(args.segments)
    if args.impl == "reference":
        run_reference_arm(args, wl, rank, world)
        return
    if args.sequence:
        run_sequence_arm(args, wl)
        return
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch with torchrun: python -m torch.distributed.run --nnodes=1 "
                         f"--nproc-per-node {args.gpus} --master-addr 127.0.0.1 bench.py --gpus {args.gpus}")
    run_b200_arm(args, wl, rank, local_rank, world)


if __name__ == "__main__":
    main()
