"""Phase timeline of the advantage kernels on a GPU (a tracing aid, not a benchmark).

    python -m pufferlib_b200.timeline cfg2            # warp-specialised tma2d kernel: where its warps' cycles go
    python -m pufferlib_b200.timeline cfg4            # one-stage bulk1d kernel: per-CTA phase stamps
    PUFF_ADV_WS=0 python -m pufferlib_b200.timeline cfg1   # single-warp tma2d kernel: per-CTA phase stamps
    python -m pufferlib_b200.timeline odd_large       # warp-specialised bulk1d kernel, 131072 x 127

Builds the kernel library with -DPUFF_TIMELINE into a scratch folder (the
release library is not touched), runs the workload's kernel back to back from a
CUDA graph, and reads the stamps back through puff_advantage_sm100_timeline:

* single-warp tma2d / one-stage bulk1d kernels: clock64 at the phase boundaries
  of every CTA's first tile, turned into nanoseconds relative to the earliest
  CTA start of the last launch through %globaltimer anchors at each CTA's first
  and last stamp; shown as min / median / max over the CTAs;
* warp-specialised kernels: clock64 totals of the loop phases of the chain warp,
  one terms warp (and, for bulk1d, the producer), per work item (a 32 x 32
  chunk for tma2d, a tile for bulk1d).

The instrumented kernels run a few percent slower than the release build.
"""
import ctypes
import os
import sys
import tempfile

import numpy as np
import torch

from . import build, cabi
from .workloads import WORKLOADS, Workload, make_inputs

SLOTS = 16
EXTRA = {"drive": Workload("drive", 8192, 91, gamma=0.98, lam=0.95, seed=7),
         "odd_large": Workload("odd_large", 131072, 127, seed=8)}

PHASES = {
    "tma2d": ["CTA start", "set-up done", "predecessor complete (pdl_wait)", "first loads issued",
              "item 0: data arrived", "item 0: computed", "item 0: store issued",
              "item 1: data arrived", "item 1: computed", "item 1: store issued", "stores left shared memory"],
    "bulk1d": ["CTA start", "set-up done", "predecessor complete (pdl_wait)", "tile 0: thread 0 has the data",
               "tile 0: every thread has the data", "tile 0: terms in registers", "tile 0: (delta, k) pairs in shared memory",
               "tile 0: chain done, bulk store issued", None, None, "CTA end"],
}


def build_timeline_library(folder):
    path = os.path.join(folder, "libpuff_advantage_sm100_timeline.so")
    sources = [os.path.join(build.CSRC, s) for s in build.CU_SOURCES]
    build._run([build.NVCC] + build.NVCC_FLAGS + ["-DPUFF_TIMELINE", "-o", path] + sources, False)
    lib = ctypes.CDLL(path)
    for name, (res, args) in cabi.SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    lib.puff_advantage_sm100_timeline.restype = ctypes.c_int
    lib.puff_advantage_sm100_timeline.argtypes = [ctypes.c_void_p, ctypes.c_int]
    return lib


def run(name, launches=50):
    wl = WORKLOADS.get(name) or EXTRA[name]
    dev = torch.device("cuda", torch.cuda.current_device())
    S, H = wl.segments, wl.horizon
    with tempfile.TemporaryDirectory() as folder:
        lib = build_timeline_library(folder)
        set_bytes = 20 * S * H
        n_sets = 1 if set_bytes >= 252 << 20 else -(-(252 << 20) // set_bytes)
        first = [t.to(dev) for t in make_inputs(wl)]
        sets = [first + [torch.zeros((S, H), device=dev), torch.empty(S, device=dev)]]
        for _ in range(n_sets - 1):
            sets.append([t.clone() for t in first] + [torch.zeros((S, H), device=dev), torch.empty(S, device=dev)])
        stream = torch.cuda.Stream()
        variant = cabi.VARIANTS[wl.variant]

        def launch(i):
            v, r, d, w, adv, sums = sets[i % n_sets]
            rc = lib.puff_advantage_sm100_launch(v.data_ptr(), r.data_ptr(), d.data_ptr(), w.data_ptr(), adv.data_ptr(),
                                                 sums.data_ptr(), *wl.hyper(), S, H, variant,
                                                 torch.cuda.current_stream().cuda_stream)
            assert rc == 0, rc

        n = max(n_sets, launches)
        with torch.cuda.stream(stream):
            for i in range(min(n, n_sets + 3)):
                launch(i)
        kernel = cabi.KERNEL_NAMES[lib.puff_advantage_sm100_last_kernel()]
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(n):
                launch(i)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        print(f"{wl.name}: {S} x {H}, kernel {kernel}, {1e3 * a.elapsed_time(b) / n:.2f} us per launch "
              f"(instrumented build, {n} launches from one graph)")
        ctas = 2048
        buf = (ctypes.c_ulonglong * (SLOTS * ctas))()
        assert lib.puff_advantage_sm100_timeline(buf, ctas) == 0
        t = np.array(buf, dtype=np.int64).reshape(ctas, SLOTS)
        t = t[(t != 0).any(axis=1)]
        # slot 8 holds an item count in the warp-specialised tma2d kernel and a clock64 stamp otherwise
        ws = kernel == "tma2d" and len(t) > 0 and 0 < np.median(t[:, 8]) < 1e7
        if ws:
            t = t[t[:, 8] > 0]
            items = t[:, 8].astype(np.float64)
            print(f"warp-specialised kernel, {len(t)} CTAs, {np.median(items):.0f} work items (32 x 32 chunks) per CTA; "
                  "cycles per item, median over CTAs:")
            for slot, what in ((4, "chain warp: waiting for terms"), (5, "chain warp: loading terms, issuing the previous store"),
                               (6, "chain warp: the recurrence"), (7, "chain warp: writing the output box"),
                               (9, "terms warp: waiting (data, free buffer)"), (10, "terms warp: working")):
                print(f"  {what:55s} {np.median(t[:, slot] / items):8.1f}")
            return
        if kernel == "bulk1d" and len(t) > 0 and 0 < np.median(t[:, 1]) < 1e9 and t[:, 10].max() == 0:
            # warp-specialised bulk1d: slot 1 holds a tile count, the rest clock64 totals
            tiles = t[:, 1].astype(np.float64)
            print(f"warp-specialised bulk1d kernel, {len(t)} CTAs, {np.median(tiles):.0f} tiles per CTA; "
                  "cycles per tile, median over CTAs (a chain warp takes every other tile):")
            for slot, what in ((0, "producer: waiting for a free stage"), (2, "terms warp: waiting for data"),
                               (4, "terms warp: waiting for a free terms buffer"), (3, "terms warp: computing terms"),
                               (6, "chain warp 0: waiting for terms"), (7, "chain warp 0: chaining, storing")):
                print(f"  {what:55s} {np.median(t[:, slot] / tiles):8.1f}")
            return
        names = PHASES.get(kernel)
        if names is None:
            print("no timeline stamps in this kernel")
            return
        t = t[(t[:, 10] > 0) & (t[:, 12] > 0) & (t[:, 14] > t[:, 12])]
        if len(t) == 0:
            print("this kernel form carries no timeline stamps")
            return
        # stamps are clock64 values; slots 12 and 14 hold %globaltimer at the first and the last stamp
        ghz = (t[:, 10] - t[:, 0]) / (t[:, 14] - t[:, 12]).astype(np.float64)
        t0 = t[:, 12].min()
        print(f"{len(t)} CTAs stamped, SM clock {1e3 * np.median(ghz):.0f} MHz; ns after the earliest CTA start "
              "(min / median / max over CTAs):")
        if kernel == "bulk1d":
            print(f"chain loop of the first tile: median {np.median(t[:, 8]):.0f} cycles for {H - 1} steps "
                  f"({np.median(t[:, 8]) / max(H - 1, 1):.1f} per step)")
        for i, nm in enumerate(names):
            if nm is None:
                continue
            ok = t[:, i] > 0
            if ok.any():
                col = (t[ok, 12] - t0) + (t[ok, i] - t[ok, 0]) / ghz[ok]
                print(f"  {nm:45s} {col.min():7.0f} {np.median(col):7.0f} {col.max():7.0f}")


if __name__ == "__main__":
    run(sys.argv[1] if len(sys.argv) > 1 else "cfg1")
