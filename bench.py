#!/usr/bin/env python
"""Benchmark of the Clebsch-Gordan hot path: SO3vec full CG product, forward + backward, per call.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3|cfg2|cfg1|cfg4|cfg5] [--impl reference]

Workload (default ``cfg3``, the configuration the headline target is quoted on): x and y are SO3vecs
with parts l = 0..6, 32 channels per l, batch 4096, complex64 with re/im ~ N(0,1); the product is truncated
at maxl = 6 (175 (l1,l2)->l triples); the upstream gradient is N(0,1) of the output's shape.  One step =
one forward call + one fused backward call through the C ABI (``libgelib_b200.so``), i.e. the calls the
autograd Functions of ``gelib_b200`` make.  Data is synthetic (seeded), as the reference has no dataset.

Numbers on the JSON line:
  value / ms_per_step   forward+backward milliseconds per call with every operand resident in HBM
                        (CUDA events on the launching stream, max over ranks).
  e2e                   the same step driven from pinned HOST buffers: x,y copied host->device, forward,
                        backward, the gradients copied device->host, all inside the timed region.  The 47.7 GB
                        product itself stays on the device in both numbers (it is consumed there by the next
                        layer and does not fit a host copy per step); its upstream gradient is device-resident.
  roofline              for the kernel with the largest share of the step: algorithmic bytes (write r once /
                        read g once, plus x,y,xg,yg) divided by its CUDA-event time, against the measured
                        HBM copy bandwidth of MEASURED_PEAKS.json.
  cpu_baseline          the CPU oracle (a restatement of the reference's CPU loops; the reference itself cannot
                        be compiled without its un-vendored cnine submodule) on all host threads over a slice
                        of the batch, extrapolated linearly to the full batch (cells are independent).
Multi-GPU: one process per GPU (torchrun); every rank runs the full per-GPU workload on its own shard of a
batch of N x 4096 (weak scaling); there is no collective on the data path.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (description, x type, y type, maxl, batch, diag)
    "cfg1": ("SO3part CGproduct l1=l2=l=2, 32 channels, batch 1024 (as a one-part SO3vec product, maxl=2 keeps l=0..2)",
             {2: 32}, {2: 32}, 2, 1024, False),
    "cfg2": ("SO3part l1=3 x l2=4 -> l=1..7, 64 channels, batch 4096", {3: 64}, {4: 64}, -1, 4096, False),
    "cfg3": ("SO3vec full CGproduct maxl=6, 32 channels per l, batch 4096", {l: 32 for l in range(7)},
             {l: 32 for l in range(7)}, 6, 4096, False),
    "cfg4": ("SO3vec DiagCGproduct maxl=8, 128 channels per l, batch 16384", {l: 128 for l in range(9)},
             {l: 128 for l in range(9)}, 8, 16384, True),
    "cfg5": ("spharm(1 ch) x mixed 16-channel SO3vec, maxl=6, 262144 points", {l: 1 for l in range(7)},
             {l: 16 for l in range(7)}, 6, 262144, False),
}


def band(l1, l2, l):
    return sum(max(0, min(l1, m + l2) - max(-l1, m - l2) + 1) for m in range(-l, l + 1))


def algorithmic_work(tx, ty, maxl, B, diag):
    """complex MACs and bytes of one forward and one backward call (8 bytes per complex number)."""
    macs, out = 0, {}
    for l1, n1 in tx.items():
        for l2, n2 in ty.items():
            for l in range(abs(l1 - l2), l1 + l2 + 1):
                if maxl == -1 or l <= maxl:
                    w = n1 if diag else n1 * n2
                    macs += band(l1, l2, l) * w
                    out[l] = out.get(l, 0) + w
    xin = sum((2 * l + 1) * n for l, n in tx.items()) + sum((2 * l + 1) * n for l, n in ty.items())
    rout = sum((2 * l + 1) * n for l, n in out.items())
    return {"macs": macs * B, "fwd_bytes": 8 * B * (xin + rout), "bwd_bytes": 8 * B * (rout + 2 * xin), "tau_r": out}


# DRAM traffic of one launch relative to its algorithmic bytes: dram__bytes_read + dram__bytes_write of one ncu capture
# of a batch-296 launch of the named kernel (every cell reads and writes its own rows once, so traffic grows in
# proportion to the batch and the ratio carries over).  A kernel without a capture reports traffic null.
TRAFFIC_RATIO = {
    "cg_fwd_tc_kernel": (0.98, "cfg3, batch 296, ncu 2025.2 --set full"),
    "cg_fwd_kernel": (0.98, "cfg3, batch 296, ncu 2025.2 --set full"),
    "cg_bwd_kernel": (1.002, "cfg3, batch 296, ncu 2025.2 --set full"),
    "cg_bwd_pair_kernel": (1.016, "cfg3, batch 296, ncu 2025.2 --set full"),
}


def kernel_name(args, dom):
    """Name of the kernel the roofline object describes (the slower of the step's two kernels)."""
    if args.workload == "cfg4":
        return "diag_fwd_cell_kernel" if dom == "forward" else "diag_bwd_cell_kernel"
    if args.workload == "cfg5":
        return "cg_narrow_fwd_kernel" if dom == "forward" else "cg_narrow1_bwd_kernel"
    if dom == "forward":
        tc = args.fwd_kernel == "tcgen05" or (args.fwd_kernel == "auto" and args.workload == "cfg3")
        return "cg_fwd_tc_kernel" if tc else "cg_fwd_kernel"
    if args.bwd_kernel == "tcgen05":
        return "cg_bwd_tc_kernel"
    pair = (args.bwd_kernel == "pair" and args.workload in ("cfg1", "cfg2", "cfg3")) or (
        args.bwd_kernel == "auto" and args.workload in ("cfg2", "cfg3"))   # cfg1 has 5 groups per cell: below the threshold
    return "cg_bwd_pair_kernel" if pair else "cg_bwd_kernel"


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- CPU legs -------------------------------------------------------------------------------------------------


def host_threads():
    """Host threads the CPU legs use: every core this process may run on (torchrun sets OMP_NUM_THREADS=1, which
    would otherwise silently make the OpenMP oracle single-threaded)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_fwd_bwd(O, tx, ty, maxl, Bs, diag, nthreads, reps=1):
    """One forward + back0 + back1 of the oracle on a batch slice; returns seconds per repetition."""
    import numpy as np
    rng = np.random.default_rng(1003)

    def rnd(l, n):
        return (rng.standard_normal((Bs, 2 * l + 1, n)) + 1j * rng.standard_normal((Bs, 2 * l + 1, n))).astype(np.complex64)

    x, y = {l: rnd(l, n) for l, n in tx.items()}, {l: rnd(l, n) for l, n in ty.items()}
    tr = O.cg_type(tx, ty, maxl, diag)
    r = {l: np.zeros((Bs, 2 * l + 1, n), np.complex64) for l, n in tr.items()}
    g = {l: rnd(l, n) for l, n in tr.items()}
    xg, yg = {l: np.zeros_like(v) for l, v in x.items()}, {l: np.zeros_like(v) for l, v in y.items()}
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        O.vec_cg(r, x, y, diag, nthreads)
        O.vec_cg_back0(xg, g, y, diag, nthreads)
        O.vec_cg_back1(yg, g, x, diag, nthreads)
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_baseline(tx, ty, maxl, B, diag, budget_s=15.0):
    """Two CPU legs of the oracle (a restatement of the reference's loops): all host threads (OpenMP over the batch),
    and one thread, which is the reference's default session size (include/GElibSession.hpp:30,
    python/bindings/GElib_py.cpp:43).  Both on a slice of the batch, extrapolated linearly (cells are independent)."""
    from oracle import oracle as O
    O.build()
    nt = host_threads()
    Bs = max(nt, 8)
    t = cpu_fwd_bwd(O, tx, ty, maxl, Bs, diag, nt)
    # grow the slice towards the time budget (cost is linear in the batch)
    scale = int(min(B // Bs, max(1, budget_s / 3 / max(t, 1e-4))))
    if scale > 1:
        Bs *= scale
        t = cpu_fwd_bwd(O, tx, ty, maxl, Bs, diag, nt)
    ms_full = t * 1e3 * B / Bs
    # one thread: a slice sized from the all-threads rate so that it takes a few seconds
    B1 = int(max(1, min(B, Bs * 4.0 / max(t * nt, 1e-3))))
    t1 = cpu_fwd_bwd(O, tx, ty, maxl, B1, diag, 1)
    return {"value": ms_full, "unit": "ms", "cores": nt, "kind": "port",
            "sample": "oracle (CPU restatement of the reference loops, OpenMP over the batch) on %d of %d batch rows: "
                      "%.1f ms measured, extrapolated linearly" % (Bs, B, t * 1e3),
            "single_thread_ms": t1 * 1e3 * B / B1,
            "single_thread_sample": "the same loops on 1 thread (the reference's default) on %d of %d batch rows: "
                                    "%.1f ms measured, extrapolated linearly" % (B1, B, t1 * 1e3)}


def run_reference(args, tx, ty, maxl, B, diag, desc):
    """--impl reference: the reference's CPU path for the same config, on the host cores.  GElib itself cannot be
    compiled here (its cnine submodule is not vendored), so this arm times the CPU oracle, which restates the
    reference's loops, with every host thread, each step on a bounded slice of the batch."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    nt = host_threads()
    Bs = max(nt, 8) * 4
    times = []
    for i in range(args.warmup + args.steps):
        t = cpu_fwd_bwd(O, tx, ty, maxl, Bs, diag, nt)
        if i >= args.warmup:
            times.append(t)
    ms = statistics.mean(times) * 1e3 * B / Bs
    cb = {"value": ms, "unit": "ms", "cores": nt, "kind": "port",
          "sample": "oracle on %d of %d batch rows per step, extrapolated linearly" % (Bs, B)}
    print(json.dumps({"impl": "reference", "kind": "port", "extrapolated": True, "measured_rows": Bs,
                      "measured_ms_per_step": statistics.mean(times) * 1e3, "cores": nt,
                      "metric": "cg_product_fwd_bwd_ms_per_call", "value": ms, "unit": "ms",
                      "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                      "higher_is_better": False, "scaling": "strong" if args.workload == "cfg5" else "weak",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "%s: %s; per-GPU batch %d, global batch %d" % (
                          (args.workload, desc, B // args.gpus, B) if args.workload == "cfg5"
                          else (args.workload, desc, B, B * args.gpus))},
                      "cpu_baseline": cb,
                      "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ---- GPU arm -----------------------------------------------------------------------------------------------------


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (for profiling small cases)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the extra strong-scaling region of multi-GPU runs")
    ap.add_argument("--bwd-kernel", default="auto", choices=["auto", "simt", "pair", "tcgen05"],
                    help="backward kernel for channel counts that are multiples of 32 (auto = the pair kernel)")
    ap.add_argument("--fwd-kernel", default="auto", choices=["auto", "simt", "tcgen05"],
                    help="forward kernel for channel counts that are multiples of 32")
    args = ap.parse_args()
    os.environ["GELIB_B200_BWD"] = args.bwd_kernel
    os.environ["GELIB_B200_FWD"] = args.fwd_kernel
    args.warmup = max(args.warmup, 0)
    desc, tx, ty, maxl, B, diag = WORKLOADS[args.workload]
    if args.batch:
        B = args.batch
    if args.impl == "reference":
        return run_reference(args, tx, ty, maxl, B, diag, desc)
    strong = args.workload == "cfg5"   # its points are split evenly over the ranks; every other workload is weak
    if strong:
        B = B // max(1, int(os.environ.get("WORLD_SIZE", "1")))

    import torch
    import torch.distributed as dist
    import gelib_b200
    from gelib_b200 import backend as gb

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path)")
    torch.cuda.set_device(local)
    devc = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=devc)
    gelib_b200._lib.lib()

    work = algorithmic_work(tx, ty, maxl, B, diag)
    tau_r = dict(sorted(work["tau_r"].items()))
    gen = torch.Generator(device=devc).manual_seed(1003 + rank)

    def crandn(*shape):
        return torch.view_as_complex(torch.randn(*shape, 2, device=devc, generator=gen))

    pipeline = args.workload == "cfg5"
    if pipeline:
        # The named pipeline: points on the sphere scaled by radii U(0.5,2) -> spherical harmonics l = 0..6 (1 channel)
        # -> a 16-channel SO3vec mixed by per-l complex weights N(0,1/sqrt 16) -> full CG product, maxl 6, forward and
        # backward (gradients reach v and the weights), all through the Python API of gelib_b200.  The product stage is
        # the C-ABI call pair of the other workloads.
        d = torch.randn(B, 3, 1, device=devc, generator=gen)
        X = (d / d.norm(dim=1, keepdim=True) * (0.5 + 1.5 * torch.rand(B, 1, 1, device=devc, generator=gen))).contiguous()
        xs = [X]                                                   # what travels host -> device in the e2e step
        ys = [crandn(B, 2 * l + 1, n).requires_grad_() for l, n in ty.items()]
        Wp = [(crandn(n, n) / 4.0).requires_grad_() for l, n in ty.items()]
        Wobj = gelib_b200.SO3weights(*Wp)
        gs = [crandn(B, 2 * l + 1, n) for l, n in tau_r.items()]
        rs = []
        xg, yg = [], []
        state = {}

        def st_spharm():
            state["u"] = gelib_b200.SO3vec.spharms(maxl, X)

        def st_mix():
            state["vw"] = gelib_b200.SO3vec(*[gelib_b200.SO3part(t) for t in ys]) * Wobj

        def st_forward():
            state["z"] = gelib_b200.CGproduct(state["u"], state["vw"], maxl=maxl)

        def st_backward():
            for t in ys + Wp:
                t.grad = None
            torch.autograd.backward(list(state["z"].parts.values()), grad_tensors=gs)
            state.clear()

        stages = [("spharm", st_spharm), ("mix", st_mix), ("forward", st_forward), ("backward", st_backward)]
        bwd = None
    else:
        xs = [crandn(B, 2 * l + 1, n) for l, n in tx.items()]
        ys = [crandn(B, 2 * l + 1, n) for l, n in ty.items()]
        rs = [torch.empty(B, 2 * l + 1, n, dtype=torch.complex64, device=devc) for l, n in tau_r.items()]
        gs = [crandn(B, 2 * l + 1, n) for l, n in tau_r.items()]
        xg = [torch.zeros_like(t) for t in xs]
        yg = [torch.zeros_like(t) for t in ys]
        xv, yv, rv, gv = gb.SO3vec.view(xs), gb.SO3vec.view(ys), gb.SO3vec.view(rs), gb.SO3vec.view(gs)
        xgv, ygv = gb.SO3vec.view(xg), gb.SO3vec.view(yg)
        fwd = rv.addDiagCGproduct if diag else rv.addCGproduct
        bwd = gb.SO3vec.addDiagCGproduct_back01 if diag else gb.SO3vec.addCGproduct_back01

        def st_forward():
            fwd(xv, yv, overwrite=True)

        def st_backward():
            for t in xg + yg:
                t.zero_()
            bwd(xgv, ygv, gv, xv, yv)

        stages = [("forward", st_forward), ("backward", st_backward)]

    def step():
        for _, f in stages:
            f()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()

    # ---- device-resident timing: per-step events around the forward and the backward launch
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)] for _ in range(K)]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = gb.kernel_launch_count()
    sync_all()
    t_wall = time.perf_counter()
    for k in range(K):
        ev[k][0].record()
        for i, (_, f) in enumerate(stages):
            f()
            ev[k][i + 1].record()
    sync_all()
    t_wall = time.perf_counter() - t_wall
    launches = gb.kernel_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    stage_ms = {name: sum(e[i].elapsed_time(e[i + 1]) for e in ev) / K for i, (name, _) in enumerate(stages)}
    fwd_ms, bwd_ms = stage_ms["forward"], stage_ms["backward"]
    tot_ms = ev[0][0].elapsed_time(ev[-1][-1]) / K

    # ---- end to end from pinned host buffers
    e2e_ms = None
    h2d = d2h = 0
    if not args.no_e2e and pipeline:
        # host points and host v parts in, gradients of v and of the weights out, every step
        hin = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t.detach()) for t in [X] + ys]
        hout = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in ys + Wp]
        h2d = sum(t.numel() * t.element_size() for t in hin)
        d2h = sum(t.numel() * t.element_size() for t in hout)

        def e2e_step():
            with torch.no_grad():
                for dst, h in zip([X] + ys, hin):
                    dst.copy_(h, non_blocking=True)
            step()
            for h, t in zip(hout, ys + Wp):
                h.copy_(t.grad, non_blocking=True)

        e2e_step()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            e2e_step()
        e1.record()
        sync_all()
        e2e_ms = e0.elapsed_time(e1) / K
    elif not args.no_e2e:
        hx = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in xs + ys]
        hg = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in xg + yg]
        h2d = sum(t.numel() * 8 for t in hx)
        d2h = sum(t.numel() * 8 for t in hg)

        # The step in NC batch chunks through the public API (batch slices are plain views): the copies of a chunk
        # run on their own streams beside the kernels of its neighbours, as a caller with host data would do it.
        NC = 4 if B >= 64 else 1
        bounds = [(B * c // NC, B * (c + 1) // NC) for c in range(NC)]
        s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        chunks = []
        for c0, c1 in bounds:
            sl = lambda ts: [t[c0:c1] for t in ts]
            chunks.append({
                "x": gb.SO3vec.view(sl(xs)), "y": gb.SO3vec.view(sl(ys)), "r": gb.SO3vec.view(sl(rs)), "g": gb.SO3vec.view(sl(gs)),
                "xg": gb.SO3vec.view(sl(xg)), "yg": gb.SO3vec.view(sl(yg)),
                "dev_in": sl(xs + ys), "host_in": sl(hx), "dev_out": sl(xg + yg), "host_out": sl(hg),
                "ev_in": torch.cuda.Event(), "ev_done": torch.cuda.Event()})

        def e2e_step():
            s_in.wait_stream(s_main)    # the previous step's kernels no longer read x, y
            s_out.wait_stream(s_main)
            for ch in chunks:
                with torch.cuda.stream(s_in):
                    for d, h in zip(ch["dev_in"], ch["host_in"]):
                        d.copy_(h, non_blocking=True)
                    ch["ev_in"].record(s_in)
                s_main.wait_event(ch["ev_in"])
                (ch["r"].addDiagCGproduct if diag else ch["r"].addCGproduct)(ch["x"], ch["y"], overwrite=True)
                for t in ch["dev_out"]:
                    t.zero_()
                bwd(ch["xg"], ch["yg"], ch["g"], ch["x"], ch["y"])
                ch["ev_done"].record(s_main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ch["ev_done"])
                    for h, d in zip(ch["host_out"], ch["dev_out"]):
                        h.copy_(d, non_blocking=True)
            s_main.wait_stream(s_out)   # the step ends when its gradients are on the host
            s_main.wait_stream(s_in)

        e2e_step()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            e2e_step()
        e1.record()
        sync_all()
        e2e_ms = e0.elapsed_time(e1) / K

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=devc)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    tot_ms, fwd_ms, bwd_ms = reduce_max(tot_ms), reduce_max(fwd_ms), reduce_max(bwd_ms)
    if e2e_ms is not None:
        e2e_ms = reduce_max(e2e_ms)

    # ---- the second roof: FP32 multiply-add rate measured on this device (148 SMs x 8 CTAs of 256 threads)
    probe_buf = torch.empty(148 * 8 * 256, dtype=torch.float32, device=devc)
    fp32_peak = float(gelib_b200._lib.lib().gelib_probe_fp32_tflops(probe_buf.data_ptr(), 148 * 8, 3,
                                                                    torch.cuda.current_stream().cuda_stream))

    # ---- strong scaling: the per-GPU batch of the 1-GPU run split over the ranks (extra key; `value` stays weak)
    strong_ms = None
    if world > 1 and B >= world and not args.no_strong and not pipeline:
        Bq = B // world
        sl = lambda ts: [t[:Bq] for t in ts]
        sx, sy, sr, sg, sxg, syg = (gb.SO3vec.view(sl(v)) for v in (xs, ys, rs, gs, xg, yg))
        sfwd = sr.addDiagCGproduct if diag else sr.addCGproduct

        def sstep():
            sfwd(sx, sy, overwrite=True)
            for t in xg + yg:
                t[:Bq].zero_()
            bwd(sxg, syg, sg, sx, sy)

        for _ in range(3):
            sstep()
        sync_all()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(K):
            sstep()
        s1.record()
        sync_all()
        strong_ms = reduce_max(s0.elapsed_time(s1) / K)

    if rank == 0:
        peak, peak_kind = measured_peak()
        fwd_gbs = work["fwd_bytes"] / (fwd_ms * 1e-3) / 1e9
        bwd_gbs = work["bwd_bytes"] / (bwd_ms * 1e-3) / 1e9
        dom = "forward" if fwd_ms >= bwd_ms else "backward"
        kname = kernel_name(args, dom)
        dom_ms = fwd_ms if dom == "forward" else bwd_ms
        dom_bytes = work["fwd_bytes"] if dom == "forward" else work["bwd_bytes"]
        dom_flops = (8.0 if dom == "forward" else 16.0) * work["macs"]   # 8 flops per complex MAC and product
        flops = 24.0 * work["macs"]
        # both roofs of the dominant kernel; the binding one is the slower
        hbm_ms = dom_bytes / (peak * 1e9) * 1e3
        fp32_ms = dom_flops / (fp32_peak * 1e12) * 1e3 if fp32_peak > 0 else None
        fp32_binds = fp32_ms is not None and fp32_ms > hbm_ms
        tr = TRAFFIC_RATIO.get(kname) if args.workload == "cfg3" else None
        roof = {"bound": "fp32" if fp32_binds else "hbm", "kernel": kname}
        if fp32_binds:
            ach = dom_flops / (dom_ms * 1e-3) / 1e12
            roof.update({"achieved": ach, "peak": fp32_peak, "unit": "TFLOP/s", "frac": ach / fp32_peak,
                         "peak_kind": "measured in this run (FFMA probe kernel)"})
        else:
            ach = dom_bytes / (dom_ms * 1e-3) / 1e9
            roof.update({"achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_kind": peak_kind})
        roof.update({
            "traffic": tr[0] * dom_bytes if tr else None,
            "traffic_source": ("%s of %s" % (tr[1], kname)) if tr else None,
            "algorithmic_bytes_per_launch": dom_bytes, "algorithmic_flops_per_launch": dom_flops,
            "hbm_ms": hbm_ms, "fp32_ms": fp32_ms, "hbm_peak_gbs": peak, "hbm_peak_kind": peak_kind,
            "fp32_peak_tflops": fp32_peak, "hbm_frac": dom_bytes / (dom_ms * 1e-3) / 1e9 / peak,
            "fwd": {"ms": fwd_ms, "GBps": fwd_gbs, "frac": fwd_gbs / peak},
            "bwd": {"ms": bwd_ms, "GBps": bwd_gbs, "frac": bwd_gbs / peak},
            "fwd_bwd_frac_of_hbm_roofline": (work["fwd_bytes"] + work["bwd_bytes"]) / 1e9 / peak / (tot_ms * 1e-3),
            "fp32_tflops": flops / (tot_ms * 1e-3) / 1e12})
        out = {
            "metric": "cg_product_fwd_bwd_ms_per_call", "value": tot_ms, "unit": "ms", "n_gpus": world, "steps": K,
            "warmup": args.warmup, "ms_per_step": tot_ms, "higher_is_better": False,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s: %s; per-GPU batch %d, global batch %d" % (args.workload, desc, B, B * world),
                       "l2": "operands larger than L2 (output and upstream gradient %.1f GB each per GPU)"
                             % (work["fwd_bytes"] / 1e9),
                       "parallelism": "batch sharded over %d GPU(s), no collective on the data path" % world,
                       "fwd_kernel": args.fwd_kernel, "bwd_kernel": args.bwd_kernel},
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "stages_ms": stage_ms,
            "cells_per_s": B * world / (tot_ms * 1e-3),
            "roofline": roof,
            "gpu_launches": launches,
            "clocks": clocks,
            "wall_ms_per_step": t_wall * 1e3 / K,
        }
        if strong_ms is not None:
            out["strong_scaling"] = {"global_batch": B, "ms_per_step": strong_ms,
                                     "efficiency": tot_ms / (world * strong_ms),
                                     "note": "fixed global batch %d split over %d ranks; efficiency = t(1 GPU, this run's "
                                             "per-rank weak step) / (N x t_N)" % (B, world)}
        if e2e_ms is not None:
            out["e2e"] = {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(tx, ty, maxl, B, diag)
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
