#!/usr/bin/env python
"""Throughput of the contraction hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one pass  C += sum A*B  of one benchmark configuration over synthetic,
seeded uniform[-1,1) inputs.  Metric: GFLOP/s per contraction (2 * prod(extents)
flops per pass), whole job.

  N = 1   workload "cfg2" (fp64, C[a,b,c,d] += sum(e) A[a,e,b,d] B[e,c], extents 96).
          The other configurations are measured briefly and listed under "configs".
  N > 1   the same "cfg2" with its slowest output index d extended to 96 N and cut into
          N contiguous slabs, one cfg2-sized slab of C per rank, no communication: per-GPU
          work is fixed, so "scaling" is "weak" and the N = 1 line is its first point.
          The partitioned configuration "cfg5" (fp64 6-D, extents 40, 32.8 GB of output,
          cut along f; total work fixed) is timed in the same run on N GPUs and on rank 0
          alone, and listed under "configs" with its parallel efficiency.

The timed region holds exactly K passes on device-resident tensors (larger than
L2), between barrier + synchronize pairs, timed with CUDA events on the stream
the kernels are launched on, max over ranks.  "e2e" is the same pass through the
host-pointer C-ABI call (allocate, copy in from pinned host memory, run, copy the
output back) -- what the reference's generated wrapper does around its kernel.

--impl reference times the reference's CPU loop-nest path (its restatement in
oracle/, OpenMP over the outermost output loop on all host cores; the reference's
own compiled nest where the workload's expression is one it ships) on a bounded
sample of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

WORKLOADS = {
    "cfg1": ("C [i,64,j,48,k,32] += sum(l,40) * A [l,k,i] * B [j,l];", "f64", 0),
    "cfg2": ("C [a,96,b,96,c,96,d,96] += sum(e,96) * A [a,e,b,d] * B [e,c];", "f64", 1),
    "cfg3": ("C [a,64,b,64,c,64,d,64] += sum(e,64,f,64) * A [e,c,a,f] * B [b,f,d,e];", "f64", 2),
    "cfg4": ("C [a,24,b,24,c,24,i,24,j,24,k,24] += sum(l,24) * A [l,a,i,j] * B [b,c,k,l];", "f32", 3),
    "cfg5": ("C [a,40,b,40,c,40,d,40,e,40,f,40] += sum(g,40) * A [g,a,b,c] * B [d,e,f,g];", "f64", 4),
    # what one GPU runs when cfg5 is cut 8 ways along f (4.1 GB of output): small enough to profile
    "cfg5_shard8": ("C [a,40,b,40,c,40,d,40,e,40,f,5] += sum(g,40) * A [g,a,b,c] * B [d,e,f,g];", "f64", 4),
}
METRIC = "GFLOP/s per contraction"
# DRAM bytes one launch of the workload's kernel moves (dram__bytes_read.sum + dram__bytes_write.sum of one
# ncu capture, summarised under profiles/); cfg5 is 8 x the captured one-eighth slab.
NCU_TRAFFIC_BYTES = {"cfg2": 1984793088, "cfg3": 1341919744, "cfg4": 1472193280,
                     "cfg5_shard8": 8369612032, "cfg5": 8 * 8369612032}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 6650.0)), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------- clocks ----
class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index, period=0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------- our arm ----
def device_tensors(pkg, torch, expr, dtype, seed, sizes):
    tdt = torch.float64 if dtype == "f64" else torch.float32
    out = []
    for tid, n in enumerate(sizes):
        t = torch.empty(n, dtype=tdt, device="cuda")
        pkg.fill_uniform(t, seed, tid)
        out.append(t)
    return out


def time_passes(torch, run, steps, warmup, sync_all=None):
    """K passes between barrier+synchronize pairs, CUDA events on the launching (current) stream."""
    for _ in range(warmup):
        run()
    if sync_all:
        sync_all()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    if sync_all:
        sync_all()
    return e0.elapsed_time(e1) * 1e-3


def quick_config(pkg, orc, torch, name, steps=5):
    expr, dtype, seed = WORKLOADS[name]
    dc, da, db = device_tensors(pkg, torch, expr, dtype, seed, orc.sizes(expr))
    plan = pkg.Plan(expr, pkg.F64 if dtype == "f64" else pkg.F32).commit()
    stream = torch.cuda.current_stream().cuda_stream
    sec = time_passes(torch, lambda: plan.execute(dc, da, db, stream=stream), steps, 3)
    flops, nbytes = plan.cost()
    d = plan.describe()
    plan.close()
    del dc, da, db
    torch.cuda.empty_cache()
    return {"workload": name, "dtype": dtype, "gflops": flops * steps / sec * 1e-9, "ms": sec / steps * 1e3,
            "algorithmic_gbs": nbytes * steps / sec * 1e-9, "kernel": d["kernel"]}


def host_threads(orc):
    """Host cores this process may use.  torchrun exports OMP_NUM_THREADS=1 to its ranks, which would make
    OpenMP report one thread; the CPU arm uses the cores the process is allowed on instead."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(n, orc.max_threads())


def weak_cfg2(world):
    """cfg2 with its slowest output index extended so that every rank owns a cfg2-sized slab."""
    return WORKLOADS["cfg2"][0].replace("d,96", "d,%d" % (96 * world))


def workload_label(name, world):
    return name if world == 1 or name != "cfg2" else "cfg2 x %d (d = 96 x %d, one cfg2-sized slab per GPU)" % (world, world)


def strong_scaling_cfg5(pkg, shard, torch, dist, rank, world, stream, steps=5):
    """cfg5 cut along its slowest output index over all ranks (max over ranks), then whole on rank 0 alone."""
    expr, dtype, seed = WORKLOADS["cfg5"]

    def timed(r, w, barrier):
        sh = shard.ExternalShard(expr, pkg.F64, r, w)
        g = sh.geom
        nc, na, nb = g.full_sizes
        dc = torch.empty(g.c_slab_elems, dtype=torch.float64, device="cuda")
        da = torch.empty(na, dtype=torch.float64, device="cuda")
        db = torch.empty(nb, dtype=torch.float64, device="cuda")
        pkg.fill_uniform(dc, seed, 0, first_index=g.offsets[0])
        pkg.fill_uniform(da, seed, 1)
        pkg.fill_uniform(db, seed, 2)
        sh.plan.commit()
        sec = time_passes(torch, lambda: sh.execute(dc, da, db, stream=stream, c_is_slab=True), steps, 3,
                          dist.barrier if barrier else None)
        sh.plan.close()
        del dc, da, db
        torch.cuda.empty_cache()
        return sec / steps

    flops = 2.0 * 40.0 ** 7
    sec_n = timed(rank, world, True)
    t = torch.tensor([sec_n], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec_n = float(t.item())
    sec_1 = timed(0, 1, False) if rank == 0 else 0.0
    dist.barrier()
    if rank != 0:
        return None
    return {"workload": "cfg5", "dtype": "f64", "scaling": "strong", "n_gpus": world,
            "sharding": "output index f cut into %d contiguous slabs, no communication" % world,
            "gflops": flops / sec_n * 1e-9, "ms": sec_n * 1e3, "ms_one_gpu": sec_1 * 1e3,
            "gflops_one_gpu": flops / sec_1 * 1e-9, "parallel_efficiency": sec_1 / (world * sec_n)}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    pkg, orc = entry.load_package(), entry.load_oracle()
    shard = __import__("importlib").import_module("cgo2019_ae_b200.shard")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world > 1:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    name = args.workload or "cfg2"
    expr, dtype, seed = WORKLOADS[name]
    if world > 1 and name == "cfg2":
        expr = weak_cfg2(world)  # one cfg2-sized slab per rank
    tdt = torch.float64 if dtype == "f64" else torch.float32
    es = 8 if dtype == "f64" else 4
    stream = torch.cuda.current_stream().cuda_stream

    # This rank's share: the whole contraction, or the slab of the slowest output index.
    plan_kw = {}
    if args.path != "auto":  # pin the arithmetic path (the profiles of non-default kernels are made this way)
        plan_kw["path"] = {"dmma": pkg.PATH_DMMA, "dfma": pkg.PATH_DFMA, "ffma": pkg.PATH_FFMA, "3xtf32": pkg.PATH_3XTF32,
                           "tcgen05": pkg.PATH_TCGEN05}[args.path]
    sh = shard.ExternalShard(expr, pkg.F64 if dtype == "f64" else pkg.F32, rank, world, **plan_kw)
    g = sh.geom
    if world > 1 and not g.c_slab_contiguous:
        raise SystemExit("workload %s cannot be cut into contiguous output slabs" % name)
    nc, na, nb = g.full_sizes
    dc = torch.empty(g.c_slab_elems, dtype=tdt, device="cuda")
    da = torch.empty(na, dtype=tdt, device="cuda")
    db = torch.empty(nb, dtype=tdt, device="cuda")
    pkg.fill_uniform(dc, seed, 0, first_index=g.offsets[0])
    pkg.fill_uniform(da, seed, 1)
    pkg.fill_uniform(db, seed, 2)
    sh.plan.commit()
    desc = sh.plan.describe()

    def one_pass():
        sh.execute(dc, da, db, stream=stream, c_is_slab=True)

    def sync_all():
        if world > 1:
            dist.barrier()

    sampler = ClockSampler(local)
    for _ in range(max(args.warmup, 3)):
        one_pass()
    torch.cuda.synchronize()
    sampler.start()
    sec = time_passes(torch, one_pass, args.steps, 0, sync_all)
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([sec], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    full_flops = 2.0 * float(np.prod([float(x) for x in g.full_extents.values()]))
    full_bytes = es * (2.0 * nc + na + nb)
    value = full_flops * args.steps / sec * 1e-9
    shard_flops, shard_bytes = sh.cost()

    # ---- end to end through the host-pointer C-ABI call (this rank's share) ----
    e2e_steps = max(1, min(args.steps, 3))
    slab_bytes = g.c_slab_elems * es

    def host_buf(n):
        try:
            return torch.empty(n, dtype=tdt, pin_memory=True)
        except Exception:
            return torch.empty(n, dtype=tdt)

    hc, ha, hb = host_buf(g.c_slab_elems), host_buf(na), host_buf(nb)
    hc.copy_(dc)
    ha.copy_(da)
    hb.copy_(db)
    torch.cuda.synchronize()
    # the host call sees full input tensors and this rank's C slab: a plan over the slab's own extents
    hplan = g.make_plan(pkg.F64 if dtype == "f64" else pkg.F32, **plan_kw)
    hviews = (hc, ha[g.offsets[1]:], hb[g.offsets[2]:])
    hplan.execute_host(*hviews)  # warm-up (also commits the plan)
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        hplan.execute_host(*hviews)
    t_e2e = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([t_e2e], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_e2e = float(t.item())
    e2e_value = full_flops * e2e_steps / t_e2e * 1e-9
    h2d = (g.c_slab_elems + (na - g.offsets[1]) + (nb - g.offsets[2])) * es
    hplan.close()
    del hc, ha, hb

    strong = None
    if world > 1 and not args.workload:
        del dc, da, db
        torch.cuda.empty_cache()
        strong = strong_scaling_cfg5(pkg, shard, torch, dist, rank, world, stream)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the (single) kernel of the pass ----
    hbm_peak, hbm_src = measured_peaks()
    pipe = "dmma_m8n8k4" if dtype == "f64" else "ffma"
    pipe_peak = pkg.measure_peaks(which=(0,) if dtype == "f64" else (5,))[pipe]
    launch_s = sec / args.steps
    t_hbm = shard_bytes / (hbm_peak * 1e9)
    t_pipe = shard_flops / (pipe_peak * 1e12)
    if t_pipe >= t_hbm:
        roof = {"bound": "tensor", "achieved": shard_flops / launch_s * 1e-12, "peak": pipe_peak, "unit": "TFLOP/s",
                "peak_source": "live register-only %s probe of this library (of measured; the driver's peak file "
                               "has no fp64/fp32 pipe figure)" % pipe}
    else:
        roof = {"bound": "hbm", "achieved": shard_bytes / launch_s * 1e-9, "peak": hbm_peak, "unit": "GB/s",
                "peak_source": "MEASURED_PEAKS.json hbm_gbs (of %s)" % hbm_src}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(name) if (world == 1 or name == "cfg2") and args.path == "auto" else None  # per launch: every rank runs a cfg2-sized slab
    roof["kernel"] = desc["kernel"]
    roof["algorithmic_bytes_per_launch"] = shard_bytes
    roof["algorithmic_flops_per_launch"] = shard_flops
    roof["hbm"] = {"achieved": shard_bytes / launch_s * 1e-9, "peak": hbm_peak, "unit": "GB/s",
                   "frac": shard_bytes / launch_s * 1e-9 / hbm_peak, "peak_source": "MEASURED_PEAKS.json (%s)" % hbm_src}

    line = {
        "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak" if name == "cfg2" or world == 1 else "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": workload_label(name, world), "expression": expr, "seed": seed,
                   "sharding": "output index %s cut into %d contiguous slabs, no communication" % (g.index, world)
                   if world > 1 else "none",
                   "l2": "inputs larger than L2 (%.0f MB touched per pass per GPU)" % (shard_bytes / 2 ** 20),
                   "plan": {k: desc[k] for k in ("kernel", "math", "tile", "tiles", "ksplit", "vec_c")}},
        "roofline": roof,
        "e2e": {"value": e2e_value, "unit": "GFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": slab_bytes,
                "steps": e2e_steps, "call": "tc_execute_host on pinned host buffers (H2D of C, A, B, kernels, D2H of C; "
                                            "slabs of the slowest output index pipelined over two streams)"},
        "gpu_launches": sh.plan.launches * args.steps,
        "clocks": clocks,
    }

    if world == 1:
        # CPU baseline beside it (bounded sample, rank 0 only).
        line["cpu_baseline"] = cpu_baseline(orc, name, budget_s=12.0)
        if not args.workload:
            del dc, da, db
            torch.cuda.empty_cache()
            line["configs"] = [quick_config(pkg, orc, torch, n) for n in ("cfg1", "cfg3", "cfg4", "cfg5")]
    if strong:
        line["configs"] = [strong]
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------ CPU loop-nest arm ----
def _sample_problem(orc, name, count):
    """The first `count` values of the slowest output index: (expr, C, A, B, strides, flops, description)."""
    import numpy as np
    expr, dtype, seed = WORKLOADS[name]
    p = orc.parse(expr)
    ext = dict(zip(p["out_idx"] + p["sum_idx"], p["out_ext"] + p["sum_ext"]))
    cut = p["out_idx"][-1]
    count = max(1, min(count, ext[cut]))
    local = dict(ext)
    local[cut] = count
    sub = orc.with_extents(expr, {cut: count})
    ndt = np.float64 if dtype == "f64" else np.float32
    tensors = (p["out_idx"], p["left_idx"], p["right_idx"])
    strides, arrays = {}, []
    for tid, idx in enumerate(tensors):
        st, acc = [], 1
        for i in idx:
            st.append(acc)
            acc *= ext[i]
        strides[tid] = st
        if cut in idx and idx[-1] != cut:
            n = acc                       # cut index is in the middle: keep the full tensor, view by strides
        else:
            n = 1
            for i in idx:
                n *= local[i]             # a prefix of the full tensor (or the tensor does not carry the index)
        arr = np.empty(n, dtype=ndt)
        orc.fill_c(arr, seed, tid)
        arrays.append(arr)
    flops = 2.0
    for v in local.values():
        flops *= v
    what = "first %d of %d values of output index %s of %s (%.3g of the pass)" % (count, ext[cut], cut, name, count / ext[cut])
    return sub, arrays, strides, flops, what, ext[cut]


def _time_sample(orc, name, count, threads):
    sub, (c, a, b), strides, flops, what, full = _sample_problem(orc, name, count)
    t0 = time.perf_counter()
    orc.contract(sub, c, a, b, threads=threads, strides=strides)
    return time.perf_counter() - t0, flops, what, full


def cpu_baseline(orc, name, budget_s):
    """GFLOP/s of the loop nest on all host threads over a sample sized for about budget_s seconds."""
    threads = host_threads(orc)
    sec, flops, what, full = _time_sample(orc, name, 1, threads)
    count = int(max(1, min(full, budget_s / max(sec, 1e-4))))
    if count > 1:
        sec, flops, what, _ = _time_sample(orc, name, count, threads)
    return {"value": flops / sec * 1e-9, "unit": "GFLOP/s", "cores": threads, "kind": "port",
            "sample": what + "; C restatement of the reference loop nest, OpenMP over the outermost output loop"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    orc = entry.load_oracle()
    try:
        orc.lib()
    except ImportError:
        entry._load_script(os.path.join(ROOT, "oracle", "build_oracle.py"), "tc_oracle_build").build_all()
    name = args.workload or "cfg2"
    expr, dtype, seed = WORKLOADS[name]
    threads = host_threads(orc)
    # size one step so that warm-up + steps stay near two minutes
    per_step = max(0.05, 110.0 / (args.steps + args.warmup))
    t1, _, _, full = _time_sample(orc, name, 1, threads)
    count = int(max(1, min(full, per_step / max(t1, 1e-4))))
    sub, (c, a, b), strides, flops, what, _ = _sample_problem(orc, name, count)
    for _ in range(args.warmup):
        orc.contract(sub, c, a, b, threads=threads, strides=strides)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.contract(sub, c, a, b, threads=threads, strides=strides)
    sec = time.perf_counter() - t0
    value = flops * args.steps / sec * 1e-9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak" if name == "cfg2" or world == 1 else "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": workload_label(name, world),
                   "expression": weak_cfg2(world) if world > 1 and name == "cfg2" else expr, "seed": seed},
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": threads, "kind": "port",
                         "sample": what + "; the reference's CPU loop nest (restated in C, bit-identical to its "
                                          "compiled drivers), OpenMP over the outermost output loop"},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--path", default="auto", choices=["auto", "dmma", "dfma", "ffma", "3xtf32", "tcgen05"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
