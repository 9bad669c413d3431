#!/usr/bin/env python
"""Throughput of the contraction hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--path P]

One step = one pass  C += sum A*B  of one benchmark configuration over synthetic,
seeded uniform[-1,1) inputs.  Metric: GFLOP/s per contraction (2 * prod(extents)
flops per pass), whole job.

Headline workload at every N: "cfg5", the partitioned configuration (fp64 6-D,
C[a,b,c,d,e,f] += sum(g) A[g,a,b,c] B[d,e,f,g], extents 40, 32.8 GB of output).  Its
slowest output index f is cut into N contiguous slabs, one per rank, with no
communication; the total work is fixed, so "scaling" is "strong" and N = 1 runs the
whole problem on one GPU.  At N = 1 the other configurations are measured briefly and
listed under "configs" (configuration 4 on both of its arithmetic paths, and the
reference generator's own kernels compiled for sm_100 where they were built); at N > 1
"configs" holds a contraction-split case (K cut across ranks, one NCCL reduce-scatter).

The timed region holds exactly K passes on device-resident tensors (larger than
L2), between barrier + synchronize pairs, timed with CUDA events on the stream
the kernels are launched on, max over ranks.  After it every rank restores its slab
of C, runs one pass and compares a slab and sampled coordinates with the CPU
checker ("parity").  "e2e" is the same pass through the host-pointer C-ABI call
(copy in from page-locked host memory, run, copy the output back) -- what the
reference's generated wrapper does around its kernel; "e2e_pageable" is that call on
plain malloc memory (what the reference's drivers pass) on configuration 2.

--workload tccg (N = 1) times the reference's own benchmark list at its own sizes
(read from baseline/_ref/tccg_items.json, made by baseline/make_tccg_table.py).
--workload fused (N = 1) runs nine contractions that share one output as one fused pass
and one by one.

--impl reference times the reference's CPU loop-nest path (its restatement in
oracle/, OpenMP over the outermost output loop on all host cores) on a bounded
sample of the same workload.
"""
import argparse
import ctypes
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
    # small cases that run the kernels the five configurations do not reach (one CTA per tile, K slices + combine)
    "kslices_f64": ("C [a,320,b,288] += sum(c,256,d,320) * A [a,c,d] * B [d,b,c];", "f64", 6),
    "gemm_f32": ("C [a,4096,b,4096] += sum(c,2048) * A [c,a] * B [c,b];", "f32", 8),
    "small_f32": ("C [a,48,b,40,c,36] += sum(d,64) * A [d,c,a] * B [b,d];", "f32", 7),
}
# contraction-split case for N > 1: small output, one long contraction index cut across the ranks
KSPLIT_CASE = ("C [a,312,b,296] += sum(c,4096,d,312) * A [a,c,d] * B [d,b,c];", "f64", 13)
METRIC = "GFLOP/s per contraction"
TOL = {"f64": 1e-12, "f32": 1e-5}
# DRAM bytes one launch moves (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture, summarised under
# profiles/), keyed by the KERNEL that was captured and the workload: a plan that picks another kernel reports null.
# cfg5 is 8 x the captured one-eighth slab (traffic is proportional to the number of f values).
NCU_TRAFFIC_BYTES = {
    ("dmma_ws_64x96", "cfg2"): 1984793088, ("dmma_ws_128x64", "cfg3"): 1341919744, ("tf32tc_96x128", "cfg4"): 1472193280, ("tf32wt_96x128", "cfg4"): 1475021824,
    ("dmma_ws_128x64", "cfg5_shard8"): 8369612032, ("dmma_ws_128x64", "cfg5"): 8 * 8369612032,
    ("dmma_wc_128x64", "cfg5_shard8"): 8197418496, ("dmma_wc_128x64", "cfg5"): 8 * 8197418496,
}


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


# ------------------------------------------------------------- helpers ----
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


def path_code(pkg, name):
    return {"auto": pkg.PATH_AUTO, "dmma": pkg.PATH_DMMA, "dfma": pkg.PATH_DFMA, "ffma": pkg.PATH_FFMA,
            "3xtf32": pkg.PATH_3XTF32, "tcgen05": pkg.PATH_TCGEN05}[name]


class PinnedArray:
    """A numpy array whose pages are locked with cudaHostRegister (exact size; torch's pinned allocator would round
    a 33 GB request up to the next power of two)."""

    def __init__(self, torch, n, ndt):
        import numpy as np
        self.torch = torch
        self.arr = np.empty(n, dtype=ndt)
        self.arr[:: max(1, 4096 // self.arr.itemsize)] = 0  # touch every page before locking it
        rc = torch.cuda.cudart().cudaHostRegister(self.arr.ctypes.data, self.arr.nbytes, 0)
        self.pinned = int(rc) == 0

    def release(self):
        if self.pinned:
            self.torch.cuda.cudart().cudaHostUnregister(self.arr.ctypes.data)
            self.pinned = False


def parity_check(pkg, orc, torch, sh, dc, da, db, dtype, seed, stream, samples=100000):
    """This rank's slab of C is restored to its seeded start, one pass runs, and a slab (the rank's first value of
    every output index but the three fastest) plus `samples` sampled coordinates are compared with the CPU checker.
    The checker is used here as a checker only, outside every timed region."""
    import numpy as np
    g = sh.geom
    ndt = np.float64 if dtype == "f64" else np.float32
    p = g.parsed
    full = g.full_extents
    pkg.fill_uniform(dc, seed, 0, first_index=g.offsets[0])
    sh.execute(dc, da, db, stream=stream, c_is_slab=True)
    torch.cuda.synchronize()
    if sh.plan.status() != 0:
        return {"max_rel_err": None, "checked_elements": 0, "error": "a bounded device wait gave up"}
    nc, na, nb = g.full_sizes
    a, b = orc.uniform(seed, 1, na, ndt), orc.uniform(seed, 2, nb, ndt)
    out_idx = p["out_idx"]
    strides = {}
    for t, idx in enumerate((out_idx, p["left_idx"], p["right_idx"])):
        s, acc = [], 1
        for i in idx:
            s.append(acc)
            acc *= full[i]
        strides[t] = s
    worst, checked = 0.0, 0
    # (1) a slab: the slower output indices fixed (the cut index at this rank's first and last value)
    fast = out_idx[:3]
    for which in (0, 1):
        fix = {i: (0 if which == 0 else full[i] - 1) for i in out_idx[3:]}
        fix[g.index] = g.start if which == 0 else g.start + g.count - 1
        sub = orc.with_extents(g.full_expr, {i: 1 for i in fix})
        off = lambda idx, st: sum(fix.get(i, 0) * s for i, s in zip(idx, st))
        oc = off(out_idx, strides[0])
        span = 1 + sum((1 if i in fix else full[i]) * s - s for i, s in zip(out_idx, strides[0]))
        ref = orc.uniform(seed, 0, span, ndt, first=oc)
        init = ref.copy()
        orc.contract(sub, ref, a[off(p["left_idx"], strides[1]):], b[off(p["right_idx"], strides[2]):],
                     threads=host_threads(orc), strides=strides)
        got = dc[oc - g.offsets[0]: oc - g.offsets[0] + span].cpu().numpy()
        m = ref != init
        worst = max(worst, orc.rel_error(got[m], ref[m]))
        checked += int(m.sum())
    # (2) sampled coordinates of the rank's slab
    rng = np.random.default_rng(1000 + g.rank)
    lin = np.sort(rng.integers(0, g.c_slab_elems, size=samples, dtype=np.int64)) + g.offsets[0]
    coord, r = {}, lin.copy()
    for i in out_idx:
        coord[i] = r % full[i]
        r //= full[i]
    ref = orc.uniform_at(seed, 0, lin, ndt).astype(np.float64)
    sign = -1.0 if p["op"] == "-=" else 1.0
    ks = [full[i] for i in p["sum_idx"]]

    def offsets(idx, fixed):
        off, acc = np.zeros(samples, dtype=np.int64), 1
        for i in idx:
            off = off + (coord[i] if i in coord else fixed[i]) * acc
            acc *= full[i]
        return off

    for flat in range(int(np.prod(ks))):
        fixed, q = {}, flat
        for i, e in zip(p["sum_idx"], ks):
            fixed[i] = q % e
            q //= e
        ref += sign * a[offsets(p["left_idx"], fixed)].astype(np.float64) * b[offsets(p["right_idx"], fixed)].astype(np.float64)
    got = dc[torch.from_numpy(lin - g.offsets[0]).cuda()].cpu().numpy().astype(np.float64)
    worst = max(worst, float(np.max(np.abs(got - ref)) / np.max(np.abs(ref))))
    checked += samples
    return {"max_rel_err": worst, "checked_elements": checked, "tolerance": TOL[dtype],
            "ok": bool(worst <= TOL[dtype])}


def cogent_kernel_gflops(name, orc, flops, reps=3):
    """The reference generator's own kernel for this configuration, compiled for sm_100 by
    baseline/build_cogent_kernels.py: kernel-only time through its emitted host wrapper."""
    import numpy as np
    table_path = os.path.join(ROOT, "baseline", "_ref", "cogent_kernels.json")
    if not os.path.exists(table_path):
        return None
    info = json.load(open(table_path)).get(name)
    if not info or "lib" not in info:
        return None
    lib_path = os.path.join(ROOT, "baseline", "_ref", info["lib"])
    if not os.path.exists(lib_path):
        return None
    h = ctypes.CDLL(lib_path)
    h.cogent_last_kernel_ms.restype = ctypes.c_float
    ndt = np.float64 if info["dtype"] == "f64" else np.float32
    expr, _, seed = WORKLOADS[name]
    nc, na, nb = orc.sizes(expr)
    a, b = orc.uniform(seed, 1, na, ndt), orc.uniform(seed, 2, nb, ndt)
    c = np.zeros(nc, dtype=ndt)  # its kernel overwrites the output
    n = len(info["sizes"])
    h.sd_t_d2_fusion_.restype = None
    h.sd_t_d2_fusion_.argtypes = [ctypes.c_int] * n + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 2
    best = None
    for _ in range(reps):
        h.sd_t_d2_fusion_(*info["sizes"], c.ctypes.data, a.ctypes.data, b.ctypes.data, 1, -1)
        ms = float(h.cogent_last_kernel_ms())
        if ms > 0 and (best is None or ms < best):
            best = ms
    if best is None or h.cogent_last_error() != 0:
        return None
    return {"cogent_sm100_gflops": flops / best * 1e-6, "cogent_sm100_ms": best,
            "cogent_note": "the reference generator's emitted kernel for this expression, compiled unchanged with "
                           "-arch=sm_100; kernel-only time (CUDA events), best of %d" % reps}


def quick_config(pkg, orc, torch, name, steps=5, path="auto", cogent=False, label=None, **plan_kw):
    expr, dtype, seed = WORKLOADS[name]
    dc, da, db = device_tensors(pkg, torch, expr, dtype, seed, orc.sizes(expr))
    plan = pkg.Plan(expr, pkg.F64 if dtype == "f64" else pkg.F32, path=path_code(pkg, path), **plan_kw).commit()
    stream = torch.cuda.current_stream().cuda_stream
    sec = time_passes(torch, lambda: plan.execute(dc, da, db, stream=stream), steps, 3)
    status = plan.status()
    flops, nbytes = plan.cost()
    d = plan.describe()
    plan.close()
    del dc, da, db
    torch.cuda.empty_cache()
    row = {"workload": name, "dtype": dtype, "path": label or path, "gflops": flops * steps / sec * 1e-9, "ms": sec / steps * 1e3,
           "algorithmic_gbs": nbytes * steps / sec * 1e-9, "kernel": d["kernel"], "device_status": status}
    if cogent:
        extra = cogent_kernel_gflops(name, orc, flops)
        if extra:
            row.update(extra)
    return row


def host_threads(orc):
    """Host cores this process may use.  torchrun exports OMP_NUM_THREADS=1 to its ranks, which would make
    OpenMP report one thread; the CPU arm uses the cores the process is allowed on instead."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(n, orc.max_threads())


def config_of(name, expr, seed, index, world, shard_bytes):
    """The `config` object: identical in both arms (it names the workload, not the implementation)."""
    return {"workload": name, "expression": expr, "seed": seed,
            "sharding": ("output index %s cut into %d contiguous slabs, no communication" % (index, world)) if world > 1 else "none",
            "l2": "inputs larger than L2 (%.0f MB touched per pass per GPU)" % (shard_bytes / 2 ** 20)}


def shard_bytes_of(name, world):
    """Algorithmic bytes one rank touches per pass (for the config's L2 note; needs no GPU)."""
    expr, dtype, _ = WORKLOADS[name]
    es = 8 if dtype == "f64" else 4
    import re
    tok = expr.replace("[", "").replace("]", "").replace(";", "").split()
    out = tok[1].split(",")
    ext = dict(zip(out[0::2], (int(x) for x in out[1::2])))
    sm = tok[3][4:-1].split(",")
    ext.update(zip(sm[0::2], (int(x) for x in sm[1::2])))
    cut = max(out[0::2], key=lambda i: (ext[i], out.index(i)))
    local = dict(ext)
    local[cut] = max(1, -(-ext[cut] // world))
    n = lambda idx: __import__("math").prod(local[i] for i in idx.split(","))
    return es * (2 * n(",".join(out[0::2])) + n(tok[6]) + n(tok[9])), cut


# ------------------------------------------------------------- our arm ----
def ksplit_case(pkg, orc, shard, torch, dist, rank, world, stream, steps=5):
    """A long contraction index cut across the ranks: partial outputs, one NCCL reduce-scatter, add into C."""
    import numpy as np
    expr, dtype, seed = KSPLIT_CASE
    sh = shard.ContractionShard(expr, pkg.F64, rank, world)
    g = sh.geom
    nc, na, nb = g.full_sizes
    dc = torch.empty(nc, dtype=torch.float64, device="cuda")
    da = torch.empty(na, dtype=torch.float64, device="cuda")
    db = torch.empty(nb, dtype=torch.float64, device="cuda")
    for t, tid in ((dc, 0), (da, 1), (db, 2)):
        pkg.fill_uniform(t, seed, tid)
    sh.execute(dc, da, db, stream=stream)  # commits, allocates the partial buffer, warms NCCL up
    sh.execute(dc, da, db, stream=stream)
    pkg.fill_uniform(dc, seed, 0)
    torch.cuda.synchronize()
    dist.barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    t_comp = t_rs = t_add = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ev[0].record()
        sh.plan.execute(sh._partial, da[g.offsets[1]:], db[g.offsets[2]:], stream=stream)
        ev[1].record()
        dist.reduce_scatter_tensor(sh._reduced, sh._partial, op=dist.ReduceOp.SUM)
        ev[2].record()
        lo, hi = sh.chunk_range()
        if hi > lo:
            pkg.axpy(dc[lo:hi], sh._reduced[:hi - lo], sh.sign, stream=stream)
        ev[3].record()
        torch.cuda.synchronize()
        t_comp += ev[0].elapsed_time(ev[1])
        t_rs += ev[1].elapsed_time(ev[2])
        t_add += ev[2].elapsed_time(ev[3])
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1), t_comp, t_rs, t_add], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total, t_comp, t_rs, t_add = (float(x) / steps for x in t.tolist())
    # parity: sampled elements of this rank's chunk, recomputed from the seeded inputs (steps passes were added)
    lo, hi = sh.chunk_range()
    err = 0.0
    if hi > lo:
        p = g.parsed
        full = g.full_extents
        rng = np.random.default_rng(50 + rank)
        lin = rng.integers(lo, hi, size=8, dtype=np.int64)
        got = dc[torch.from_numpy(lin).cuda()].cpu().numpy()
        ks = [full[i] for i in p["sum_idx"]]
        kk = np.arange(int(np.prod(ks)), dtype=np.int64)
        kc, r = {}, kk.copy()
        for i, e in zip(p["sum_idx"], ks):
            kc[i] = r % e
            r //= e
        for j, l in enumerate(lin):
            oc, r = {}, int(l)
            for i in p["out_idx"]:
                oc[i] = r % full[i]
                r //= full[i]

            def offs(idx):
                off, acc = np.zeros(kk.size, dtype=np.int64), 1
                for i in idx:
                    off = off + (kc[i] if i in kc else oc[i]) * acc
                    acc *= full[i]
                return off
            s = float(np.dot(orc.uniform_at(seed, 1, offs(p["left_idx"])), orc.uniform_at(seed, 2, offs(p["right_idx"]))))
            ref = float(orc.uniform_at(seed, 0, np.array([l]))[0]) + steps * s
            err = max(err, abs(got[j] - ref) / max(1.0, abs(ref)))
    t = torch.tensor([err], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    err = float(t.item())
    sh.close()
    del dc, da, db
    torch.cuda.empty_cache()
    flops = 2.0 * float(np.prod([float(v) for v in g.full_extents.values()]))
    rs_bytes = sh.padded * 8 * (world - 1) / world  # bytes each rank sends (and receives) in the reduce-scatter
    return {"workload": "contraction split", "expression": expr, "dtype": dtype, "n_gpus": world,
            "sharding": "contraction index %s cut into %d ranges; partial outputs combined by one NCCL reduce-scatter" % (g.index, world),
            "gflops": flops / (total * 1e-3) * 1e-9, "ms": total, "ms_compute": t_comp, "ms_reduce_scatter": t_rs, "ms_add": t_add,
            "reduce_scatter_bus_gbs": rs_bytes / (t_rs * 1e-3) * 1e-9 if t_rs > 0 else None,
            "nvlink_peer_gbs_measured": 770.0,
            "note": "the exchange moves %.2f MB per rank: latency-bound, far below link bandwidth" % (rs_bytes / 2 ** 20),
            "parity": {"max_rel_err": err, "checked_elements": 8 * world, "tolerance": 1e-12, "ok": bool(err <= 1e-12)}}


def e2e_pageable_cfg2(pkg, orc, torch):
    """Configuration 2 through the host-pointer entry on pageable (plain malloc / numpy) and on page-locked buffers."""
    import numpy as np
    expr, dtype, seed = WORKLOADS["cfg2"]
    nc, na, nb = orc.sizes(expr)
    dev = device_tensors(pkg, torch, expr, dtype, seed, (nc, na, nb))
    out = {}
    flops = None
    for kind in ("pageable", "pinned"):
        bufs = []
        for t in dev:
            if kind == "pinned":
                pa = PinnedArray(torch, t.numel(), np.float64)
                bufs.append(pa)
                torch.from_numpy(pa.arr).copy_(t)
            else:
                bufs.append(t.cpu().numpy())
        arrs = [x.arr if isinstance(x, PinnedArray) else x for x in bufs]
        plan = pkg.Plan(expr, pkg.F64)
        flops = plan.cost()[0]
        plan.execute_host(*arrs)  # warm-up: commits, allocates device buffers and bounce buffers
        t0 = time.perf_counter()
        for _ in range(2):
            plan.execute_host(*arrs)
        sec = (time.perf_counter() - t0) / 2
        plan.close()
        for x in bufs:
            if isinstance(x, PinnedArray):
                x.release()
        out[kind] = {"gflops": flops / sec * 1e-9, "ms": sec * 1e3}
    del dev
    torch.cuda.empty_cache()
    return {"value": out["pageable"]["gflops"], "unit": "GFLOP/s", "workload": "cfg2", "ms": out["pageable"]["ms"],
            "pinned_same_workload": out["pinned"],
            "h2d_bytes_per_step": (nc + na + nb) * 8, "d2h_bytes_per_step": nc * 8,
            "call": "tc_execute_host on pageable host memory (what the reference's drivers pass, malloc): staged through "
                    "plan-owned page-locked bounce buffers, slabs pipelined over two streams"}


def run_tccg(args):
    """The reference's benchmark list at its own sizes (one GPU)."""
    import torch
    pkg, orc = entry.load_package(), entry.load_oracle()
    path = os.path.join(ROOT, "baseline", "_ref", "tccg_items.json")
    if not os.path.exists(path):
        print(json.dumps({"workload": "tccg", "unavailable": "baseline/_ref/tccg_items.json not built (needs the reference tree)"}))
        return
    items = json.load(open(path))
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    hbm_peak, _ = measured_peaks()
    peaks = pkg.measure_peaks(which=(0, 5))
    rows = []
    for it in items:
        dtype = it["dtype"]
        plan = pkg.Plan(it["line"], pkg.F64 if dtype == "f64" else pkg.F32, extents=it["extents"]).commit()
        d = plan.describe()
        n = lambda idx: __import__("math").prod(it["extents"][i] for i in idx)
        sizes = (n(d["expr"]["out_idx"]), n(d["expr"]["left_idx"]), n(d["expr"]["right_idx"]))
        dc, da, db = device_tensors(pkg, torch, it["line"], dtype, 7, sizes)
        reps = 20 if d["flops"] < 5e10 else 5
        sec = time_passes(torch, lambda: plan.execute(dc, da, db, stream=stream), reps, 3) / reps
        st = plan.status()
        pipe = peaks["dmma_m8n8k4"] if dtype == "f64" else peaks["ffma"]
        t_roof = max(d["bytes"] / (hbm_peak * 1e9), d["flops"] / (pipe * 1e12))
        row = {"tag": it["tag"], "dtype": dtype, "kernel": d["kernel"], "ms": sec * 1e3, "gflops": d["flops"] / sec * 1e-9,
               "algorithmic_gbs": d["bytes"] / sec * 1e-9, "of_roofline": t_roof / sec, "device_status": st,
               "tma": [d.get("tma_x"), d.get("tma_y"), d.get("tma_c"), d.get("tma_ct")]}
        for k in ("cogent_v100_gflops", "cogent_p100_gflops", "nwchem_v100_gflops"):
            if k in it:
                row[k] = it[k]
        rows.append(row)
        plan.close()
        del dc, da, db
    torch.cuda.empty_cache()
    f64 = sorted(r["gflops"] for r in rows if r["dtype"] == "f64")
    print(json.dumps({"workload": "tccg", "metric": METRIC, "unit": "GFLOP/s", "n_gpus": 1, "rows": rows,
                      "peaks": {"hbm_gbs": hbm_peak, "dmma_tflops": peaks["dmma_m8n8k4"], "ffma_tflops": peaks["ffma"]},
                      "summary": {"items": len(rows), "f64_median_gflops": f64[len(f64) // 2] if f64 else None,
                                  "f64_min_gflops": f64[0] if f64 else None}}))


# the nine CCSD(T) doubles terms in the expression grammar: (operator, left indices, right indices); every term has its
# own pair of inputs and all accumulate into t3[h3,h2,h1,p6,p5,p4]
FUSED_TERMS = [("-=", "p7,p4,h1,h2", "p7,h3,p6,p5"), ("-=", "p7,p4,h2,h3", "p7,h1,p6,p5"), ("+=", "p7,p4,h1,h3", "p7,h2,p6,p5"),
               ("+=", "p7,p5,h1,h2", "p7,h3,p6,p4"), ("+=", "p7,p5,h2,h3", "p7,h1,p6,p4"), ("-=", "p7,p5,h1,h3", "p7,h2,p6,p4"),
               ("-=", "p7,p6,h1,h2", "p7,h3,p5,p4"), ("-=", "p7,p6,h2,h3", "p7,h1,p5,p4"), ("+=", "p7,p6,h1,h3", "p7,h2,p5,p4")]


def run_fused(args):
    """Nine contractions into one output: one fused pass (tc_execute_fused) beside the same terms run one by one."""
    import numpy as np
    import torch
    pkg, orc = entry.load_package(), entry.load_oracle()
    torch.cuda.set_device(0)
    E = 24
    out = "t3 [h3,%d,h2,%d,h1,%d,p6,%d,p5,%d,p4,%d]" % ((E,) * 6)
    lines = ["%s %s sum(p7,%d) * t2_%d [%s] * v2_%d [%s];" % (out, op, E, k + 1, l, k + 1, r) for k, (op, l, r) in enumerate(FUSED_TERMS)]
    n_out, na, nb = orc.sizes(lines[0])
    dc = torch.empty(n_out, dtype=torch.float64, device="cuda")
    pkg.fill_uniform(dc, 9, 0)
    das = [pkg.fill_uniform(torch.empty(na, dtype=torch.float64, device="cuda"), 10 + k, 1) for k in range(9)]
    dbs = [pkg.fill_uniform(torch.empty(nb, dtype=torch.float64, device="cuda"), 10 + k, 2) for k in range(9)]
    fused = pkg.FusedPlan(lines).commit()
    plans = [pkg.Plan(l).commit() for l in lines]
    # parity of the fused pass on a slab (p6, p5, p4 fixed): the nine loop nests of the checker, one after another
    fused.execute(dc, das, dbs)
    torch.cuda.synchronize()
    worst = 0.0
    for fix in ({"p6": 0, "p5": 0, "p4": 0}, {"p6": E - 1, "p5": 7, "p4": E - 1}):
        idx = ["h3", "h2", "h1", "p6", "p5", "p4"]
        st = {i: E ** n for n, i in enumerate(idx)}
        oc = sum(fix[i] * st[i] for i in fix)
        ref = orc.uniform(9, 0, E ** 3, np.float64, first=oc)
        for k, line in enumerate(lines):
            p = orc.parse(line)
            a, b = orc.uniform(10 + k, 1, na), orc.uniform(10 + k, 2, nb)
            strides, offs = {0: [st[i] for i in idx]}, {}
            for t, key in ((1, "left_idx"), (2, "right_idx")):
                s_, acc = [], 1
                for i in p[key]:
                    s_.append(acc)
                    acc *= E
                strides[t] = s_
                offs[t] = sum(fix.get(i, 0) * x for i, x in zip(p[key], s_))
            orc.contract(orc.with_extents(line, {i: 1 for i in fix}), ref, a[offs[1]:], b[offs[2]:], threads=host_threads(orc), strides=strides)
        worst = max(worst, orc.rel_error(dc[oc:oc + E ** 3].cpu().numpy(), ref))
    stream = torch.cuda.current_stream().cuda_stream
    steps = max(1, args.steps)
    t_f = time_passes(torch, lambda: fused.execute(dc, das, dbs, stream=stream), steps, max(1, args.warmup)) / steps
    t_s = time_passes(torch, lambda: [q.execute(dc, a, b, stream=stream) for q, a, b in zip(plans, das, dbs)], steps, max(1, args.warmup)) / steps
    d = fused.describe()
    print(json.dumps({"workload": "fused: nine CCSD(T) doubles terms into one 6-D output, extents %d" % E, "metric": METRIC, "unit": "GFLOP/s",
                      "n_gpus": 1, "dtype": "f64", "fused": {"gflops": d["flops"] / t_f * 1e-9, "ms": t_f * 1e3, "launches": 1,
                                                               "algorithmic_bytes": d["bytes"], "kernel": d["kernel"], "box": d["box"]},
                      "term_by_term": {"gflops": d["flops"] / t_s * 1e-9, "ms": t_s * 1e3, "launches": 9,
                                       "algorithmic_bytes": d["bytes_term_by_term"], "kernel": plans[0].describe()["kernel"]},
                      "parity": {"max_rel_err": worst, "tolerance": 1e-12, "ok": bool(worst <= 1e-12),
                                 "how": "two slabs of the fused result against the nine loop nests applied in order"}}))


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    if args.workload == "tccg":
        return run_tccg(args)
    if args.workload == "fused":
        return run_fused(args)
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
    name = args.workload or "cfg5"
    expr, dtype, seed = WORKLOADS[name]
    tdt = torch.float64 if dtype == "f64" else torch.float32
    ndt = np.float64 if dtype == "f64" else np.float32
    es = 8 if dtype == "f64" else 4
    stream = torch.cuda.current_stream().cuda_stream
    code = pkg.F64 if dtype == "f64" else pkg.F32

    # This rank's share: the whole contraction, or its slab of the slowest output index.
    plan_kw = {}
    if args.path != "auto":  # pin the arithmetic path (the profiles of non-default kernels are made this way)
        plan_kw["path"] = path_code(pkg, args.path)
    sh = shard.ExternalShard(expr, code, rank, world, **plan_kw)
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

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    for _ in range(max(args.warmup, 3)):
        one_pass()
    torch.cuda.synchronize()
    sampler.start()
    sec = time_passes(torch, one_pass, args.steps, 0, sync_all)
    clocks = sampler.stop()
    sec = max_over_ranks(sec)
    status = sh.plan.status()
    if max_over_ranks(float(status)) != 0:
        raise SystemExit("a bounded device wait gave up during the timed region (status %d): the run is void" % status)
    full_flops = 2.0 * float(np.prod([float(x) for x in g.full_extents.values()]))
    value = full_flops * args.steps / sec * 1e-9
    shard_flops, shard_bytes = sh.cost()

    # ---- parity of what was just timed: every rank, its own slab ----
    parity = parity_check(pkg, orc, torch, sh, dc, da, db, dtype, seed, stream)
    worst = max_over_ranks(parity["max_rel_err"] if parity["max_rel_err"] is not None else float("inf"))
    parity = {"max_rel_err": worst, "checked_elements": parity["checked_elements"] * world, "tolerance": TOL[dtype],
              "ok": bool(worst <= TOL[dtype]), "ranks": world,
              "how": "per rank after the timed region: C restored, one pass, one slab at the first and one at the last value "
                     "of the rank's range of %s plus sampled coordinates against the CPU loop nest" % g.index}

    # ---- end to end through the host-pointer C-ABI call (this rank's share) ----
    e2e_steps = 2 if g.c_slab_elems * es > (8 << 30) else max(1, min(args.steps, 3))
    slab_bytes = g.c_slab_elems * es
    pkg.fill_uniform(dc, seed, 0, first_index=g.offsets[0])
    hc = PinnedArray(torch, g.c_slab_elems, ndt)
    ha = PinnedArray(torch, na, ndt)
    hb = PinnedArray(torch, nb, ndt)
    torch.from_numpy(hc.arr).copy_(dc)
    torch.from_numpy(ha.arr).copy_(da)
    torch.from_numpy(hb.arr).copy_(db)
    torch.cuda.synchronize()
    del dc  # the host call keeps its own device copy of the slab
    torch.cuda.empty_cache()
    # the host call sees full input tensors and this rank's C slab: a plan over the slab's own extents
    hplan = g.make_plan(code, **plan_kw)
    hviews = (hc.arr, ha.arr[g.offsets[1]:], hb.arr[g.offsets[2]:])
    hplan.execute_host(*hviews)  # warm-up (also commits the plan and allocates its device buffers)
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        hplan.execute_host(*hviews)
    t_e2e = max_over_ranks(time.perf_counter() - t0)
    e2e_value = full_flops * e2e_steps / t_e2e * 1e-9
    h2d = (g.c_slab_elems + (na - g.offsets[1]) + (nb - g.offsets[2])) * es
    hplan.close()
    pinned_ok = hc.pinned and ha.pinned and hb.pinned
    for x in (hc, ha, hb):
        x.release()
    del hc, ha, hb, hviews, da, db
    torch.cuda.empty_cache()

    extra_rows = []
    if world > 1 and not args.workload:
        extra_rows.append(ksplit_case(pkg, orc, shard, torch, dist, rank, world, stream))

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the (single) kernel of the pass ----
    hbm_peak, hbm_src = measured_peaks()
    # the pipe the chosen kernel computes on; fp32 on the tensor cores costs three TF32 products per product, so its
    # ceiling in fp32 FLOP/s is a third of the TF32 probe's figure
    which, scale = {"dmma": (0, 1.0), "dfma": (4, 1.0), "ffma": (5, 1.0), "tf32x3": (6, 1.0 / 3.0),
                    "tf32x3_tcgen05": (7, 1.0 / 3.0)}.get(desc["math"], (0 if dtype == "f64" else 5, 1.0))
    pipe, pipe_peak = next(iter(pkg.measure_peaks(which=(which,)).items()))
    if scale != 1.0:
        pipe, pipe_peak = pipe + " / 3 (three TF32 products per fp32 product)", pipe_peak * scale
    launch_s = sec / args.steps
    t_hbm = shard_bytes / (hbm_peak * 1e9)
    t_pipe = shard_flops / (pipe_peak * 1e12)
    if t_pipe >= t_hbm:
        roof = {"bound": "tensor", "achieved": shard_flops / launch_s * 1e-12, "peak": pipe_peak, "unit": "TFLOP/s",
                "peak_source": "live %s probe (bench-only probe library; of measured -- the driver's peak "
                               "file has no fp64/fp32 pipe figure)" % pipe}
    else:
        roof = {"bound": "hbm", "achieved": shard_bytes / launch_s * 1e-9, "peak": hbm_peak, "unit": "GB/s",
                "peak_source": "MEASURED_PEAKS.json hbm_gbs (of %s)" % hbm_src}
    roof["frac"] = roof["achieved"] / roof["peak"]
    # per launch, from one ncu capture of THIS kernel on this workload (null when the plan picked another kernel,
    # another arithmetic path, or the shard is not a captured size)
    key = (desc["kernel"], name if world == 1 else ("cfg5_shard8" if (name, world) == ("cfg5", 8) else None))
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(key) if args.path == "auto" else None
    roof["kernel"] = desc["kernel"]
    roof["algorithmic_bytes_per_launch"] = shard_bytes
    roof["algorithmic_flops_per_launch"] = shard_flops
    roof["hbm"] = {"achieved": shard_bytes / launch_s * 1e-9, "peak": hbm_peak, "unit": "GB/s",
                   "frac": shard_bytes / launch_s * 1e-9 / hbm_peak, "peak_source": "MEASURED_PEAKS.json (%s)" % hbm_src}
    roof["pipe"] = {"achieved": shard_flops / launch_s * 1e-12, "peak": pipe_peak, "unit": "TFLOP/s",
                    "frac": shard_flops / launch_s * 1e-12 / pipe_peak, "peak_source": "live %s probe" % pipe}

    line = {
        "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": config_of(name, expr, seed, g.index, world, shard_bytes),
        "plan": {k: desc[k] for k in ("kernel", "math", "tile", "tiles", "ksplit", "vec_c")},
        "roofline": roof,
        "parity": parity,
        "e2e": {"value": e2e_value, "unit": "GFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": slab_bytes,
                "steps": e2e_steps, "page_locked": pinned_ok,
                "call": "tc_execute_host on page-locked host buffers (H2D of C, A, B, kernels, D2H of C; slabs of the "
                        "slowest output index pipelined over two streams); per rank, max over ranks"},
        "gpu_launches": sh.plan.launches * args.steps,
        "clocks": clocks,
    }

    if world == 1:
        # CPU baseline beside it (bounded sample, rank 0 only).
        line["cpu_baseline"] = cpu_baseline(orc, name, budget_s=12.0)
        if not args.workload:
            line["e2e_pageable"] = e2e_pageable_cfg2(pkg, orc, torch)
            rows = [quick_config(pkg, orc, torch, n, cogent=True) for n in ("cfg1", "cfg2", "cfg3")]
            # configuration 4 compares its arithmetic paths
            rows.append(quick_config(pkg, orc, torch, "cfg4", path="tcgen05", cogent=True))
            rows.append(quick_config(pkg, orc, torch, "cfg4", path="tcgen05", label="tcgen05, one CTA per tile", tile=(96, 128), variant=1))
            rows.append(quick_config(pkg, orc, torch, "cfg4", path="3xtf32"))
            rows.append(quick_config(pkg, orc, torch, "cfg4", path="ffma"))
            line["configs"] = rows
    if extra_rows:
        line["configs"] = extra_rows
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


def _max_sample(name):
    """Values of the slowest output index a CPU sample may hold: cfg5's slabs are 0.82 GB each."""
    return 4 if name == "cfg5" else 1 << 30


def cpu_baseline(orc, name, budget_s):
    """GFLOP/s of the loop nest on all host threads over a sample sized for about budget_s seconds."""
    threads = host_threads(orc)
    sec, flops, what, full = _time_sample(orc, name, 1, threads)
    count = int(max(1, min(full, _max_sample(name), budget_s / max(sec, 1e-4))))
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
    name = args.workload or "cfg5"
    expr, dtype, seed = WORKLOADS[name]
    threads = host_threads(orc)
    # size one step so that warm-up + steps stay near two minutes
    per_step = max(0.05, 110.0 / (args.steps + args.warmup))
    t1, _, _, full = _time_sample(orc, name, 1, threads)
    count = int(max(1, min(full, _max_sample(name), per_step / max(t1, 1e-4))))
    sub, (c, a, b), strides, flops, what, _ = _sample_problem(orc, name, count)
    for _ in range(args.warmup):
        orc.contract(sub, c, a, b, threads=threads, strides=strides)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.contract(sub, c, a, b, threads=threads, strides=strides)
    sec = time.perf_counter() - t0
    value = flops * args.steps / sec * 1e-9
    shard_bytes, cut = shard_bytes_of(name, world)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": config_of(name, expr, seed, cut, world, shard_bytes),
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": threads, "kind": "port",
                         "sample": what + "; the reference's CPU loop nest (restated in C, bit-identical to its "
                                          "compiled drivers), OpenMP over the outermost output loop; one step = this sample"},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + ["tccg", "fused"])
    ap.add_argument("--path", default="auto", choices=["auto", "dmma", "dfma", "ffma", "3xtf32", "tcgen05"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
