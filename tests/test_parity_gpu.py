"""Parity of the CUDA path (through the C ABI) with the CPU checker.

Gate everywhere: max|got - ref| / max|ref| <= 1e-12 (fp64) or 1e-5 (fp32),
inputs uniform[-1,1) from the seeded generator.
"""
import random

import numpy as np
import pytest

from conftest import CONFIGS, TOL
from test_parser import _random_expr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


def _dt(pkg, dtype):
    return pkg.F64 if np.dtype(dtype) == np.float64 else pkg.F32


def _run(pkg, orc, torch, expr, dtype, seed, **kw):
    """Executes on the GPU and returns (rel_err, plan description)."""
    c0, a, b = orc.make_inputs(expr, seed, dtype)
    ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    plan = pkg.Plan(expr, _dt(pkg, dtype), **kw)
    dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
    plan.execute(dc, da, db)
    torch.cuda.synchronize()
    desc = plan.describe()
    assert plan.status() == 0, "a bounded wait inside a persistent kernel gave up"
    plan.close()
    return orc.rel_error(dc.cpu().numpy(), ref), desc


def _scaled(expr, extent):
    """Same expression with every extent replaced (a reduced copy of a benchmark configuration)."""
    import re
    return re.sub(r",(\d+)", lambda m: ",%d" % extent, expr)


# ------------------------------------------------------------ generator ----
def test_device_generator_matches_checker(pkg, orc, torch_cuda):
    torch = torch_cuda
    for tdt, ndt in ((torch.float64, np.float64), (torch.float32, np.float32)):
        for seed, tid, first in ((0, 0, 0), (3, 1, 12345), (4, 2, (1 << 33) + 5)):
            t = torch.empty(4099, dtype=tdt, device="cuda")
            pkg.fill_uniform(t, seed, tid, first)
            assert np.array_equal(t.cpu().numpy(), orc.uniform(seed, tid, 4099, ndt, first))


# ------------------------------------------------- benchmark configurations ----
def test_config1_full_size_all_paths(pkg, orc, torch_cuda):
    expr, dt, seed = CONFIGS[0]
    for kw in ({}, {"path": pkg.PATH_DFMA}, {"tile": (128, 128)}, {"tile": (128, 64), "variant": 2},
               {"tile": (64, 96)}, {"tile": (64, 64), "split_k": 2}, {"tile": (128, 64), "variant": 3},
               {"tile": (64, 96), "variant": 3},
               {"tile": (128, 64), "variant": 3, "c_path": 1}, {"tile": (128, 64), "variant": 4}):
        err, _ = _run(pkg, orc, torch_cuda, expr, dt, seed, **kw)
        assert err <= TOL[dt], (kw, err)


@pytest.mark.parametrize("idx,extent", [(1, 24), (2, 16), (3, 8), (4, 10)])
def test_reduced_configs(pkg, orc, torch_cuda, idx, extent):
    expr, dt, seed = CONFIGS[idx]
    expr = _scaled(expr, extent)
    if idx == 3:
        expr = expr.replace("sum(l,8)", "sum(l,24)")
    if idx == 4:
        expr = expr.replace("sum(g,10)", "sum(g,40)")
    tiles = [None, (128, 128), (64, 64)] + ([(128, 64), (128, 96), (64, 96)] if dt == "float64" else [(96, 128)])
    if dt == "float64":
        for kw in ({"tile": (128, 32), "variant": 3}, {"tile": (128, 32), "variant": 3, "c_path": 1}, {"tile": (128, 32), "variant": 3, "tma": 1}):
            err, d = _run(pkg, orc, torch_cuda, expr, dt, seed, **kw)
            assert err <= TOL[dt] and d["kernel"] == "dmma_ws_128x32", (expr, kw, err)
    for tile in tiles:
        err, d = _run(pkg, orc, torch_cuda, expr, dt, seed, **({"tile": tile} if tile else {}))
        assert err <= TOL[dt], (expr, tile, err)
    if dt == "float32":  # both fp32 arithmetic paths, both ways of reaching the output
        for path in (pkg.PATH_FFMA, pkg.PATH_3XTF32):
            for kw in ({}, {"tile": (96, 128), "c_path": 1}, {"tile": (128, 128), "c_path": 3}, {"tile": (64, 64), "split_k": 2},
                       {"tile": (64, 64), "c_path": 2}):
                err, d = _run(pkg, orc, torch_cuda, expr, dt, seed, path=path, **kw)
                assert err <= TOL[dt], (expr, path, kw, err)
        err, d = _run(pkg, orc, torch_cuda, expr, dt, seed, path=pkg.PATH_FFMA, tile=(128, 64))
        assert err <= TOL[dt]
    if dt == "float64":
        for kw in ({"path": pkg.PATH_DFMA}, {"tile": (128, 128), "variant": 2}, {"tile": (128, 64), "variant": 2},
                   {"tile": (64, 64), "l2_prefetch": 1}, {"tile": (64, 64), "c_path": 2},
                   {"tile": (128, 64), "variant": 3}, {"tile": (64, 96), "variant": 3},
                   {"tile": (128, 64), "variant": 3, "c_path": 1},
                   {"tile": (64, 96), "variant": 3, "c_path": 1, "l2_prefetch": 2}, {"tile": (128, 64), "variant": 3, "tma": 1},
                   {"tile": (128, 64), "variant": 4}, {"tile": (128, 64), "variant": 4, "tma": 3}):
            err, _ = _run(pkg, orc, torch_cuda, expr, dt, seed, **kw)
            assert err <= TOL[dt], (expr, kw, err)


def _slab_check(pkg, orc, torch, expr, dtype, seed, fixes, keep=None, **plan_kw):
    """Full-size run; the checker recomputes only slabs (some output indices fixed)."""
    p = orc.parse(expr)
    ext = dict(zip(p["out_idx"] + p["sum_idx"], p["out_ext"] + p["sum_ext"]))
    nc, na, nb = orc.sizes(expr)
    tdt = torch.float64 if np.dtype(dtype) == np.float64 else torch.float32
    dc = torch.empty(nc, dtype=tdt, device="cuda")
    da = torch.empty(na, dtype=tdt, device="cuda")
    db = torch.empty(nb, dtype=tdt, device="cuda")
    pkg.fill_uniform(dc, seed, 0)
    pkg.fill_uniform(da, seed, 1)
    pkg.fill_uniform(db, seed, 2)
    plan = pkg.Plan(expr, _dt(pkg, dtype), **plan_kw)
    plan.execute(dc, da, db)
    torch.cuda.synchronize()
    assert plan.status() == 0
    if keep is not None:
        keep["desc"] = plan.describe()
    a, b = orc.uniform(seed, 1, na, dtype), orc.uniform(seed, 2, nb, dtype)

    def strides(idx):
        s, acc = [], 1
        for i in idx:
            s.append(acc)
            acc *= ext[i]
        return s

    sc, sa, sb = strides(p["out_idx"]), strides(p["left_idx"]), strides(p["right_idx"])
    worst = 0.0
    for fix in fixes:
        sub = orc.with_extents(expr, {i: 1 for i in fix})
        off = lambda idx, st: sum(fix.get(i, 0) * s for i, s in zip(idx, st))
        oc = off(p["out_idx"], sc)
        # the slab of C spans [oc, oc + span); regenerate just that range of the initial output
        span = 1 + sum((1 if i in fix else ext[i]) * s - s for i, s in zip(p["out_idx"], sc))
        c_ref = orc.uniform(seed, 0, span, dtype, first=oc)
        c_init = c_ref.copy()
        orc.contract(sub, c_ref, a[off(p["left_idx"], sa):], b[off(p["right_idx"], sb):],
                     threads=orc.max_threads(), strides={0: sc, 1: sa, 2: sb})
        got = dc[oc:oc + span].cpu().numpy()
        touched = c_ref != c_init
        assert touched.any()
        # elements outside the slab inside the span must not be compared against the slab's reference
        worst = max(worst, orc.rel_error(got[touched], c_ref[touched]))
    plan.close()
    if keep is not None:
        keep["dc"] = dc
    del dc, da, db
    torch.cuda.empty_cache()
    return worst


def test_config2_full_size_slabs(pkg, orc, torch_cuda):
    expr, dt, seed = CONFIGS[1]
    err = _slab_check(pkg, orc, torch_cuda, expr, dt, seed, [{"d": 0, "c": 0}, {"d": 95, "c": 95}, {"d": 41, "b": 7}])
    assert err <= TOL[dt]


def test_config3_full_size_slabs(pkg, orc, torch_cuda):
    expr, dt, seed = CONFIGS[2]
    err = _slab_check(pkg, orc, torch_cuda, expr, dt, seed, [{"c": 0, "d": 0}, {"c": 63, "d": 63}, {"a": 17, "b": 33}])
    assert err <= TOL[dt]


def test_config4_full_size_slabs(pkg, orc, torch_cuda):
    expr, dt, seed = CONFIGS[3]
    err = _slab_check(pkg, orc, torch_cuda, expr, dt, seed,
                      [{"i": 0, "j": 0, "k": 0}, {"i": 23, "j": 23, "k": 23}, {"b": 5, "c": 11, "k": 2}])
    assert err <= TOL[dt]


def test_config5_one_eighth_slabs(pkg, orc, torch_cuda):
    # the shard one GPU owns when the large configuration is split 8 ways along f (4.1 GB of output)
    expr, dt, seed = CONFIGS[4]
    expr = expr.replace("f,40", "f,5")
    err = _slab_check(pkg, orc, torch_cuda, expr, dt, seed,
                      [{"d": 0, "e": 0, "f": 0}, {"d": 39, "e": 39, "f": 4}, {"a": 3, "b": 1, "f": 2, "e": 7}])
    assert err <= TOL[dt]


def _sampled_check(orc, torch, dc, expr, dtype, seed, count, rng_seed):
    """`count` uniformly sampled output coordinates of a full-size run, recomputed on the host from the
    counter-based inputs (the whole output need not exist on the host).  Returns max|got-ref| / max|ref|."""
    p = orc.parse(expr)
    names = p["out_idx"] + p["sum_idx"]
    ext = dict(zip(names, p["out_ext"] + p["sum_ext"]))
    nc, na, nb = orc.sizes(expr)
    a = orc.uniform(seed, 1, na, dtype)
    b = orc.uniform(seed, 2, nb, dtype)
    rng = np.random.default_rng(rng_seed)
    lin = np.sort(rng.integers(0, nc, size=count, dtype=np.int64))
    coord, r = {}, lin.copy()
    for i in p["out_idx"]:
        coord[i] = r % ext[i]
        r //= ext[i]

    def offsets(idx, fixed):
        off, acc = np.zeros(count, dtype=np.int64), 1
        for i in idx:
            off = off + (coord[i] if i in coord else fixed[i]) * acc
            acc *= ext[i]
        return off

    ref = orc.uniform_at(seed, 0, lin, dtype).astype(np.float64)
    sign = -1.0 if p["op"] == "-=" else 1.0
    if p["op"] == "=":
        ref[:] = 0.0
    ks = [ext[i] for i in p["sum_idx"]]
    for flat in range(int(np.prod(ks))):
        fixed, q = {}, flat
        for i, e in zip(p["sum_idx"], ks):
            fixed[i] = q % e
            q //= e
        ref += sign * a[offsets(p["left_idx"], fixed)].astype(np.float64) * b[offsets(p["right_idx"], fixed)].astype(np.float64)
    got = dc[torch.from_numpy(lin).cuda()].cpu().numpy().astype(np.float64)
    return float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))


def test_config5_full_size(pkg, orc, torch_cuda):
    """The large configuration at its full extents on one GPU: 4.096e9 output elements (32.8 GB), offsets beyond
    2^31 elements, 500 x 1000 tiles.  Checked on slabs at both ends and inside, and on 2e5 sampled coordinates."""
    torch = torch_cuda
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * (1 << 30):
        pytest.skip("needs 40 GB of free device memory")
    expr, dt, seed = CONFIGS[4]
    fixes = [{"d": 0, "e": 0, "f": 0}, {"d": 39, "e": 39, "f": 39}, {"d": 17, "e": 3, "f": 22}, {"a": 39, "b": 0, "c": 21, "e": 5, "f": 31}]
    keep = {}
    err = _slab_check(pkg, orc, torch, expr, dt, seed, fixes, keep=keep)
    assert err <= TOL[dt], err
    serr = _sampled_check(orc, torch, keep["dc"], expr, dt, seed, 200000, 5)
    keep.clear()
    torch.cuda.empty_cache()
    assert serr <= TOL[dt], serr


# ------------------------------------------------------- random expressions ----
@pytest.mark.parametrize("path", ["dmma", "dfma", "ffma", "tf32x3", "persistent", "persistent_bulk"])
def test_random_contractions(pkg, orc, torch_cuda, path):
    rng = random.Random({"dmma": 11, "dfma": 12, "ffma": 13, "tf32x3": 16, "persistent": 14, "persistent_bulk": 15}[path])
    dt = "float32" if path in ("ffma", "tf32x3") else "float64"
    kw = {"path": {"dfma": pkg.PATH_DFMA, "ffma": pkg.PATH_FFMA, "tf32x3": pkg.PATH_3XTF32}.get(path, pkg.PATH_AUTO)}
    if path.startswith("persistent"):  # small problems would not pick the persistent kernel by themselves
        kw = {"tile": (128, 64), "variant": 3, "c_path": 3 if path.endswith("bulk") else 1}
    for n in range(40):
        expr = _random_expr(rng, max_out=5, max_sum=3, multi_char=(n % 4 == 0))
        err, d = _run(pkg, orc, torch_cuda, expr, dt, 100 + n, **kw)
        assert err <= TOL[dt], (expr, err, d)


def test_random_midsize_contractions_with_forced_kernels_and_options(pkg, orc, torch_cuda):
    """Random expressions with 0.3-3 M outputs, ragged and aligned extents, contractions of 1 to 64, pushed through
    the persistent fp64 tiles and the tcgen05 / mma.sync / FFMA fp32 kernels with random epilogue, tensor-map and
    K-slice options: many tiles per CTA, one K step per tile, clipped boxes -- the mix that exposes hand-over bugs."""
    rng = random.Random(4242)
    done = 0
    while done < 36:
        expr = _random_expr(rng, max_out=6, max_sum=2)
        p = orc.parse(expr)
        base = max(2, int(round(rng.choice([3e5, 1e6, 3e6]) ** (1.0 / len(p["out_idx"])))))
        pick = lambda b: max(1, rng.choice([b, b + 1, b - 1, (b + 3) // 4 * 4, (b + 7) // 8 * 8, 2 * b, max(1, b // 2)]))
        ext = {i: pick(base) for i in p["out_idx"]}
        ext.update({i: rng.choice([1, 3, 8, 16, 24, 40, 64]) for i in p["sum_idx"]})
        if np.prod([float(v) for v in ext.values()]) > 1.5e8:
            continue
        expr = orc.with_extents(expr, ext)
        kw64 = {"tile": rng.choice([(64, 96), (128, 64), (128, 32)]), "variant": 3, "c_path": rng.choice([0, 1, 2, 3]),
                "tma": rng.choice([0, 1, 2, 3, 4]), "l2_prefetch": rng.choice([0, 1, 2])}
        if done % 3 == 2:  # the output-resident kernel (falls back to the 128 x 64 persistent kernel where C is no box tensor)
            kw64 = {"tile": (128, 64), "variant": 4, "tma": rng.choice([0, 3, 4])}
        kw32 = rng.choice([
            {"path": pkg.PATH_TCGEN05, "tile": rng.choice([(96, 128), (128, 128)]), "c_path": rng.choice([0, 1, 3]),
             "split_k": rng.choice([0, 1, 3])},
            {"path": pkg.PATH_3XTF32, "c_path": rng.choice([0, 1, 3]), "split_k": rng.choice([0, 1, 2])},
            {"path": pkg.PATH_FFMA, "c_path": rng.choice([0, 1, 2, 3])}])
        for dt, kw in (("float64", kw64), ("float32", kw32)):
            err, d = _run(pkg, orc, torch_cuda, expr, dt, 700 + done, **kw)
            assert err <= TOL[dt], (expr, dt, kw, err, d["kernel"])
        # the persistent fp32 kernel wherever the output's layout allows it (the plan is refused elsewhere), both ways
        # of sending the tile; and the persistent fp64 kernel with K slices
        kwt = {"path": pkg.PATH_TCGEN05, "tile": rng.choice([(96, 128), (128, 128)]), "variant": 2, "c_path": rng.choice([0, 1, 3])}
        try:
            err, d = _run(pkg, orc, torch_cuda, expr, "float32", 800 + done, **kwt)
            assert d["kernel"].startswith("tf32wt_") and err <= TOL["float32"], (expr, kwt, err, d["kernel"])
        except pkg.TcError as e:
            assert e.status == 3, (expr, kwt, e)
        kws = {"tile": rng.choice([(128, 64), (128, 32), (64, 96)]), "variant": 3, "split_k": rng.choice([2, 3, 7])}
        err, d = _run(pkg, orc, torch_cuda, expr, "float64", 900 + done, **kws)
        assert err <= TOL["float64"], (expr, kws, err, d["kernel"], d["ksplit"])
        done += 1


def test_cuda_path_against_every_compiled_reference_nest(pkg, orc, torch_cuda):
    """All 57 loop nests the reference ships (48 fp64 + 9 fp32 drivers), compiled from its own sources:
    the CUDA path is compared with THEIR output, not with the restatement."""
    if not orc.ref_available():
        pytest.skip("the reference's nests are not compiled here (oracle/_ref absent)")
    torch = torch_cuda
    rng = np.random.default_rng(2024)
    for tag, info in sorted(orc.ref_table().items()):
        p = orc.parse(info["expr"])
        ext = {n: int(rng.integers(3, 13)) for n in p["out_idx"] + p["sum_idx"]}
        expr = orc.with_extents(info["expr"], ext)
        dt = "float64" if info["dtype"] == "f64" else "float32"
        c0, a, b = orc.make_inputs(expr, 500, dt)
        ref = orc.ref_contract(tag, ext, c0.copy(), a, b)
        plan = pkg.Plan(expr, _dt(pkg, dt))
        dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
        plan.execute(dc, da, db)
        torch.cuda.synchronize()
        assert orc.rel_error(dc.cpu().numpy(), ref) <= TOL[dt], (tag, expr)
        plan.close()


@pytest.mark.parametrize("extents", ["ragged", "multiples_of_8"])
def test_every_reference_class_at_kernel_scale(pkg, orc, torch_cuda, extents):
    """The same 57 expression classes with extents large enough (4-16 M outputs) that the planner picks the
    kernels the benchmarks run on -- persistent fp64, tcgen05 fp32, tensor-map copies where the shape allows --
    checked against the checker's loop nest.  Throughput per class is written as JSON into the directory named by the
    environment variable TC_SWEEP_OUT, when it is set."""
    if not orc.ref_available():
        pytest.skip("the reference's expression table is not built here (oracle/_ref absent)")
    import json
    import os
    torch = torch_cuda
    rng = np.random.default_rng(77)
    rows = []
    kernels = set()
    for tag, info in sorted(orc.ref_table().items()):
        p = orc.parse(info["expr"])
        rank, nsum = len(p["out_idx"]), len(p["sum_idx"])
        base = {2: 2600, 3: 190, 4: 52, 5: 23, 6: 14}.get(rank, 10)
        ext = {n: int(base + rng.integers(-base // 8, base // 8 + 1)) for n in p["out_idx"]}
        kbase = {1: 40, 2: 7, 3: 4}.get(nsum, 3)
        ext.update({n: int(kbase + rng.integers(0, kbase // 2 + 1)) for n in p["sum_idx"]})
        if extents == "multiples_of_8":  # the sizes benchmark suites for this operation typically use
            ext = {n: max(8, (e + 4) // 8 * 8) for n, e in ext.items()}
        expr = orc.with_extents(info["expr"], ext)
        dt = "float64" if info["dtype"] == "f64" else "float32"
        c0, a, b = orc.make_inputs(expr, 900, dt)
        ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
        plan = pkg.Plan(expr, _dt(pkg, dt))
        dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
        plan.execute(dc, da, db)
        torch.cuda.synchronize()
        d = plan.describe()
        assert plan.status() == 0, (tag, expr)
        err = orc.rel_error(dc.cpu().numpy(), ref)
        assert err <= TOL[dt], (tag, expr, err, d["kernel"])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            plan.execute(dc, da, db)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 3
        rows.append({"tag": tag, "dtype": info["dtype"], "expr": expr, "kernel": d["kernel"], "ms": ms,
                     "gflops": d["flops"] / ms * 1e-6, "gbs": d["bytes"] / ms * 1e-6, "rel_err": err,
                     "tma": [d.get("tma_x"), d.get("tma_y"), d.get("tma_c"), d.get("tma_ct")]})
        kernels.add(d["kernel"])
        plan.close()
        del dc, da, db
    assert len(rows) == 57
    assert any(k.startswith("dmma_ws") for k in kernels), kernels
    out = os.environ.get("TC_SWEEP_OUT")
    if out and os.path.isdir(out):
        with open(os.path.join(out, "sweep_reference_classes_%s.json" % extents), "w") as f:
            json.dump(rows, f, indent=1)


EDGE = [
    "C [a,1,b,1] += sum(c,1) * A [c,a] * B [b,c];",                         # everything is a scalar
    "C [a,5] += sum(b,7) * A [b,a] * B [b];",                               # right operand has no external index
    "C [a,5] -= sum(b,7) * A [b] * B [a,b];",                               # left operand has no external index
    "C [a,13,b,11] += sum(c,1) * A [a,c] * B [c,b];",                       # outer product
    "C [a,127,b,129] += sum(c,17) * A [c,a] * B [c,b];",                    # one off the tile sizes, K just over a step
    "C [a,2,b,3,c,5,d,7,e,2,f,3] += sum(g,11,h,2) * A [h,f,d,b,g] * B [g,a,c,h,e];",  # 6-D output, prime extents
    "C [a,31,b,37] = sum(c,4099) * A [c,a] * B [b,c];",                     # long prime contraction, overwrite
    "C [a,64,b,64] -= sum(c,64) * A [a,c] * B [b,c];",                      # both operands external-contiguous
    "C [a,64,b,64] += sum(c,64) * A [c,a] * B [c,b];",                      # both operands contraction-contiguous
    "C [a,150,b,70] -= sum(d,37) * A [d,a] * B [d,b];",                     # 2-D operands (TMA boxes), ragged everywhere
    "C [a,24,b,8,c,70] = sum(d,50) * A [d,a,b] * B [d,c];",                 # fused externals behind one TMA map
]


@pytest.mark.parametrize("expr", EDGE)
def test_edge_shapes(pkg, orc, torch_cuda, expr):
    for dt in ("float64", "float32"):
        err, d = _run(pkg, orc, torch_cuda, expr, dt, 42)
        assert err <= TOL[dt], (expr, dt, err, d)
    err, d = _run(pkg, orc, torch_cuda, expr, "float32", 42, path=pkg.PATH_FFMA)
    assert err <= TOL["float32"], (expr, err, d)
    for kw in ({"path": pkg.PATH_DFMA}, {"tile": (128, 64), "variant": 3}, {"tile": (64, 96), "variant": 3, "c_path": 1},
               {"tile": (128, 32), "variant": 3}, {"tile": (128, 64), "variant": 4}):
        err, _ = _run(pkg, orc, torch_cuda, expr, "float64", 42, **kw)
        assert err <= TOL["float64"], (expr, kw, err)


TENSOR_OUT = [
    # one M run and one N dimension: tails of both are clipped by the copy engine
    "C [a,200,b,70] += sum(c,40) * A [c,a] * B [c,b];",
    "C [a,136,b,50] -= sum(c,24) * A [a,c] * B [b,c];",
    "C [a,132,b,34] = sum(c,19) * A [c,a] * B [b,c];",
    # the fastest M dimension is a multiple of both tiles; slower M and N dimensions become tensor dimensions
    "C [a,128,b,32,c,3,d,2] += sum(e,24) * A [e,a,c] * B [b,d,e];",
    "C [a,128,b,3,c,16,d,5] -= sum(e,33) * A [a,e,b] * B [e,c,d];",
    "C [a,64,b,2,c,96] += sum(e,32) * A [a,e,b] * B [e,c];",
    # one K step per tile: a consumer group is back at the shared staging area before its previous tile has been
    # read out (the staging hand-over must not confuse that phase with the one it waits for)
    "t2 [c,20,e,40,h,20,q,40,w,20] += sum(z,16) * C [c,e,z,h] * B [z,w,q];",
    "C [a,256,b,64,c,96] -= sum(e,8) * A [e,a,b] * B [e,c];",
    # (b, c) are contiguous in C, not in B: one N dimension of 96 for the output view
    "C [a,128,b,24,c,4] += sum(e,16) * A [e,a] * B [b,e,c];",
    # N's fastest dimension is not a multiple of 16 while N has two dimensions: must fall back
    "C [a,128,b,24,c,3,d,4] += sum(e,16) * A [e,a,c] * B [b,d,e];",
]


@pytest.mark.parametrize("expr", TENSOR_OUT)
def test_persistent_tensor_box_epilogue(pkg, orc, torch_cuda, expr):
    """Output batches as tiled TMA reduce/store boxes agree with the checker and, bit for bit, with the per-row
    bulk copies they replace (both add the same products to the same words)."""
    torch = torch_cuda
    for tile in ((128, 64), (64, 96), (128, 32)):
        outs = []
        for tma in (0, 2):
            c0, a, b = orc.make_inputs(expr, 77, "float64")
            ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
            plan = pkg.Plan(expr, pkg.F64, tile=tile, variant=3, c_path=3, tma=tma)
            dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
            plan.execute(dc, da, db)
            torch.cuda.synchronize()
            assert plan.status() == 0
            d = plan.describe()
            plan.close()
            got = dc.cpu().numpy()
            assert orc.rel_error(got, ref) <= TOL["float64"], (expr, tile, tma, d)
            outs.append(got)
        assert np.array_equal(outs[0], outs[1]), (expr, tile)


@pytest.mark.parametrize("expr", TENSOR_OUT + [
    "C [a,40,b,40,c,40,d,40,e,10,f,2] += sum(g,40) * A [g,a,b,c] * B [d,e,f,g];",   # the large configuration's shape, reduced
    "C [a,40,b,40,c,40,d,40,e,10,f,2] -= sum(g,7) * A [g,a,b,c] * B [d,e,f,g];",
    "C [a,200,b,70] = sum(c,40) * A [c,a] * B [c,b];",                               # overwrite: no loads of C
])
@pytest.mark.parametrize("tile", [(128, 64)])
def test_output_resident_kernel(pkg, orc, torch_cuda, expr, tile):
    """The persistent kernel that keeps the output tile in shared memory (tiled TMA load of C, add in shared memory,
    tiled TMA store) against the checker; where whole tiles are not boxes of C it must fall back and still be right."""
    torch = torch_cuda
    c0, a, b = orc.make_inputs(expr, 78, "float64")
    ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    ref2 = orc.contract(expr, ref.copy(), a, b, threads=orc.max_threads())
    plan = pkg.Plan(expr, pkg.F64, tile=tile, variant=4)
    dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
    plan.execute(dc, da, db)
    torch.cuda.synchronize()
    d = plan.describe()
    assert d["kernel"] == "dmma_wc_%dx%d" % tile and plan.status() == 0
    assert orc.rel_error(dc.cpu().numpy(), ref) <= TOL["float64"], (expr, d)
    plan.execute(dc, da, db)       # a second pass over the result of the first
    torch.cuda.synchronize()
    assert plan.status() == 0 and orc.rel_error(dc.cpu().numpy(), ref2) <= TOL["float64"], (expr, d)
    # off 16-byte alignment the copy engine cannot address C: same plan, stand-in kernel
    pad = torch.cat([torch.zeros(1, dtype=torch.float64), torch.from_numpy(c0)]).cuda()
    plan.execute(pad[1:], da, db)
    torch.cuda.synchronize()
    assert plan.status() == 0 and orc.rel_error(pad[1:].cpu().numpy(), ref) <= TOL["float64"], (expr, "unaligned")
    plan.close()


TCGEN05 = [
    ("C [a,96,b,128] = sum(c,8) * A [a,c] * B [b,c];", (96, 128)),                 # one tile, one group of 8 k
    ("C [a,96,b,128] += sum(c,16) * A [a,c] * B [b,c];", (96, 128)),               # one full K step
    ("C [a,128,b,128] -= sum(c,40) * A [c,a] * B [c,b];", (128, 128)),             # three K steps, the last half full
    ("C [a,200,b,300] -= sum(c,37) * A [c,a] * B [b,c];", (128, 128)),             # ragged tiles: element-wise output
    ("C [a,200,b,300] += sum(c,37) * A [c,a] * B [b,c];", (96, 128)),
    ("C [a,24,b,24,c,24,i,8,j,8,k,8] += sum(l,24) * A [l,a,i,j] * B [b,c,k,l];", None),  # the shape of configuration 4
    ("C [a,48,b,8,c,16] += sum(d,1000,e,3) * A [a,e,d] * B [d,b,c,e];", (96, 128)),      # long contraction
]


@pytest.mark.parametrize("expr,tile", TCGEN05)
def test_tcgen05_three_tf32_products(pkg, orc, torch_cuda, expr, tile):
    """fp32 on tcgen05.mma with tensor-memory accumulators: same arithmetic as the mma.sync path, same tolerance."""
    kw = {"path": pkg.PATH_TCGEN05}
    if tile:
        kw["tile"] = tile
    err, d = _run(pkg, orc, torch_cuda, expr, "float32", 21, **kw)
    assert d["math"] == "tf32x3_tcgen05", d
    assert err <= TOL["float32"], (expr, err, d)
    # K slices (partials through the workspace) and the read-modify-write output
    err, d = _run(pkg, orc, torch_cuda, expr, "float32", 22, split_k=8, **kw)
    assert err <= TOL["float32"], (expr, "split_k", err, d)
    err, d = _run(pkg, orc, torch_cuda, expr, "float32", 23, c_path=1, **kw)
    assert err <= TOL["float32"], (expr, "c_path 1", err, d)


WT = [
    ("C [a,96,b,128] = sum(c,8) * A [a,c] * B [b,c];", (96, 128)),                    # one tile, half a K step
    ("C [a,128,b,256] += sum(c,16) * A [a,c] * B [b,c];", (128, 128)),                # two tiles, one K step
    ("C [a,256,b,384] -= sum(c,40) * A [c,a] * B [c,b];", (128, 128)),                # contraction-major operands
    ("C [a,512,b,640] += sum(c,300) * A [a,c] * B [c,b];", (128, 128)),               # more tiles than buffers; E0 = 128
    ("C [a,512,b,640] = sum(c,300) * A [c,a] * B [b,c];", (128, 128)),                # `=`: nothing fetched
    ("C [a,200,b,300] -= sum(c,37) * A [c,a] * B [b,c];", (128, 128)),                # ragged tiles: E0 = 8, per-n chunks refused
    ("C [a,192,b,300] += sum(c,37) * A [c,a] * B [b,c];", (96, 128)),                 # ragged in n only; E0 = 96
    ("C [a,320,b,300] += sum(c,37) * A [c,a] * B [b,c];", (128, 128)),                # E0 = 64: two runs, last tile half empty
    ("C [a,24,b,24,c,24,i,8,j,8,k,8] += sum(l,24) * A [l,a,i,j] * B [b,c,k,l];", (96, 128)),   # configuration 4's shape: dense runs
    ("C [a,24,b,24,c,24,i,8,j,8,k,8] -= sum(l,24) * A [l,a,i,j] * B [b,c,k,l];", None),
    ("C [a,48,b,40,c,16,d,6] += sum(e,20,f,3) * A [a,f,d,e] * B [e,b,c,f];", (96, 128)),      # element gathers of X
    ("C [a,256,b,8,c,48] += sum(d,1000,e,3) * A [a,e,d] * B [d,b,c,e];", (128, 128)),          # 188 K steps: six segments
    ("C [a,384,b,256] = sum(c,2100) * A [c,a] * B [c,b];", (128, 128)),                        # segments with `=`
    ("C [a,2048,b,2048] += sum(c,512) * A [c,a] * B [c,b];", (128, 128)),     # long K, several tiles per CTA: one tile buffer
    ("C [a,1536,b,2048] -= sum(c,72) * A [a,c] * B [b,c];", (96, 128)),       # short K, several tiles per CTA: three buffers
    ("C [a,320,b,8,c,50] += sum(d,52) * A [d,a] * B [d,b,c];", (128, 128)),    # boxes that run off the matrix in rows and in k
    ("C [a,64,b,5,c,300] += sum(d,60) * A [d,a,b] * B [c,d];", (128, 128)),   # one operand in boxes, the other in 16-byte copies
    ("C [a,320,b,300] = sum(d,28) * A [a,d] * B [d,b];", (128, 128)),         # ... and the other way round
]


@pytest.mark.parametrize("expr,tile", WT)
def test_persistent_tcgen05_kernel(pkg, orc, torch_cuda, expr, tile):
    """The persistent fp32 kernel (two accumulators in tensor memory, output tile resident in shared memory, chains cut
    into segments inside the kernel) against the loop nest; where its output layout is not possible the plan is refused."""
    kw = {"path": pkg.PATH_TCGEN05}
    if tile:
        kw.update(tile=tile, variant=2)
    if "a,200" in expr:
        with pytest.raises(pkg.TcError):
            pkg.Plan(expr, pkg.F32, **kw).commit()
        return
    err, d = _run(pkg, orc, torch_cuda, expr, "float32", 24, **kw)
    assert d["kernel"].startswith("tf32wt_") and d["chain"] <= 512 and d["ksplit"] == 1 and d["passes"] == 1, d
    assert err <= TOL["float32"], (expr, err, d)
    # (default: the tile leaves as bulk reduce-adds of the products)  The other way: old values fetched, sums stored.
    err, d = _run(pkg, orc, torch_cuda, expr, "float32", 27, c_path=1, **kw)
    assert d["kernel"].startswith("tf32wt_") and err <= TOL["float32"], (expr, "fetch and store", err, d)
    # operands that are plain matrices arrive as tiled TMA boxes by default; the same plan with per-thread copies
    if d["tma_x"] or d["tma_y"] or d["tma_xe"] or d["tma_ye"]:
        err, d = _run(pkg, orc, torch_cuda, expr, "float32", 28, tma=1, **kw)
        assert d["kernel"].startswith("tf32wt_") and err <= TOL["float32"], (expr, "no boxes", err, d)


def test_persistent_tcgen05_kernel_boxes_on_long_contractions_repeatedly(pkg, orc, torch_cuda):
    """Both operands in TMA boxes and three to five accumulation segments per tile: the shape on which a stage that was
    handed back before its values had left the registers' owner came out wrong about once in four hundred stages.
    Twenty executions per length, each checked."""
    torch = torch_cuda
    for k in (1028, 2112):
        expr = "C [a,384,b,256] = sum(c,%d) * A [c,a] * B [c,b];" % k
        c0, a, b = orc.make_inputs(expr, 41, "float32")
        ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
        plan = pkg.Plan(expr, pkg.F32, path=pkg.PATH_TCGEN05, tile=(128, 128), variant=2)
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for rep in range(20):
            dc = torch.from_numpy(c0).cuda()
            plan.execute(dc, da, db)
            torch.cuda.synchronize()
            assert plan.status() == 0
            assert orc.rel_error(dc.cpu().numpy(), ref) <= TOL["float32"], (expr, rep)
        d = plan.describe()
        assert d["tma_x"] and d["tma_y"] and d["kernel"] == "tf32wt_128x128", d
        plan.close()


def test_persistent_tcgen05_kernel_random_matrices(pkg, orc, torch_cuda):
    """Random matrix products through the persistent fp32 kernel: ragged column counts, contraction lengths with and
    without a short last step and with one to five accumulation segments, every operand order (so boxes for both
    operands, for one, for none), every operator."""
    rng = random.Random(777)
    ran = boxes = 0
    for case in range(18):
        bm = rng.choice([96, 128])
        m = bm * rng.randint(1, 5) if bm == 96 or rng.random() < 0.5 else 64 * rng.randint(2, 9)   # runs of 64 and more
        n = rng.choice([rng.randint(60, 700), 128 * rng.randint(1, 5)])
        k = rng.choice([52, 64, 100, 256, 516, 1040, 1100, 2052])
        a_ = rng.choice(["A [c,a]", "A [c,a]", "A [a,c]"])
        b_ = rng.choice(["B [c,b]", "B [c,b]", "B [b,c]"])
        op = rng.choice(["+=", "-=", "="])
        expr = "C [a,%d,b,%d] %s sum(c,%d) * %s * %s;" % (m, n, op, k, a_, b_)
        kw = {"path": pkg.PATH_TCGEN05, "tile": (bm, 128), "variant": 2, "c_path": rng.choice([0, 1])}
        try:
            err, d = _run(pkg, orc, torch_cuda, expr, "float32", 600 + case, **kw)
        except pkg.TcError as e:
            assert e.status == 3, (expr, kw, e)
            continue
        assert d["kernel"].startswith("tf32wt_") and d["chain"] <= 512, (expr, d)
        assert err <= TOL["float32"], (expr, kw, err)
        ran += 1
        boxes += bool(d["tma_x"] or d["tma_xe"]) + bool(d["tma_y"] or d["tma_ye"])
    assert ran >= 12 and boxes >= 16, (ran, boxes)


def test_persistent_tcgen05_kernel_on_blocks_of_larger_matrices(pkg, orc, torch_cuda):
    """Operands and output that are blocks of larger matrices (leading dimensions beyond the extents, shifted bases):
    the boxes' tensor maps carry the pitch, and what lies beside the block -- more k, more rows -- is not read."""
    torch = torch_cuda
    full = "C [a,512,b,640] += sum(c,300) * A [c,a] * B [b,c];"
    c0, a, b = orc.make_inputs(full, 51, "float32")
    sub = "C [a,512,b,384] += sum(c,260) * A [c,a] * B [b,c];"       # b in [64, 448), c in [32, 292)
    oc, oa, ob = 512 * 64, 32, 64 + 640 * 32
    ref = c0.copy()
    orc.contract(sub, ref[oc:], a[oa:], b[ob:], threads=orc.max_threads(), strides={0: [1, 512], 1: [1, 300], 2: [1, 640]})
    assert (ref != c0).any() and (ref[:oc] == c0[:oc]).all()
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    for tma in (0, 1):
        plan = pkg.Plan(sub, pkg.F32, path=pkg.PATH_TCGEN05, tile=(128, 128), variant=2, tma=tma)
        plan.set_strides(pkg.TENSOR_LEFT, [1, 300]).set_strides(pkg.TENSOR_RIGHT, [1, 640])
        d = plan.describe()
        assert d["kernel"] == "tf32wt_128x128" and d["tma_x"] and d["tma_ye"], d
        dc = torch.from_numpy(c0).cuda()
        plan.execute(dc[oc:], da[oa:], db[ob:])
        torch.cuda.synchronize()
        assert plan.status() == 0
        got = dc.cpu().numpy()
        assert orc.rel_error(got, ref) <= TOL["float32"], tma
        assert (got[:oc] == c0[:oc]).all() and (got[oc + 512 * 384:] == c0[oc + 512 * 384:]).all()
        plan.close()


def test_persistent_tcgen05_kernel_wait_that_gives_up(pkg, orc, torch_cuda):
    """The same failure drill as for the fp64 kernels: one loader thread leaves one stage unannounced; every role's
    waits run out, tensor memory is freed, the status names a wait of this kernel, and the next plan runs correctly."""
    torch = torch_cuda
    expr = "C [a,512,b,640] += sum(c,300) * A [a,c] * B [c,b];"
    c0, a, b = orc.make_inputs(expr, 26, "float32")
    ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    kw = dict(path=pkg.PATH_TCGEN05, tile=(128, 128), variant=2)
    bad = pkg.Plan(expr, pkg.F32, test_fault=1, **kw)
    dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
    bad.execute(dc, da, db)
    torch.cuda.synchronize()
    assert bad.status() in range(10, 18)
    bad.close()
    for _ in range(2):   # tensor memory was released: the kernel can be resident again, twice
        good = pkg.Plan(expr, pkg.F32, **kw)
        dc = torch.from_numpy(c0).cuda()
        good.execute(dc, da, db)
        torch.cuda.synchronize()
        assert good.status() == 0 and orc.rel_error(dc.cpu().numpy(), ref) <= TOL["float32"]
        good.close()


def test_persistent_tcgen05_kernel_on_an_unaligned_output(pkg, orc, torch_cuda):
    """An output without 16-byte alignment cannot leave as bulk copies: the same plan runs one CTA per tile, as
    sequential passes where the persistent kernel would have cut the chain itself."""
    torch = torch_cuda
    expr = "C [a,256,b,384] += sum(c,1100) * A [c,a] * B [c,b];"
    c0, a, b = orc.make_inputs(expr, 25, "float32")
    ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    plan = pkg.Plan(expr, pkg.F32, path=pkg.PATH_TCGEN05, tile=(128, 128), variant=2)
    pad = torch.zeros(c0.size + 1, dtype=torch.float32, device="cuda")
    pad[1:] = torch.from_numpy(c0).cuda()
    plan.execute(pad[1:], torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    torch.cuda.synchronize()
    assert plan.status() == 0 and orc.rel_error(pad[1:].cpu().numpy(), ref) <= TOL["float32"]
    plan.close()


@pytest.mark.parametrize("path", ["tcgen05", "mma.sync", "auto"])
def test_fp32_long_contractions_stay_within_tolerance(pkg, orc, torch_cuda, path):
    """Tensor-core fp32 accumulation truncates, so one chain of 8192 products would be off by 7e-5; the planner
    slices the contraction into chains of at most 512 and the combine kernel adds them in round-to-nearest."""
    expr = "C [a,96,b,128] = sum(c,8192) * A [c,a] * B [c,b];"
    kw = {"tcgen05": {"path": pkg.PATH_TCGEN05, "tile": (96, 128)}, "mma.sync": {"path": pkg.PATH_3XTF32, "tile": (96, 128)},
          "auto": {}}[path]
    err, d = _run(pkg, orc, torch_cuda, expr, "float32", 31, **kw)
    assert d["ksplit"] >= 16, d
    assert err <= TOL["float32"], (path, err, d)


@pytest.mark.parametrize("n_b,mode", [(4096, "persistent"), (4096, "slices"), (8192, "passes")])
def test_fp32_long_contractions_on_large_outputs(pkg, orc, torch_cuda, n_b, mode):
    """K = 8192 on outputs of 64 MB and 128 MB.  Under the default path the persistent tcgen05 kernel cuts the chain
    itself (16 segments added into the resident output tile); on the one-CTA-per-tile kernel the planner slices K where
    16 slices fill the 1 GiB of slice scratch exactly and runs 16 sequential passes of 512 products into C where they
    would not fit.  Either way no tensor-core chain is longer than 512 and the result stays inside the fp32 gate."""
    expr = "C [a,4096,b,%d] += sum(c,8192) * A [c,a] * B [c,b];" % n_b
    keep = {}
    kw = {} if mode == "persistent" else {"path": pkg.PATH_TCGEN05, "tile": (128, 128), "variant": 1}
    err = _slab_check(pkg, orc, torch_cuda, expr, "float32", 33, [{"b": 0}, {"b": n_b - 1}, {"b": 1234}, {"a": 4095}], keep=keep, **kw)
    d = keep["desc"]
    keep.clear()
    assert d["math"].startswith("tf32x3") and d["chain"] <= 512, d
    if mode == "persistent":
        assert d["kernel"] == "tf32wt_128x128" and d["ksplit"] == 1 and d["passes"] == 1, d
    elif mode == "slices":
        assert d["kernel"] == "tf32tc_128x128" and d["ksplit"] == 16 and d["passes"] == 1, d
    else:
        assert d["kernel"] == "tf32tc_128x128" and d["passes"] == 16 and d["ksplit"] == 1, d
    assert err <= TOL["float32"], (err, d)


def test_persistent_fp64_kernel_with_k_slices(pkg, orc, torch_cuda):
    """Few output tiles and a long contraction: the planner keeps the persistent fp64 kernel and slices K over its
    CTAs (partial tiles in the plan's workspace, added in slice order by the combine kernel); also on request, with
    ragged tiles, a contraction that is no multiple of the K step, every operator and every loader."""
    err, d = _run(pkg, orc, torch_cuda, "C [a,312,b,296] += sum(c,312,d,96) * A [c,a,d] * B [d,c,b];", "float64", 51)
    assert d["kernel"] == "dmma_ws_128x64" and d["ksplit"] > 1 and d["workspace_bytes"] > 0, d
    assert err <= TOL["float64"], (err, d)
    for expr in ("C [a,200,b,70] -= sum(c,1003) * A [c,a] * B [b,c];",          # 2-D operands: tiled TMA copies
                 "C [a,200,b,70] = sum(c,1003) * A [a,c] * B [c,b];",           # the other way round
                 "C [a,40,b,9,c,30] += sum(d,77,e,13) * A [e,a,d,b] * B [d,c,e];"):   # element gathers
        for split in (2, 5, 64):
            err, d = _run(pkg, orc, torch_cuda, expr, "float64", 52, tile=(128, 64), variant=3, split_k=split)
            assert d["kernel"] == "dmma_ws_128x64" and d["ksplit"] > 1, d
            assert err <= TOL["float64"], (expr, split, err, d)


def test_a_wait_that_gives_up_is_reported_and_the_context_survives(pkg, orc, torch_cuda):
    """Failure detection without a fault: with tc_options.test_fault the persistent kernel's producers leave one
    stage unannounced and waits give up after 2^14 polls.  The kernel must end by itself, the status word must
    name a wait, the host-pointer entry must return TC_ERR_DEVICE_WAIT, and a fresh plan must then run correctly."""
    torch = torch_cuda
    expr = "C [a,256,b,64,c,96] += sum(e,40) * A [e,a,b] * B [e,c];"
    c0, a, b = orc.make_inputs(expr, 91)
    ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    for tile, variant in (((128, 64), 3), ((64, 96), 3), ((128, 64), 4)):
        bad = pkg.Plan(expr, tile=tile, variant=variant, test_fault=1)
        dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
        bad.execute(dc, da, db)
        torch.cuda.synchronize()          # returns: every wait is bounded
        assert bad.status() in (1, 2, 3, 4, 5, 6, 7), "the skipped stage must make a wait give up"
        bad.status_reset()
        assert bad.status() == 0
        bad.close()
        good = pkg.Plan(expr, tile=tile, variant=variant)
        dc = torch.from_numpy(c0).cuda()
        good.execute(dc, da, db)
        torch.cuda.synchronize()
        assert good.status() == 0 and orc.rel_error(dc.cpu().numpy(), ref) <= 1e-12
        good.close()
    # through the host-pointer entry the failure is a status code, not a silent wrong answer
    big = "C [a,256,b,64,c,96,d,4] += sum(e,40) * A [e,a,b] * B [e,c,d];"   # 50 MB of output: slabs over two streams
    c0, a, b = orc.make_inputs(big, 92)
    bad = pkg.Plan(big, tile=(128, 64), variant=3, test_fault=1)
    with pytest.raises(pkg.TcError) as e:
        bad.execute_host(c0.copy(), a, b)
    assert e.value.status == 9
    bad.close()


def test_tcgen05_small_problems_use_the_mma_sync_kernel(pkg):
    d = pkg.Plan("C [a,40,b,40] += sum(c,40) * A [c,a] * B [c,b];", pkg.F32, path=pkg.PATH_TCGEN05).describe()
    assert d["math"] == "tf32x3" and d["kernel"] == "tf32_64x64"


def test_overwrite_ignores_initial_output_even_nan(pkg, orc, torch_cuda):
    torch = torch_cuda
    expr = "C [a,40,b,24] = sum(c,33) * A [c,a] * B [b,c];"
    c0, a, b = orc.make_inputs(expr, 9)
    ref = orc.contract(expr, c0.copy(), a, b)
    for kw in ({}, {"split_k": 2}):
        dc = torch.full((c0.size,), float("nan"), dtype=torch.float64, device="cuda")
        plan = pkg.Plan(expr, **kw)
        plan.execute(dc, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
        torch.cuda.synchronize()
        got = dc.cpu().numpy()
        assert np.isfinite(got).all() and orc.rel_error(got, ref) <= 1e-12


# ------------------------------------------------------- views / alignment ----
def test_strided_slab_of_a_larger_problem(pkg, orc, torch_cuda):
    """One rank's share when an external index is split: strides of the full tensors, shifted bases."""
    torch = torch_cuda
    full = "C [a,24,b,10,c,12] += sum(d,20) * A [d,c,a] * B [b,d];"
    c0, a, b = orc.make_inputs(full, 21)
    ref = orc.contract(full, c0.copy(), a, b)
    dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
    # split b (middle index of C, fastest of B) into [0,4) and [4,10); run both slabs
    for start, count in ((0, 4), (4, 6)):
        plan = pkg.Plan(orc.with_extents(full, {"b": count}))
        plan.set_strides(pkg.TENSOR_OUT, [1, 24, 240]).set_strides(pkg.TENSOR_RIGHT, [1, 10])
        plan.execute(dc[24 * start:], da, db[start:])
        plan.close()
    torch.cuda.synchronize()
    assert orc.rel_error(dc.cpu().numpy(), ref) <= 1e-12


def test_contraction_slab_accumulates(pkg, orc, torch_cuda):
    """Splitting the contraction index: two executes over halves of d accumulate to the full sum."""
    torch = torch_cuda
    full = "C [a,24,b,10,c,12] += sum(d,20) * A [d,c,a] * B [b,d];"
    c0, a, b = orc.make_inputs(full, 22)
    ref = orc.contract(full, c0.copy(), a, b)
    dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
    for start, count in ((0, 12), (12, 8)):
        plan = pkg.Plan(orc.with_extents(full, {"d": count}))
        plan.set_strides(pkg.TENSOR_LEFT, [1, 20, 240]).set_strides(pkg.TENSOR_RIGHT, [1, 10])
        plan.execute(dc, da[start:], db[10 * start:])
        plan.close()
    torch.cuda.synchronize()
    assert orc.rel_error(dc.cpu().numpy(), ref) <= 1e-12


def test_pointers_off_16_byte_alignment(pkg, orc, torch_cuda):
    torch = torch_cuda
    for dt, tdt in (("float64", torch.float64), ("float32", torch.float32)):
        expr = "C [a,32,b,20] += sum(c,24) * A [a,c] * B [c,b];"
        c0, a, b = orc.make_inputs(expr, 5, dt)
        ref = orc.contract(expr, c0.copy(), a, b)
        pad = lambda x: torch.cat([torch.zeros(1, dtype=tdt), torch.from_numpy(x)]).cuda()
        dc, da, db = pad(c0), pad(a), pad(b)
        plan = pkg.Plan(expr, _dt(pkg, dt))
        assert plan.describe()["vec_x"] and plan.describe()["vec_c"] == 4
        plan.execute(dc[1:], da[1:], db[1:])  # every base is one element off a 16-byte boundary
        torch.cuda.synchronize()
        assert orc.rel_error(dc[1:].cpu().numpy(), ref) <= TOL[dt]
        assert dc[0].item() == 0.0
        plan.close()
    # a pointer off the element size is an error, not a fault
    plan = pkg.Plan("C [a,4,b,4] += sum(c,4) * A [a,c] * B [c,b];")
    buf = torch.zeros(64, dtype=torch.float64, device="cuda")
    with pytest.raises(pkg.TcError) as e:
        plan.execute(buf.data_ptr() + 4, buf.data_ptr() + 128, buf.data_ptr() + 256)
    assert e.value.status == 6


# ------------------------------------------------------ K split / workspace ----
def test_k_split_and_caller_workspace(pkg, orc, torch_cuda):
    torch = torch_cuda
    expr = "C [a,33,b,17] += sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];"
    c0, a, b = orc.make_inputs(expr, 7)
    ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    for dt in ("float64",):
        plan = pkg.Plan(expr)
        plan.commit()
        assert plan.describe()["ksplit"] > 1 and plan.launches == 2
        need = plan.workspace_bytes()
        assert need > 0
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        dc = torch.from_numpy(c0).cuda()
        plan.execute(dc, da, db)  # plan-owned workspace
        dc2 = torch.from_numpy(c0).cuda()
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        plan.execute(dc2, da, db, workspace=ws)  # caller's workspace
        torch.cuda.synchronize()
        assert orc.rel_error(dc.cpu().numpy(), ref) <= 1e-12
        assert np.array_equal(dc.cpu().numpy(), dc2.cpu().numpy())  # slices are combined in a fixed order
        small = torch.empty(need - 16, dtype=torch.uint8, device="cuda")
        with pytest.raises(pkg.TcError) as e:
            plan.execute(dc2, da, db, workspace=small)
        assert e.value.status == 8
        plan.close()


# ----------------------------------------------------------- host pointers ----
def test_host_pointer_execute(pkg, orc, torch_cuda):
    for dt in ("float64", "float32"):
        expr = "t3 [a,20,b,6,c,14] += sum(d,18) * t2 [d,c,a] * v2 [b,d];"
        c0, a, b = orc.make_inputs(expr, 31, dt)
        ref = orc.contract(expr, c0.copy(), a, b)
        c = c0.copy()
        plan = pkg.Plan(expr, _dt(pkg, dt))
        plan.execute_host(c, a, b)
        assert orc.rel_error(c, ref) <= TOL[dt]
        plan.close()


def test_host_pointer_execute_pipelined_slabs(pkg, orc, torch_cuda):
    """Outputs of 32 MB and more travel slab by slab along the output's slowest index over two streams."""
    cases = [
        "C [a,128,b,96,c,40,d,10] += sum(e,6) * A [a,e,b,d] * B [e,c];",      # left input sliced with the output
        "C [a,128,b,96,c,40,d,11] -= sum(e,6) * A [d,e,a] * B [e,c,b];",      # cut index fastest in the left input
        "C [a,128,b,96,c,40,d,9] = sum(e,6) * A [e,b,a] * B [c,e,d];",        # right input sliced, overwrite, short last slab
    ]
    for expr in cases:
        c0, a, b = orc.make_inputs(expr, 61)
        ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
        plan = pkg.Plan(expr)
        c = c0.copy()
        plan.execute_host(c, a, b)
        assert orc.rel_error(c, ref) <= 1e-12, expr
        if " = " not in expr:  # a second pass through the cached buffers and slab plans accumulates again
            ref2 = orc.contract(expr, ref.copy(), a, b, threads=orc.max_threads())
            plan.execute_host(c, a, b)
            assert orc.rel_error(c, ref2) <= 1e-12, expr
        plan.close()


def test_host_pointer_execute_page_locked_slabs(pkg, orc, torch_cuda):
    """Page-locked host buffers: copies in, kernels and copies out run on three streams chained by events, slab by slab."""
    torch = torch_cuda
    cases = [
        "C [a,128,b,96,c,40,d,10] += sum(e,6) * A [a,e,b,d] * B [e,c];",
        "C [a,128,b,96,c,40,d,11] -= sum(e,6) * A [d,e,a] * B [e,c,b];",
        "C [a,128,b,96,c,40,d,9] = sum(e,6) * A [e,b,a] * B [c,e,d];",
    ]
    for expr in cases:
        c0, a, b = orc.make_inputs(expr, 62)
        ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
        pinned = [torch.from_numpy(x).pin_memory() for x in (c0, a, b)]
        c, pa, pb = (t.numpy() for t in pinned)
        plan = pkg.Plan(expr)
        plan.execute_host(c, pa, pb)
        assert orc.rel_error(c, ref) <= 1e-12, expr
        if " = " not in expr:
            ref2 = orc.contract(expr, ref.copy(), a, b, threads=orc.max_threads())
            plan.execute_host(c, pa, pb)
            assert orc.rel_error(c, ref2) <= 1e-12, expr
        # a mixed call (page-locked output, pageable inputs) takes the staged path and gives the same answer
        c2 = torch.from_numpy(c0).pin_memory().numpy()
        plan.execute_host(c2, a, b)
        assert orc.rel_error(c2, ref) <= 1e-12, expr
        plan.close()


def test_extents_overridden_at_run_time(pkg, orc, torch_cuda):
    """The sizes written in the expression are only representative, as in the reference drivers."""
    torch = torch_cuda
    written = "t3 [a,16,b,16,c,16] += sum(d,16) * t2 [d,c,a] * v2 [b,d];"
    ext = {"a": 40, "b": 9, "c": 21, "d": 33}
    actual = orc.with_extents(written, ext)
    c0, a, b = orc.make_inputs(actual, 3)
    ref = orc.contract(actual, c0.copy(), a, b)
    plan = pkg.Plan(written, extents=ext)
    dc = torch.from_numpy(c0).cuda()
    plan.execute(dc, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    torch.cuda.synchronize()
    assert orc.rel_error(dc.cpu().numpy(), ref) <= 1e-12
    with pytest.raises(pkg.TcError) as e:
        plan.set_extents({"a": 2})  # committed plans are immutable
    assert e.value.status == 7


# ------------------------------------------------------------- properties ----
def test_two_streams_and_repeated_accumulation(pkg, orc, torch_cuda):
    """Linearity at a size the checker would not finish: C2 - C1 == C1 - C0, on two streams at once."""
    torch = torch_cuda
    expr = CONFIGS[1][0].replace("96", "48")
    nc, na, nb = orc.sizes(expr)
    outs = []
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    plan = pkg.Plan(expr).commit()
    bufs = []
    for s, seed in zip(streams, (1, 2)):
        with torch.cuda.stream(s):
            dc = torch.empty(nc, dtype=torch.float64, device="cuda")
            da = torch.empty(na, dtype=torch.float64, device="cuda")
            db = torch.empty(nb, dtype=torch.float64, device="cuda")
            for t, tid in ((dc, 0), (da, 1), (db, 2)):
                pkg.fill_uniform(t, seed, tid, stream=s.cuda_stream)
            c0 = dc.clone()
            plan.execute(dc, da, db, stream=s.cuda_stream)
            c1 = dc.clone()
            plan.execute(dc, da, db, stream=s.cuda_stream)
            bufs.append((c0, c1, dc, da, db))
    torch.cuda.synchronize()
    for c0, c1, c2, da, db in bufs:
        d1, d2 = (c1 - c0), (c2 - c1)
        scale = d1.abs().max().item()
        assert scale > 1.0 and (d1 - d2).abs().max().item() <= 1e-12 * scale
    plan.close()
