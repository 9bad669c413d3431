"""One contraction over several GPUs from one process through the C entry (tc_plan_create_sharded /
tc_execute_sharded): the geometry against the host logic of shard.py on CPU, execution against the loop nest on GPUs."""
import importlib
import random

import numpy as np
import pytest

from test_parser import _random_expr


@pytest.fixture(scope="module")
def shard(pkg):
    return importlib.import_module("cgo2019_ae_b200.shard")


EXPRS = [
    "C [a,40,b,40,c,40,d,40,e,40,f,40] += sum(g,40) * A [g,a,b,c] * B [d,e,f,g];",
    "C [a,33,b,17] -= sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];",
    "t3 [a,312,b,24,c,296] += sum(d,312) * t2 [d,c,a] * v2 [b,d];",
    "C [i,5,j,3] = sum(k,2) * A [k,i] * B [j,k];",
]


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_geometry_through_the_c_entry_matches_the_host_logic(pkg, shard, world):
    rng = random.Random(world)
    for expr in EXPRS + [_random_expr(rng) for _ in range(20)]:
        p = pkg.parse(expr)
        for kind, choose in ((pkg.SHARD_EXTERNAL, shard.choose_external_index), (pkg.SHARD_CONTRACTION, shard.choose_contraction_index)):
            if kind == pkg.SHARD_CONTRACTION and not p["sum_idx"]:
                continue
            d = pkg.ShardedPlan(expr, pkg.F64, devices=list(range(world)), kind=kind).describe()
            index = choose(p)
            assert d["index"] == index and d["kind"] == ("external" if kind == pkg.SHARD_EXTERNAL else "contraction"), (expr, d)
            for r in range(world):
                g = shard.ShardGeometry(expr, index, r, world)
                s = d["shards"][r]
                assert (s["start"], s["count"], s["empty"]) == (g.start, g.count, g.empty), (expr, r)
                assert s["offsets"] == g.offsets and d["strides"] == g.strides and d["full_sizes"] == g.full_sizes
                if kind == pkg.SHARD_EXTERNAL:
                    assert s["local_expr"] == g.local_expr and d["c_slab_contiguous"] == g.c_slab_contiguous
                else:
                    assert " = sum(" in s["local_expr"]
            if kind == pkg.SHARD_CONTRACTION:
                sh = shard.ContractionShard(expr, pkg.F64, 0, world)
                assert d["chunk"] == sh.chunk and d["padded"] == sh.padded
                assert d["shards"][0]["local_expr"] == sh.partial_expr


def test_argument_errors(pkg):
    expr = EXPRS[1]
    with pytest.raises(pkg.TcError) as e:
        pkg.ShardedPlan(expr, pkg.F64, devices=[0, 1], kind=pkg.SHARD_EXTERNAL, index="c").describe()   # c is contracted
    assert e.value.status == 2
    with pytest.raises(pkg.TcError):
        pkg.ShardedPlan(expr, pkg.F64, devices=[0, 1], kind=pkg.SHARD_CONTRACTION, index="a").describe()
    with pytest.raises(pkg.TcError):
        pkg.ShardedPlan(expr, pkg.F64, devices=[], kind=pkg.SHARD_EXTERNAL)
    with pytest.raises(pkg.TcError):
        pkg.ShardedPlan("nonsense", pkg.F64, devices=[0])
    # extents can be replaced before commit; an explicit index is honoured
    sp = pkg.ShardedPlan(expr, pkg.F64, devices=[0, 1], kind=pkg.SHARD_EXTERNAL, index="a", extents={"a": 64})
    d = sp.describe()
    assert d["index"] == "a" and [s["count"] for s in d["shards"]] == [32, 32] and not d["c_slab_contiguous"]
    # executing an uncommitted plan is a state error, not a crash
    with pytest.raises(pkg.TcError) as e:
        sp.execute([0, 0], [0, 0], [0, 0])
    assert e.value.status == 7


def _devices(torch, want):
    n = torch.cuda.device_count()
    return list(range(min(n, want)))


@pytest.mark.gpu
@pytest.mark.parametrize("want", [1, 2])
def test_both_splits_on_the_gpus_of_this_process(pkg, orc, want):
    """Every device holds the full tensors; after the call device d's slab (external kind) or chunk (contraction kind)
    of its output holds the loop nest's values.  With one visible GPU the two-device case runs both shards on it."""
    import torch
    assert torch.cuda.is_available()
    devs = _devices(torch, want)
    if len(devs) < want:
        devs = [0] * want   # two shards on one GPU: still two plans and two streams (external kind only)
    cases = [
        ("C [a,64,b,48,c,40,d,12] += sum(e,56) * A [e,a,c] * B [d,b,e];", pkg.SHARD_EXTERNAL, "float64", 1e-12),
        ("C [a,96,b,8,c,64,d,10] -= sum(e,24) * A [e,a,b] * B [c,d,e];", pkg.SHARD_EXTERNAL, "float32", 1e-5),
        ("C [a,33,b,17] -= sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];", pkg.SHARD_CONTRACTION, "float64", 1e-12),
        ("C [a,40,b,24] = sum(c,600) * A [c,a] * B [b,c];", pkg.SHARD_CONTRACTION, "float64", 1e-12),
    ]
    for expr, kind, dt, tol in cases:
        if kind == pkg.SHARD_CONTRACTION and len(set(devs)) != len(devs):
            continue   # NCCL wants distinct devices per communicator rank
        c0, a, b = orc.make_inputs(expr, 71, dt)
        ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
        sp = pkg.ShardedPlan(expr, pkg.F64 if dt == "float64" else pkg.F32, devices=devs, kind=kind).commit()
        d = sp.describe()
        cs = [torch.from_numpy(c0).cuda(dev) for dev in devs]
        das = [torch.from_numpy(a).cuda(dev) for dev in devs]
        dbs = [torch.from_numpy(b).cuda(dev) for dev in devs]
        for dev in set(devs):
            torch.cuda.synchronize(dev)
        sp.execute(cs, das, dbs)
        sp.synchronize()
        got = c0.copy()
        if kind == pkg.SHARD_EXTERNAL:
            # device r wrote the values of the cut index's range r; gather them from the strided slabs
            idx = pkg.parse(expr)["out_idx"]
            ext = dict(zip(idx, pkg.parse(expr)["out_ext"]))
            shape = [ext[i] for i in reversed(idx)]
            axis = len(idx) - 1 - idx.index(d["index"])
            full = got.reshape(shape)
            for r, s in enumerate(d["shards"]):
                sl = [slice(None)] * len(shape)
                sl[axis] = slice(s["start"], s["start"] + s["count"])
                full[tuple(sl)] = cs[r].cpu().numpy().reshape(shape)[tuple(sl)]
        else:
            for r in range(len(devs)):
                lo = min(r * d["chunk"], c0.size)
                hi = min(lo + d["chunk"], c0.size)
                got[lo:hi] = cs[r].cpu().numpy()[lo:hi]
        assert orc.rel_error(got, ref) <= tol, (expr, len(devs))
        sp.close()
