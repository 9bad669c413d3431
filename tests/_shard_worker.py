"""One rank of the world_size-2 host-logic test (gloo, CPU).  The contraction itself is done by the CPU
checker here: the point is the sharding arithmetic (extents, strides, offsets, chunks) and the exchange."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg, orc = entry.load_package(), entry.load_oracle()
    import importlib
    shard = importlib.import_module("cgo2019_ae_b200.shard")

    # ---- external split: slowest output index (contiguous slabs), a middle one, and one with remainder ----
    expr = "C [a,6,b,5,c,4,d,7] += sum(e,5,f,3) * A [e,c,a,f] * B [b,f,d,e];"
    c0, a, b = orc.make_inputs(expr, 17)
    want = orc.contract(expr, c0.copy(), a, b)
    for index in (None, "b", "d", "a"):
        sh = shard.ExternalShard(expr, pkg.F64, rank, world, index=index)
        g = sh.geom
        assert g.kind == "external"
        if index is None:
            assert g.index == "d" and g.c_slab_contiguous  # largest, and slowest-varying
        mine = c0.copy()
        if not g.empty:
            orc.contract(g.local_expr, mine[g.offsets[0]:], a[g.offsets[1]:], b[g.offsets[2]:],
                         strides={0: g.strides[0], 1: g.strides[1], 2: g.strides[2]})
            d = sh.plan.describe()  # the product's planner accepts the same geometry
            assert d["Mflat"] * d["Nflat"] == g.c_slab_elems
        touched = mine != c0
        owned = torch.from_numpy(np.where(touched, mine, 0.0))
        count = torch.from_numpy(touched.astype(np.int32))
        dist.all_reduce(owned)
        dist.all_reduce(count)
        assert (count.numpy() == 1).all(), index  # every element belongs to exactly one rank
        assert np.array_equal(owned.numpy(), want), index
        if g.c_slab_contiguous:
            lo = g.offsets[0]
            assert np.array_equal(mine[lo:lo + g.c_slab_elems], want[lo:lo + g.c_slab_elems])
        sh.close()

    # ---- contraction split + exchange ----
    for op in ("+=", "-=", "="):
        e2 = expr.replace("+=", op)
        want = orc.contract(e2, c0.copy(), a, b)
        sh = shard.ContractionShard(e2, pkg.F64, rank, world)
        g = sh.geom
        assert g.kind == "contraction" and g.index == "e"
        partial = np.zeros(sh.padded)
        orc.contract(sh.partial_expr, partial, a[g.offsets[1]:], b[g.offsets[2]:],
                     strides={1: g.strides[1], 2: g.strides[2]})
        c = torch.from_numpy(c0.copy())
        sh.combine(c, torch.from_numpy(partial))
        lo, hi = sh.chunk_range()
        err = np.abs(c.numpy()[lo:hi] - want[lo:hi]).max() / np.abs(want).max()
        assert err <= 1e-12, (op, err)
        other = np.ones(c0.size, dtype=bool)
        other[lo:hi] = False
        assert np.array_equal(c.numpy()[other], c0[other])  # only this rank's chunk is written
        sh.close()

    # ---- more ranks than index values: idle ranks are legal ----
    g = shard.ShardGeometry("C [a,4,b,1] += sum(c,3) * A [c,a] * B [b,c];", "b", rank, world)
    assert g.empty == (rank > 0)
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
