"""One rank of the multi-GPU test of the sharded paths: NCCL, one GPU per rank, the CUDA kernels do the work and the
CPU checker verifies the result.  Ranks leave only after a final barrier, with nothing in flight."""
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
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pkg, orc = entry.load_package(), entry.load_oracle()
    import importlib
    shard = importlib.import_module("cgo2019_ae_b200.shard")

    # ---- external split: every rank computes its slab of C on its own GPU; no communication on the data path ----
    expr = "C [a,48,b,40,c,24,d,36] += sum(e,24,f,6) * A [e,c,a,f] * B [b,f,d,e];"
    c0, a, b = orc.make_inputs(expr, 17)
    want = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    for index in (None, "b"):
        sh = shard.ExternalShard(expr, pkg.F64, rank, world, index=index)
        dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
        sh.execute(dc, da, db)
        torch.cuda.synchronize()
        assert sh.plan.status() == 0
        mine = dc.cpu().numpy()
        touched = mine != c0
        owned = torch.from_numpy(np.where(touched, mine, 0.0)).cuda()
        count = torch.from_numpy(touched.astype(np.int32)).cuda()
        dist.all_reduce(owned)
        dist.all_reduce(count)
        assert int(count.max()) <= 1, index                      # no element is written by two ranks
        got = np.where(count.cpu().numpy() == 1, owned.cpu().numpy(), c0)
        err = np.abs(got - want).max() / np.abs(want).max()
        assert err <= 1e-12, (index, err)
        sh.close()

    # ---- contraction split: partial products per GPU, one NCCL reduce-scatter, axpy of the rank's chunk ----
    for op in ("+=", "-=", "="):
        e2 = "C [a,96,b,80] %s sum(c,4000,d,6) * A [a,c,d] * B [d,b,c];" % op
        c0, a, b = orc.make_inputs(e2, 23)
        want = orc.contract(e2, c0.copy(), a, b, threads=orc.max_threads())
        sh = shard.ContractionShard(e2, pkg.F64, rank, world)
        assert sh.geom.index == "c"
        dc, da, db = (torch.from_numpy(x).cuda() for x in (c0, a, b))
        sh.execute(dc, da, db)
        torch.cuda.synchronize()
        lo, hi = sh.chunk_range()
        got = dc.cpu().numpy()
        err = np.abs(got[lo:hi] - want[lo:hi]).max() / np.abs(want).max()
        assert err <= 1e-12, (op, err)
        other = np.ones(c0.size, dtype=bool)
        other[lo:hi] = False
        assert np.array_equal(got[other], c0[other]), op        # only this rank's chunk is written
        sh.close()

    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
