"""Multi-GPU host logic on CPU: range splitting, shard geometry, and the exchange over gloo (world size 2)."""
import importlib
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def shard(pkg):
    return importlib.import_module("cgo2019_ae_b200.shard")


def test_split_range_covers_everything_once(shard):
    for extent in (1, 5, 40, 41, 64000):
        for parts in (1, 2, 3, 4, 8):
            seen = []
            for r in range(parts):
                s, c = shard.split_range(extent, parts, r)
                seen += list(range(s, s + c))
            assert seen == list(range(extent))
    assert [shard.split_range(40, 8, r) for r in (0, 7)] == [(0, 5), (35, 5)]
    with pytest.raises(ValueError):
        shard.split_range(4, 2, 2)


def test_large_configuration_shards_along_its_slowest_index(shard):
    expr = "C [a,40,b,40,c,40,d,40,e,40,f,40] += sum(g,40) * A [g,a,b,c] * B [d,e,f,g];"
    for world in (1, 2, 4, 8):
        offs = []
        for r in range(world):
            g = shard.ShardGeometry(expr, shard.choose_external_index(shard.parse(expr)), r, world)
            assert g.index == "f" and g.c_slab_contiguous and g.count == 40 // world
            assert g.offsets[1] == 0                         # A is replicated
            assert g.offsets[2] == g.start * 1600            # B[d,e,f,g] is sliced on its third index
            assert g.offsets[0] == g.start * 40 ** 5         # contiguous slab of C
            assert g.c_slab_elems == 40 ** 5 * g.count
            assert g.strides[2] == [1, 40, 1600, 64000]      # strides of the FULL right operand
            offs.append(g.offsets[0])
            d = g.make_plan().describe()
            assert d["Nflat"] == 1600 * g.count and d["Mflat"] == 64000
        assert offs == sorted(offs)


def test_contraction_split_geometry(shard, pkg):
    expr = "C [a,33,b,17] -= sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];"
    sh = [shard.ContractionShard(expr, pkg.F64, r, 4) for r in range(4)]
    assert all(s.geom.index == "c" and s.geom.count == 250 for s in sh)
    assert [s.geom.offsets[1] for s in sh] == [r * 250 * 33 for r in range(4)]
    assert [s.geom.offsets[2] for s in sh] == [r * 250 * 9 * 17 for r in range(4)]
    assert all(s.sign == -1.0 and " = sum(" in s.partial_expr for s in sh)
    assert sh[0].chunk * 4 >= 33 * 17 and sh[3].chunk_range()[1] == 33 * 17


def test_two_ranks_over_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "_shard_worker.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "rank %d ok" % rank in out, out[-3000:]


@pytest.mark.gpu
def test_sharded_paths_on_two_gpus_over_nccl():
    """External slabs and the contraction split with NCCL's reduce-scatter, one process per GPU (needs two GPUs)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "_shard_worker_gpu.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "rank %d ok" % rank in out, out[-3000:]
