"""Splitting one contraction over the GPUs of a box (one process per GPU).

The reference is single-GPU (one stream, one device, nwchem-tccg/tccg_kernels.cu:228
is the only stream it ever creates); this layer has no counterpart there.

Two splits, both expressed as strided views of the FULL tensors, so no data is
repacked:

* external split -- an index of the output is cut into contiguous ranges, one
  per rank.  Every output element is an independent sum, so there is no
  exchange at all: each rank runs the same kernels on its slab.  When the cut
  index is the output's slowest one, a rank's slab of C is one contiguous block
  and the rank may hold only that block.
* contraction split -- a contraction index is cut; each rank computes a full-size
  partial result into scratch, one reduce-scatter (NCCL over NVLink) leaves each
  rank with the summed 1/world chunk, which is then added into its chunk of C.

Geometry (extents, strides, offsets) is pure host arithmetic and is what the
CPU tests check; execution goes through the C-ABI library like everything else.
"""
from . import F64, F32, TENSOR_OUT, TENSOR_LEFT, TENSOR_RIGHT, Plan, parse, axpy


def split_range(extent, parts, rank):
    """Contiguous [start, start+count) of `extent` for `rank` of `parts`; the first extent%parts ranks get one more."""
    if parts <= 0 or not (0 <= rank < parts):
        raise ValueError("bad rank/parts")
    base, rem = divmod(extent, parts)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def _rewrite(parsed, extents):
    oe = [extents[i] for i in parsed["out_idx"]]
    se = [extents[i] for i in parsed["sum_idx"]]
    return "%s [%s] %s sum(%s) * %s [%s] * %s [%s];" % (
        parsed["out"], ",".join("%s,%d" % x for x in zip(parsed["out_idx"], oe)), parsed["op"],
        ",".join("%s,%d" % x for x in zip(parsed["sum_idx"], se)), parsed["left"], ",".join(parsed["left_idx"]),
        parsed["right"], ",".join(parsed["right_idx"]))


def _compact_strides(idx, extents):
    out, acc = [], 1
    for i in idx:
        out.append(acc)
        acc *= extents[i]
    return out


def choose_external_index(parsed):
    """Largest output index; ties go to the slowest-varying one (its slabs of C are contiguous)."""
    ext = dict(zip(parsed["out_idx"], parsed["out_ext"]))
    best = None
    for pos, name in enumerate(parsed["out_idx"]):
        if best is None or ext[name] >= ext[best[1]]:
            best = (pos, name)
    return best[1]


def choose_contraction_index(parsed):
    ext = dict(zip(parsed["sum_idx"], parsed["sum_ext"]))
    return max(parsed["sum_idx"], key=lambda n: ext[n])


class ShardGeometry:
    """What one rank computes: a local expression plus views into the full tensors."""

    def __init__(self, expr, index, rank, world, extents=None):
        p = parse(expr)
        full = dict(zip(p["out_idx"] + p["sum_idx"], p["out_ext"] + p["sum_ext"]))
        if extents:
            full.update(extents)
        if index not in full:
            raise ValueError("unknown index %r" % index)
        self.parsed, self.index, self.rank, self.world = p, index, rank, world
        self.kind = "external" if index in p["out_idx"] else "contraction"
        self.full_extents = full
        self.start, self.count = split_range(full[index], world, rank)
        local = dict(full)
        local[index] = max(self.count, 1)
        self.local_extents = local
        self.empty = self.count == 0  # more ranks than index values: this rank has nothing to do
        self.local_expr = _rewrite(p, local)
        self.full_expr = _rewrite(p, full)
        tensors = (p["out_idx"], p["left_idx"], p["right_idx"])
        self.strides = [_compact_strides(t, full) for t in tensors]          # strides of the FULL tensors
        self.offsets = [self.start * s[t.index(index)] if index in t else 0  # element offset of this rank's view
                        for t, s in zip(tensors, self.strides)]
        self.full_sizes = [_prod(full[i] for i in t) for t in tensors]
        # The slab of C is one contiguous block iff the cut index is C's slowest (or C is not cut at all).
        self.c_slab_contiguous = self.kind == "external" and (p["out_idx"][-1] == index or world == 1)
        self.c_slab_elems = _prod(local[i] for i in p["out_idx"])

    def make_plan(self, dtype=F64, **kw):
        plan = Plan(self.local_expr, dtype, **kw)
        for t in (TENSOR_OUT, TENSOR_LEFT, TENSOR_RIGHT):
            plan.set_strides(t, self.strides[t])
        return plan


def _prod(it):
    r = 1
    for x in it:
        r *= x
    return r


def _view(t, offset):
    """Tensor (or raw address) shifted by `offset` elements."""
    if offset == 0:
        return t
    if isinstance(t, int):
        raise TypeError("raw addresses must be shifted by the caller")
    return t[offset:]


class ExternalShard:
    """Rank-local share of a contraction cut along an output index.  No communication."""

    def __init__(self, expr, dtype=F64, rank=0, world=1, index=None, extents=None, **plan_kw):
        idx = index or choose_external_index(parse(expr))
        self.geom = ShardGeometry(expr, idx, rank, world, extents)
        if self.geom.kind != "external":
            raise ValueError("%r is not an output index" % idx)
        self.plan = None if self.geom.empty else self.geom.make_plan(dtype, **plan_kw)

    def execute(self, C, A, B, stream=None, c_is_slab=False):
        """A, B: full input tensors (flat).  C: the full output, or -- with c_is_slab and a cut along the
        output's slowest index -- only this rank's contiguous slab."""
        g = self.geom
        if g.empty:
            return
        if c_is_slab and not g.c_slab_contiguous:
            raise ValueError("a rank-local C slab is only contiguous when the slowest output index is cut")
        c = C if c_is_slab else _view(C, g.offsets[0])
        self.plan.execute(c, _view(A, g.offsets[1]), _view(B, g.offsets[2]), stream=stream)

    def cost(self):
        return (0.0, 0.0) if self.geom.empty else self.plan.cost()

    def close(self):
        if self.plan:
            self.plan.close()


class ContractionShard:
    """Rank-local share of a contraction cut along a contraction index, combined by one reduce-scatter.

    After execute(), rank r's chunk [r*n, (r+1)*n) of the flat output (n = ceil(|C|/world)) holds the
    final values; the other chunks of that rank's C are untouched."""

    def __init__(self, expr, dtype=F64, rank=0, world=1, index=None, extents=None, **plan_kw):
        p = parse(expr)
        idx = index or choose_contraction_index(p)
        self.geom = ShardGeometry(expr, idx, rank, world, extents)
        if self.geom.kind != "contraction":
            raise ValueError("%r is not a contraction index" % idx)
        self.dtype = dtype
        self.sign = -1.0 if p["op"] == "-=" else 1.0
        self.overwrite = p["op"] == "="
        # every rank writes its partial sum with '=' into scratch
        q = dict(self.geom.parsed)
        q["op"] = "="
        self.partial_expr = _rewrite(q, self.geom.local_extents)
        self.plan = None
        if not self.geom.empty:
            self.plan = Plan(self.partial_expr, dtype, **plan_kw)
            for t in (TENSOR_LEFT, TENSOR_RIGHT):
                self.plan.set_strides(t, self.geom.strides[t])
        n = self.geom.full_sizes[0]
        self.chunk = -(-n // world)
        self.padded = self.chunk * world
        self._partial = None
        self._reduced = None

    def chunk_range(self):
        n = self.geom.full_sizes[0]
        lo = min(self.geom.rank * self.chunk, n)
        return lo, min(lo + self.chunk, n)

    def execute(self, C, A, B, group=None, stream=None):
        import contextlib
        import torch
        g = self.geom
        # The kernels run on `stream`; the collective and the copies around it are torch operations and run on
        # torch's current stream.  Make the two the same stream, or the exchange could read the partial result
        # before the kernel has written it.
        ctx = contextlib.nullcontext()
        if stream and C.is_cuda and stream != torch.cuda.current_stream(C.device).cuda_stream:
            ctx = torch.cuda.stream(torch.cuda.ExternalStream(stream, device=C.device))
        with ctx:
            if self._partial is None:
                self._partial = torch.zeros(self.padded, dtype=C.dtype, device=C.device)
            if g.empty:
                self._partial.zero_()
            else:
                self.plan.execute(self._partial, _view(A, g.offsets[1]), _view(B, g.offsets[2]), stream=stream)
            self.combine(C, self._partial, group=group, stream=stream)

    def combine(self, C, partial, group=None, stream=None):
        """The exchange step: sum the ranks' partial outputs, add this rank's chunk into C.

        `partial` has `self.padded` elements.  On CUDA tensors the reduce-scatter is NCCL's and the add is
        the library's axpy kernel; CPU tensors (host-logic tests over gloo, which has no reduce-scatter)
        take an all-reduce and a torch add."""
        import torch
        import torch.distributed as dist
        g = self.geom
        if self._reduced is None:
            self._reduced = torch.empty(self.chunk, dtype=C.dtype, device=C.device)
        if dist.get_backend(group) == "nccl":
            dist.reduce_scatter_tensor(self._reduced, partial, op=dist.ReduceOp.SUM, group=group)
        else:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
            self._reduced.copy_(partial[g.rank * self.chunk:(g.rank + 1) * self.chunk])
        lo, hi = self.chunk_range()
        if hi > lo:
            mine = C[lo:hi]
            if self.overwrite:
                mine.copy_(self._reduced[:hi - lo])
            elif mine.is_cuda:
                axpy(mine, self._reduced[:hi - lo], self.sign, stream=stream)
            else:
                mine.add_(self._reduced[:hi - lo], alpha=self.sign)

    def close(self):
        if self.plan:
            self.plan.close()
