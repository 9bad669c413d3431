"""Host-side mirror of the contraction operator over the C-ABI library.

The reference is driven by one expression line per contraction
(``t3 [a,312,b,24,c,296] += sum(d,312) * t2 [d,c,a] * v2 [b,d];``,
cogent/input_strings/tccg/input_tccg_02.in:4) that ``tc_code_generator.py``
turns into a ``.cu`` file with the entry ``sd_t_d2_fusion_``
(cogent/src/codes/kernels/tc_interface.py:1444-1598).  Here the same line makes
a :class:`Plan`; ``Plan.execute`` enqueues the hand-written sm_100a kernels on
device tensors.  Everything numeric happens inside ``libtc_b200.so``; there is
no Python or CPU compute path, and a missing library is an error.
"""
import ctypes
import json
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtc_b200.so")

F64, F32 = 0, 1
PATH_AUTO, PATH_DMMA, PATH_DFMA, PATH_FFMA, PATH_3XTF32, PATH_TCGEN05 = 0, 1, 2, 3, 4, 5
TENSOR_OUT, TENSOR_LEFT, TENSOR_RIGHT = 0, 1, 2

PROBES_PATH = os.path.join(_HERE, "probes", "libtc_probes.so")
PEAK_NAMES = {0: "dmma_m8n8k4", 1: "dmma_m16n8k4", 2: "dmma_m16n8k8", 3: "dmma_m16n8k16",
              4: "dfma", 5: "ffma", 6: "tf32_mma_sync", 7: "tf32_tcgen05"}


class TcError(RuntimeError):
    def __init__(self, status, where, detail=""):
        self.status = status
        msg = "%s failed: %s (status %d)" % (where, _status_string(status), status)
        if detail:
            msg += " -- " + detail
        super().__init__(msg)


class Options(ctypes.Structure):
    _fields_ = [("path", ctypes.c_int), ("tile_m", ctypes.c_int), ("tile_n", ctypes.c_int),
                ("split_k", ctypes.c_int), ("variant", ctypes.c_int), ("l2_prefetch", ctypes.c_int),
                ("c_path", ctypes.c_int), ("tma", ctypes.c_int), ("test_fault", ctypes.c_int)]


_lib = None

# name -> (restype, argtypes); every symbol include/tc_b200.h declares.
_SIGNATURES = {
    "tc_plan_create_sharded": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                              ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "tc_sharded_set_extents": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                              ctypes.POINTER(ctypes.c_int64)]),
    "tc_sharded_describe": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]),
    "tc_sharded_commit": (ctypes.c_int, [ctypes.c_void_p]),
    "tc_execute_sharded": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                          ctypes.POINTER(ctypes.c_void_p), ctypes.c_int]),
    "tc_sharded_synchronize": (ctypes.c_int, [ctypes.c_void_p]),
    "tc_sharded_destroy": (None, [ctypes.c_void_p]),
    "tc_expr_describe": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t]),
    "tc_plan_create": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(Options),
                                      ctypes.POINTER(ctypes.c_void_p)]),
    "tc_plan_set_extents": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                           ctypes.POINTER(ctypes.c_int64)]),
    "tc_plan_set_extents_ordered": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int64)]),
    "tc_sd_t_d2_fusion": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "tc_plan_set_strides": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                           ctypes.POINTER(ctypes.c_int64)]),
    "tc_plan_commit": (ctypes.c_int, [ctypes.c_void_p]),
    "tc_plan_destroy": (None, [ctypes.c_void_p]),
    "tc_plan_describe": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]),
    "tc_plan_cost": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_double),
                                    ctypes.POINTER(ctypes.c_double)]),
    "tc_plan_launches": (ctypes.c_int, [ctypes.c_void_p]),
    "tc_plan_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]),
    "tc_plan_status_reset": (ctypes.c_int, [ctypes.c_void_p]),
    "tc_plan_workspace_bytes": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_size_t)]),
    "tc_execute": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                  ctypes.c_void_p]),
    "tc_execute_ws": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "tc_execute_noalloc": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_void_p]),
    "tc_plan_create_fused": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_char_p), ctypes.c_int,
                                            ctypes.POINTER(ctypes.c_void_p)]),
    "tc_fused_set_extents": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                            ctypes.POINTER(ctypes.c_int64)]),
    "tc_fused_commit": (ctypes.c_int, [ctypes.c_void_p]),
    "tc_fused_describe": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]),
    "tc_execute_fused": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                        ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]),
    "tc_fused_destroy": (None, [ctypes.c_void_p]),
    "tc_execute_host": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "tc_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "tc_last_cuda_error": (ctypes.c_char_p, []),
    "tc_version": (ctypes.c_char_p, []),
    "tc_fill_uniform": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint64,
                                       ctypes.c_int, ctypes.c_int64, ctypes.c_void_p]),
    "tc_axpy": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                               ctypes.c_double, ctypes.c_void_p]),
}


def exported_symbols():
    return sorted(_SIGNATURES)


def lib():
    """The loaded C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: run `python %s` (or __graft_entry__.build()) first; "
                              "there is no fallback path" % (LIB_PATH, os.path.join(_HERE, "build.py")))
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def _status_string(status):
    try:
        return lib().tc_status_string(status).decode()
    except Exception:  # pragma: no cover - library missing
        return "?"


def _check(status, where):
    if status != 0:
        detail = lib().tc_last_cuda_error().decode() if status == 5 else ""
        raise TcError(status, where, detail)


def parse(expr):
    """Parsed form of one expression line (dict), or raises TcError(status 1 / 3)."""
    buf = ctypes.create_string_buffer(8192)
    st = lib().tc_expr_describe(expr.encode(), buf, len(buf))
    if st != 0:
        raise TcError(st, "tc_expr_describe", json.loads(buf.value.decode() or "{}").get("error", ""))
    return json.loads(buf.value.decode())


def _stream(stream, *tensors):
    """cudaStream_t for a call: the caller's, else torch's current stream when the arguments are torch CUDA tensors
    (so that the launch is ordered with the surrounding torch work), else the legacy default stream."""
    if stream:
        return ctypes.c_void_p(stream)
    for t in tensors:
        if hasattr(t, "is_cuda") and t.is_cuda:
            import torch
            s = torch.cuda.current_stream(t.device).cuda_stream
            return ctypes.c_void_p(s) if s else None
    return None


def _ptr(x):
    """Device/host address of a torch tensor, numpy array or raw int."""
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if hasattr(x, "data_ptr"):
        return ctypes.c_void_p(x.data_ptr())
    if hasattr(x, "ctypes"):
        return ctypes.c_void_p(x.ctypes.data)
    raise TypeError("expected a tensor, array or address, got %r" % type(x))


class Plan:
    """One contraction: expression + dtype (+ extents, strides, options)."""

    def __init__(self, expr, dtype=F64, path=PATH_AUTO, tile=None, split_k=0, extents=None, variant=0, l2_prefetch=0, c_path=0, tma=0,
                 test_fault=0):
        self._h = ctypes.c_void_p()
        opt = Options()
        opt.path = path
        if tile:
            opt.tile_m, opt.tile_n = tile
        opt.split_k = split_k
        opt.variant = variant
        opt.l2_prefetch = l2_prefetch
        opt.c_path = c_path
        opt.tma = tma
        opt.test_fault = test_fault
        self.expr = expr
        self.dtype = dtype
        _check(lib().tc_plan_create(expr.encode(), dtype, ctypes.byref(opt), ctypes.byref(self._h)), "tc_plan_create")
        if extents:
            self.set_extents(extents)

    def set_extents(self, extents):
        names = list(extents)
        arr_n = (ctypes.c_char_p * len(names))(*[n.encode() for n in names])
        arr_e = (ctypes.c_int64 * len(names))(*[int(extents[n]) for n in names])
        _check(lib().tc_plan_set_extents(self._h, len(names), arr_n, arr_e), "tc_plan_set_extents")
        return self

    def set_strides(self, tensor, strides):
        arr = (ctypes.c_int64 * len(strides))(*[int(s) for s in strides])
        _check(lib().tc_plan_set_strides(self._h, tensor, len(strides), arr), "tc_plan_set_strides")
        return self

    def commit(self):
        _check(lib().tc_plan_commit(self._h), "tc_plan_commit")
        return self

    def describe(self):
        buf = ctypes.create_string_buffer(16384)
        st = lib().tc_plan_describe(self._h, buf, len(buf))
        if st != 0:
            raise TcError(st, "tc_plan_describe", json.loads(buf.value.decode() or "{}").get("error", ""))
        return json.loads(buf.value.decode())

    def cost(self):
        f, b = ctypes.c_double(), ctypes.c_double()
        _check(lib().tc_plan_cost(self._h, ctypes.byref(f), ctypes.byref(b)), "tc_plan_cost")
        return f.value, b.value

    @property
    def launches(self):
        return lib().tc_plan_launches(self._h)

    def status(self):
        """Device status word (synchronises): 0 unless a bounded wait in a persistent kernel gave up."""
        v = ctypes.c_int()
        _check(lib().tc_plan_status(self._h, ctypes.byref(v)), "tc_plan_status")
        return v.value

    def status_reset(self):
        _check(lib().tc_plan_status_reset(self._h), "tc_plan_status_reset")

    def workspace_bytes(self):
        n = ctypes.c_size_t()
        _check(lib().tc_plan_workspace_bytes(self._h, ctypes.byref(n)), "tc_plan_workspace_bytes")
        return n.value

    def execute(self, C, A, B, stream=None, workspace=None):
        """Enqueue C (op)= sum A*B on device tensors (torch CUDA tensors or raw device addresses)."""
        s = _stream(stream, C)
        if workspace is None:
            _check(lib().tc_execute(self._h, _ptr(C), _ptr(A), _ptr(B), s), "tc_execute")
        else:
            nbytes = workspace.numel() * workspace.element_size()
            _check(lib().tc_execute_ws(self._h, _ptr(C), _ptr(A), _ptr(B), _ptr(workspace), nbytes, s), "tc_execute_ws")

    def execute_noalloc(self, C, A, B, stream=None):
        """tc_execute that takes K-slice scratch from the library's fixed array instead of allocated memory
        (for callers that cannot allocate); the plan must be committed and the scratch need must fit."""
        s = _stream(stream, C)
        _check(lib().tc_execute_noalloc(self._h, _ptr(C), _ptr(A), _ptr(B), s), "tc_execute_noalloc")

    def execute_host(self, C, A, B):
        """Blocking call on host arrays (numpy, C-contiguous 1-D storage in column-major element order)."""
        _check(lib().tc_execute_host(self._h, _ptr(C), _ptr(A), _ptr(B)), "tc_execute_host")

    def close(self):
        if self._h:
            lib().tc_plan_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


SHARD_EXTERNAL, SHARD_CONTRACTION, SHARD_C_IS_SLAB = 0, 1, 1


class ShardedPlan:
    """One contraction over several GPUs driven by this process (tc_plan_create_sharded): `kind` SHARD_EXTERNAL cuts
    an output index (no communication), SHARD_CONTRACTION a contraction index (NCCL reduce-scatter)."""

    def __init__(self, expr, dtype=F64, devices=(0,), kind=SHARD_EXTERNAL, index=None, extents=None):
        self._h = ctypes.c_void_p()
        self.devices = list(devices)
        ids = (ctypes.c_int * len(self.devices))(*self.devices)
        _check(lib().tc_plan_create_sharded(expr.encode(), dtype, len(self.devices), ids, kind,
                                            index.encode() if index else None, ctypes.byref(self._h)), "tc_plan_create_sharded")
        if extents:
            names = list(extents)
            an = (ctypes.c_char_p * len(names))(*[n.encode() for n in names])
            ae = (ctypes.c_int64 * len(names))(*[int(extents[n]) for n in names])
            _check(lib().tc_sharded_set_extents(self._h, len(names), an, ae), "tc_sharded_set_extents")

    def describe(self):
        buf = ctypes.create_string_buffer(1 << 16)
        st = lib().tc_sharded_describe(self._h, buf, len(buf))
        if st != 0:
            raise TcError(st, "tc_sharded_describe", json.loads(buf.value.decode() or "{}").get("error", ""))
        return json.loads(buf.value.decode())

    def commit(self):
        _check(lib().tc_sharded_commit(self._h), "tc_sharded_commit")
        return self

    def execute(self, Cs, As, Bs, c_is_slab=False):
        """Cs[d], As[d], Bs[d]: the tensors in device d's memory (torch CUDA tensors or device addresses)."""
        n = len(self.devices)
        if not (len(Cs) == len(As) == len(Bs) == n):
            raise ValueError("one output and two inputs per device")
        arr = lambda xs: (ctypes.c_void_p * n)(*[_ptr(x) for x in xs])
        _check(lib().tc_execute_sharded(self._h, arr(Cs), arr(As), arr(Bs), SHARD_C_IS_SLAB if c_is_slab else 0), "tc_execute_sharded")

    def synchronize(self):
        _check(lib().tc_sharded_synchronize(self._h), "tc_sharded_synchronize")

    def close(self):
        if self._h:
            lib().tc_sharded_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class FusedPlan:
    """Several contractions accumulated into one output in a single pass over it (e.g. the nine CCSD(T) terms
    of cogent/input_strings/ccsd_t/original-expressions/sd_t_d2.in); fp64."""

    def __init__(self, exprs, dtype=F64, extents=None):
        self._h = ctypes.c_void_p()
        self.exprs = list(exprs)
        arr = (ctypes.c_char_p * len(self.exprs))(*[e.encode() for e in self.exprs])
        _check(lib().tc_plan_create_fused(len(self.exprs), arr, dtype, ctypes.byref(self._h)), "tc_plan_create_fused")
        if extents:
            names = list(extents)
            an = (ctypes.c_char_p * len(names))(*[n.encode() for n in names])
            ae = (ctypes.c_int64 * len(names))(*[int(extents[n]) for n in names])
            _check(lib().tc_fused_set_extents(self._h, len(names), an, ae), "tc_fused_set_extents")

    def commit(self):
        _check(lib().tc_fused_commit(self._h), "tc_fused_commit")
        return self

    def describe(self):
        buf = ctypes.create_string_buffer(8192)
        st = lib().tc_fused_describe(self._h, buf, len(buf))
        if st != 0:
            raise TcError(st, "tc_fused_describe", json.loads(buf.value.decode() or "{}").get("error", ""))
        return json.loads(buf.value.decode())

    def execute(self, C, As, Bs, stream=None):
        """C: the output; As[k], Bs[k]: left / right input of term k (torch CUDA tensors or device addresses)."""
        n = len(self.exprs)
        if len(As) != n or len(Bs) != n:
            raise ValueError("one left and one right input per term")
        pa = (ctypes.c_void_p * n)(*[_ptr(x) for x in As])
        pb = (ctypes.c_void_p * n)(*[_ptr(x) for x in Bs])
        _check(lib().tc_execute_fused(self._h, _ptr(C), pa, pb, _stream(stream, C)), "tc_execute_fused")

    def close(self):
        if self._h:
            lib().tc_fused_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sd_t_d2_fusion(expr, sizes, t3, t2, v2, dtype=F64):
    """The reference's generated entry for one expression: sizes in output-then-contraction order, numpy host arrays."""
    arr = (ctypes.c_int * len(sizes))(*[int(x) for x in sizes])
    _check(lib().tc_sd_t_d2_fusion(expr.encode(), dtype, len(sizes), arr, _ptr(t3), _ptr(t2), _ptr(v2)), "tc_sd_t_d2_fusion")


def fill_uniform(t, seed, tensor_id, first_index=0, stream=None):
    """Fills a CUDA tensor with the seeded uniform[-1,1) stream for (seed, tensor_id)."""
    import torch
    dt = F64 if t.dtype == torch.float64 else F32
    s = _stream(stream, t)
    _check(lib().tc_fill_uniform(_ptr(t), t.numel(), dt, seed, tensor_id, first_index, s), "tc_fill_uniform")
    return t


def axpy(y, x, alpha=1.0, stream=None):
    import torch
    dt = F64 if y.dtype == torch.float64 else F32
    s = _stream(stream, y)
    _check(lib().tc_axpy(_ptr(y), _ptr(x), y.numel(), dt, alpha, s), "tc_axpy")
    return y


_probes = None


def probes():
    """The bench-only probe library (pipe peaks, streaming read-modify-write); not part of the product ABI."""
    global _probes
    if _probes is None:
        if not os.path.exists(PROBES_PATH):
            raise ImportError("%s is missing: run build.py" % PROBES_PATH)
        h = ctypes.CDLL(PROBES_PATH)
        h.tc_peak_measure.restype = ctypes.c_int
        h.tc_peak_measure.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
        h.tc_peak_measure_rmw.restype = ctypes.c_int
        h.tc_peak_measure_rmw.argtypes = [ctypes.c_int64, ctypes.POINTER(ctypes.c_double)]
        _probes = h
    return _probes


def measure_peaks(which=(0, 4, 5), iters=4096, ctas_per_sm=2):
    """TFLOP/s of the arithmetic pipes (register-only loops; 7 = TF32 on tcgen05 from shared memory) on the current device."""
    out = {}
    for w in which:
        v = ctypes.c_double()
        _check(probes().tc_peak_measure(w, iters, ctas_per_sm, ctypes.byref(v)), "tc_peak_measure")
        out[PEAK_NAMES[w]] = v.value
    return out


def measure_rmw(nbytes=4 << 30):
    v = ctypes.c_double()
    _check(probes().tc_peak_measure_rmw(nbytes, ctypes.byref(v)), "tc_peak_measure_rmw")
    return v.value
