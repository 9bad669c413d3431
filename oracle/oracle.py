"""TEST INFRASTRUCTURE -- Python face of the CPU checker.

Only tests, the smoke check and the bench's CPU-baseline / reference legs may
import this module.  It wraps

  * liboracle.so      the C restatement of the reference's loop-nest contraction
                      (oracle/tc_oracle.c; follows post_Correctness in
                      cogent/drivers/tccg/code_main_tccg_02.c:109-133 and siblings)
  * _ref/libref_nests.so  the reference's own 57 loop nests compiled in place
                      (present where oracle/build_oracle.py ran with the
                      reference tree available)

and restates, independently of the product's C++ parser, the token positions of
the reference grammar (cogent/src/algs/bases/tc_gen_inputs.py:28-108) so that
the product parser can be checked against it.
"""
import contextlib
import ctypes
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(HERE, "liboracle.so")
_REF_LIB = os.path.join(HERE, "_ref", "libref_nests.so")
_REF_JSON = os.path.join(HERE, "_ref", "ref_nests.json")

_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            raise ImportError("oracle/liboracle.so missing: run python oracle/build_oracle.py")
        h = ctypes.CDLL(_LIB)
        i64p, i32p = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int32)
        h.tc_oracle_contract.restype = ctypes.c_int
        h.tc_oracle_contract.argtypes = [ctypes.c_int, ctypes.c_int, i64p, ctypes.c_int, i64p, ctypes.c_int, i32p,
                                         ctypes.c_int, i32p, i64p, i64p, i64p, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        h.tc_oracle_fill.restype = None
        h.tc_oracle_fill.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64, ctypes.c_int,
                                     ctypes.c_int64]
        h.tc_oracle_max_threads.restype = ctypes.c_int
        _lib = h
    return _lib


# ------------------------------------------------------------------ grammar ----
def parse(line):
    """Token-position parse, as the reference does it.  Returns a dict or raises ValueError."""
    if line.startswith("#"):
        raise ValueError("comment line")
    tok = line.replace("[", "").replace("]", "").replace(";", "").split()
    if len(tok) != 10:
        raise ValueError("expected 10 tokens, got %d" % len(tok))
    out = tok[1].split(",")
    if len(out) % 2:
        raise ValueError("output list must alternate index and extent")
    sm = tok[3]
    if not (sm.startswith("sum(") and sm.endswith(")")):
        raise ValueError("fourth token must be sum(...)")
    sm = sm[4:-1].split(",")
    if len(sm) % 2:
        raise ValueError("sum list must alternate index and extent")
    if tok[2] not in ("+=", "-=", "="):
        raise ValueError("bad operator")
    if tok[4] != "*" or tok[7] != "*":
        raise ValueError("operands must be joined by ' * '")
    return {
        "out": tok[0], "left": tok[5], "right": tok[8], "op": tok[2],
        "out_idx": out[0::2], "out_ext": [int(x) for x in out[1::2]],
        "sum_idx": sm[0::2], "sum_ext": [int(x) for x in sm[1::2]],
        "left_idx": tok[6].split(","), "right_idx": tok[9].split(","),
    }


def with_extents(expr, extents):
    """The same expression with the extents of the named indices replaced."""
    p = parse(expr)
    oe = [extents.get(i, e) for i, e in zip(p["out_idx"], p["out_ext"])]
    se = [extents.get(i, e) for i, e in zip(p["sum_idx"], p["sum_ext"])]
    return "%s [%s] %s sum(%s) * %s [%s] * %s [%s];" % (
        p["out"], ",".join("%s,%d" % x for x in zip(p["out_idx"], oe)), p["op"],
        ",".join("%s,%d" % x for x in zip(p["sum_idx"], se)), p["left"], ",".join(p["left_idx"]),
        p["right"], ",".join(p["right_idx"]))


def sizes(expr):
    """(|C|, |A|, |B|) element counts for compact tensors."""
    p = parse(expr)
    ext = dict(zip(p["out_idx"] + p["sum_idx"], p["out_ext"] + p["sum_ext"]))
    n = lambda idx: int(np.prod([ext[i] for i in idx], dtype=np.int64)) if idx else 1
    return n(p["out_idx"]), n(p["left_idx"]), n(p["right_idx"])


# ----------------------------------------------------------------- seeded inputs ----
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(z):
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform(seed, tensor_id, count, dtype=np.float64, first=0):
    """Elements [first, first+count) of the uniform[-1,1) stream of (seed, tensor_id).

    tensor_id: 0 = output's initial value, 1 = left input, 2 = right input."""
    with np.errstate(over="ignore"):
        key = (np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)) ^ (np.uint64(tensor_id) << np.uint64(60))
        x = _splitmix64(key ^ (np.arange(first, first + count, dtype=np.int64).astype(np.uint64)))
    if np.dtype(dtype) == np.float64:
        return (x >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0) * 2.0 - 1.0
    return ((x >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0) * np.float32(2.0)
            - np.float32(1.0)).astype(np.float32)


def uniform_at(seed, tensor_id, indices, dtype=np.float64):
    """The same stream at scattered element indices (sampled-coordinate checks of tensors too large to hold)."""
    with np.errstate(over="ignore"):
        key = (np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)) ^ (np.uint64(tensor_id) << np.uint64(60))
        x = _splitmix64(key ^ np.asarray(indices, dtype=np.int64).astype(np.uint64))
    if np.dtype(dtype) == np.float64:
        return (x >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0) * 2.0 - 1.0
    return ((x >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0) * np.float32(2.0)
            - np.float32(1.0)).astype(np.float32)


def fill_c(arr, seed, tensor_id, first=0):
    """Same stream, produced by the C restatement (cross-checks the numpy one)."""
    dt = 0 if arr.dtype == np.float64 else 1
    lib().tc_oracle_fill(dt, arr.ctypes.data, arr.size, seed, tensor_id, first)
    return arr


def make_inputs(expr, seed, dtype=np.float64):
    nc, na, nb = sizes(expr)
    return (uniform(seed, 0, nc, dtype), uniform(seed, 1, na, dtype), uniform(seed, 2, nb, dtype))


# ------------------------------------------------------------------- contraction ----
def max_threads():
    return lib().tc_oracle_max_threads()


def contract(expr, C, A, B, threads=1, strides=None):
    """In place: C (op)= sum A*B with the reference's loop order.  Arrays are flat
    (column-major element order).  strides: optional dict tensor(0/1/2) -> list."""
    p = parse(expr)
    ids = {n: i for i, n in enumerate(p["out_idx"] + p["sum_idx"])}
    a_idx = (ctypes.c_int32 * len(p["left_idx"]))(*[ids[i] for i in p["left_idx"]])
    b_idx = (ctypes.c_int32 * len(p["right_idx"]))(*[ids[i] for i in p["right_idx"]])
    oe = (ctypes.c_int64 * max(1, len(p["out_ext"])))(*p["out_ext"])
    se = (ctypes.c_int64 * max(1, len(p["sum_ext"])))(*p["sum_ext"])
    st = [None, None, None]
    for t, s in (strides or {}).items():
        st[t] = (ctypes.c_int64 * len(s))(*s)
    assert C.dtype == A.dtype == B.dtype and C.dtype in (np.float64, np.float32)
    assert C.flags.c_contiguous and A.flags.c_contiguous and B.flags.c_contiguous
    op = {"+=": 1, "-=": -1, "=": 0}[p["op"]]
    rc = lib().tc_oracle_contract(0 if C.dtype == np.float64 else 1, len(p["out_idx"]), oe, len(p["sum_idx"]), se,
                                  len(p["left_idx"]), a_idx, len(p["right_idx"]), b_idx, st[0], st[1], st[2], op,
                                  C.ctypes.data, A.ctypes.data, B.ctypes.data, threads)
    if rc != 0:
        raise ValueError("oracle rejected the contraction")
    return C


def rel_error(got, ref):
    """max|got-ref| / max|ref| -- the gate used by every parity test."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    scale = float(np.max(np.abs(ref))) if ref.size else 1.0
    return float(np.max(np.abs(got - ref))) / (scale if scale > 0 else 1.0) if ref.size else 0.0


# --------------------------------------------------------- the reference's own nests ----
def ref_available():
    return os.path.exists(_REF_LIB) and os.path.exists(_REF_JSON)


def ref_table():
    with open(_REF_JSON) as f:
        return json.load(f)


@contextlib.contextmanager
def _quiet_stdout():
    """The reference nests print a report; keep it off the test output."""
    sys.stdout.flush()
    saved = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    try:
        os.dup2(devnull, 1)
        yield
    finally:
        ctypes.CDLL(None).fflush(None)
        os.dup2(saved, 1)
        os.close(devnull)
        os.close(saved)


def ref_contract(tag, extents, C, A, B):
    """Runs the reference's compiled post_Correctness for driver `tag` (e.g. 'f64_02'):
    accumulates into C (its h_C_chk argument).  extents: dict index -> int."""
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(_REF_LIB)
    info = ref_table()[tag]
    fn = getattr(_ref, info["symbol"])
    n = len(info["size_args"])
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * n
    dummy = np.array(C, copy=True)  # its h_C argument: only compared and printed
    with _quiet_stdout():
        fn(dummy.ctypes.data, C.ctypes.data, A.ctypes.data, B.ctypes.data, *[int(extents[i]) for i in info["size_args"]])
    return C
