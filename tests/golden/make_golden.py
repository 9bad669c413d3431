"""Regenerates tests/golden/ref_nests.npz from the reference's OWN loop nests.

Needs oracle/_ref/libref_nests.so, which oracle/build_oracle.py compiles from the
reference tree where that tree is present; the fixtures let the same checks run
where it is absent.  Each record holds what the reference's compiled
post_Correctness produced for seeded inputs:

  <tag>/expr     the contraction, recovered from the driver's code, with extents
  <tag>/seed     inputs are oracle.uniform(seed, 0|1|2, ...) (initial C, A, B)
  <tag>/out      the full output for small extents, or
  <tag>/every    the stride of the committed sample out[::every] for the large case
  <tag>/sum      exact sums (out.sum(), abs(out).sum()) over the FULL output

Usage: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import oracle as O  # noqa: E402

# (driver tag, extents, seed, keep every n-th element)
CASES = [
    # the configuration the reference CPU path is quoted on: its expression is driver 02's
    ("f64_02", {"a": 64, "b": 48, "c": 32, "d": 40}, 0, 13),
    ("f64_02", {"a": 5, "b": 3, "c": 4, "d": 7}, 10, 1),
    ("f64_05", {"a": 4, "b": 3, "c": 5, "d": 2, "e": 6}, 11, 1),
    ("f64_13", {"a": 6, "b": 5, "c": 4, "d": 3}, 12, 1),
    ("f64_29", {"a": 3, "b": 4, "c": 2, "d": 3, "e": 5, "f": 4}, 13, 1),
    ("f64_31", {"a": 3, "b": 2, "c": 2, "d": 3, "e": 2, "f": 3, "g": 5}, 14, 1),
    ("f64_40", {"a": 2, "b": 3, "c": 2, "d": 3, "e": 2, "f": 2, "g": 6}, 15, 1),
    ("f32_40", {"a": 2, "b": 3, "c": 2, "d": 3, "e": 2, "f": 2, "g": 6}, 16, 1),
    ("f32_44", {"a": 3, "b": 2, "c": 3, "d": 2, "e": 3, "f": 2, "g": 24}, 17, 1),
]


def main():
    if not O.ref_available():
        raise SystemExit("oracle/_ref is not built: run python oracle/build_oracle.py where the reference tree is present")
    table = O.ref_table()
    out = {}
    for n, (tag, ext, seed, every) in enumerate(CASES):
        info = table[tag]
        expr = O.with_extents(info["expr"], ext)
        dt = np.float64 if info["dtype"] == "f64" else np.float32
        c, a, b = O.make_inputs(expr, seed, dt)
        O.ref_contract(tag, ext, c, a, b)
        key = "%02d_%s" % (n, tag)
        out[key + "/expr"] = np.array(expr)
        out[key + "/seed"] = np.array(seed)
        out[key + "/every"] = np.array(every)
        out[key + "/out"] = c[::every].copy()
        out[key + "/sum"] = np.array([c.astype(np.float64).sum(), np.abs(c.astype(np.float64)).sum()])
    path = os.path.join(HERE, "ref_nests.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(CASES), "cases")


if __name__ == "__main__":
    main()
