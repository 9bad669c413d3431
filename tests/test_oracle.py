"""The CPU checker against the reference's own loop nests (compiled or golden)."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_nests.npz")


def _golden_cases():
    z = np.load(GOLDEN)
    keys = sorted({k.split("/")[0] for k in z.files})
    return [(k, str(z[k + "/expr"]), int(z[k + "/seed"]), int(z[k + "/every"]), z[k + "/out"], z[k + "/sum"]) for k in keys]


@pytest.mark.parametrize("key,expr,seed,every,out,sums", _golden_cases(), ids=[c[0] for c in _golden_cases()])
def test_oracle_matches_golden_bit_for_bit(orc, key, expr, seed, every, out, sums):
    c, a, b = orc.make_inputs(expr, seed, out.dtype)
    orc.contract(expr, c, a, b)
    assert np.array_equal(c[::every], out)
    assert c.astype(np.float64).sum() == sums[0]
    assert np.abs(c.astype(np.float64)).sum() == sums[1]


def test_oracle_matches_every_compiled_reference_nest(orc):
    if not orc.ref_available():
        pytest.skip("reference nests not compiled here (oracle/_ref absent); golden vectors cover them")
    rng = np.random.default_rng(1234)
    table = orc.ref_table()
    assert len(table) == 57
    for tag, info in sorted(table.items()):
        p = orc.parse(info["expr"])
        ext = {n: int(rng.integers(1, 7)) for n in p["out_idx"] + p["sum_idx"]}
        expr = orc.with_extents(info["expr"], ext)
        dt = np.float64 if info["dtype"] == "f64" else np.float32
        c0, a, b = orc.make_inputs(expr, 99, dt)
        mine = orc.contract(expr, c0.copy(), a, b)
        theirs = orc.ref_contract(tag, ext, c0.copy(), a, b)
        assert np.array_equal(mine, theirs), (tag, expr)


def test_threaded_oracle_is_bit_identical(orc):
    expr = "C [a,7,b,5,c,6,d,3] -= sum(e,9,f,4) * A [e,c,a,f] * B [b,f,d,e];"
    for dt in (np.float64, np.float32):
        c0, a, b = orc.make_inputs(expr, 5, dt)
        s = orc.contract(expr, c0.copy(), a, b, threads=1)
        t = orc.contract(expr, c0.copy(), a, b, threads=4)
        assert np.array_equal(s, t)


def test_overwrite_operator_ignores_initial_output(orc):
    expr = "C [a,4,b,3] = sum(c,5) * A [c,a] * B [b,c];"
    c0, a, b = orc.make_inputs(expr, 1)
    got = orc.contract(expr, c0.copy(), a, b)
    want = np.einsum("ca,bc->ab", a.reshape(4, 5).T.reshape(5, 4), b.reshape(5, 3).T.reshape(3, 5))
    # column-major flat: element (a,b) at a + 4*b
    assert np.allclose(got.reshape(3, 4).T, want, rtol=1e-13, atol=1e-13)


def test_oracle_against_einsum(orc):
    # independent formulation: numpy einsum on Fortran-ordered views
    expr = "C [a,5,b,4,c,3,d,2] += sum(e,6,f,3) * A [e,c,a,f] * B [b,f,d,e];"
    c0, a, b = orc.make_inputs(expr, 3)
    got = orc.contract(expr, c0.copy(), a, b)
    A = a.reshape((6, 3, 5, 3), order="F")  # e,c,a,f
    B = b.reshape((4, 3, 2, 6), order="F")  # b,f,d,e
    want = c0.reshape((5, 4, 3, 2), order="F") + np.einsum("ecaf,bfde->abcd", A, B)
    assert np.allclose(got.reshape((5, 4, 3, 2), order="F"), want, rtol=1e-13, atol=1e-13)


def test_strided_views(orc):
    # contraction over a slab [2,5) of index b of a larger output/right tensor, via strides
    full = "C [a,4,b,7] += sum(c,5) * A [c,a] * B [b,c];"
    c0, a, b = orc.make_inputs(full, 8)
    want = orc.contract(full, c0.copy(), a, b)
    slab = "C [a,4,b,3] += sum(c,5) * A [c,a] * B [b,c];"
    c = c0.copy()
    orc.contract(slab, c[4 * 2:], a, b[2:], strides={0: [1, 4], 2: [1, 7]})
    assert np.array_equal(c[8:20], want[8:20])
    assert np.array_equal(c[:8], c0[:8]) and np.array_equal(c[20:], c0[20:])


def test_generators_agree(orc):
    for dt in (np.float64, np.float32):
        for seed, tid, first in ((0, 0, 0), (3, 1, 17), (4, 2, 1 << 33)):
            x = orc.uniform(seed, tid, 257, dt, first)
            y = orc.fill_c(np.empty(257, dtype=dt), seed, tid, first)
            assert np.array_equal(x, y)
            assert x.min() >= -1.0 and x.max() < 1.0
    x = orc.uniform(0, 1, 200000)
    assert abs(x.mean()) < 0.01 and abs(x.var() - 1.0 / 3.0) < 0.01
