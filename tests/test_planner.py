"""Host-side planner (no GPU): index classes, fusion, loaders, tiles, costs, errors."""
import pytest

from conftest import CONFIGS


def _plan(pkg, expr, dtype="float64", **kw):
    return pkg.Plan(expr, pkg.F64 if dtype == "float64" else pkg.F32, **kw)


def test_algorithmic_costs_of_the_benchmark_configurations(pkg):
    # flops = 2 * prod(extents); bytes = elemsize * (2|C| + |A| + |B|)
    want = [(7864320, 2243584), (16307453952, 2038505472), (137438953472, 536870912),
            (9172942848, 1531478016), (327680000000, 65576960000)]
    for (expr, dt, _), (fl, by) in zip(CONFIGS, want):
        f, b = _plan(pkg, expr, dt).cost()
        assert (f, b) == (fl, by)


def test_index_classes_and_fusion(pkg):
    d = [_plan(pkg, e, dt).describe() for e, dt, _ in CONFIGS]
    # cfg1: M = {i,k} (left operand), N = {j}, K = {l}
    assert [x["extent"] for x in d[0]["M"]] == [64, 32] and [x["extent"] for x in d[0]["N"]] == [48]
    assert d[0]["Kflat"] == 40 and not d[0]["swapped"]
    # cfg2: nothing fuses (b,d adjacent in A but not in C)
    assert [x["extent"] for x in d[1]["M"]] == [96, 96, 96] and d[1]["Nflat"] == 96
    # cfg3: two contraction indices flatten to 4096
    assert d[2]["Mflat"] == d[2]["Nflat"] == d[2]["Kflat"] == 4096
    # cfg4: (i,j) and (b,c) fuse: adjacent in the output and in their operand
    assert [x["extent"] for x in d[3]["M"]] == [24, 576] and [x["extent"] for x in d[3]["N"]] == [576, 24]
    # cfg5: becomes a plain 64000 x 64000 x 40 product
    assert [x["extent"] for x in d[4]["M"]] == [64000] and [x["extent"] for x in d[4]["N"]] == [64000]
    assert d[4]["M"][0]["s_in"] == 40 and d[4]["M"][0]["s_out"] == 1


def test_operands_swap_when_output_fastest_index_is_in_the_right_operand(pkg):
    d = _plan(pkg, "C [a,8,b,8] += sum(c,8) * A [c,b] * B [a,c];").describe()
    assert d["swapped"] and d["M"][0]["s_out"] == 1 and d["vec_c"] == 4


def test_loader_and_vector_choices(pkg):
    d2 = _plan(pkg, CONFIGS[1][0]).describe()
    assert d2["vec_x"] and not d2["vec_y"] and d2["lanes_k_y"] == 4 and d2["vec_c"] == 4
    d4 = _plan(pkg, CONFIGS[3][0], "float32").describe()
    assert not d4["vec_x"] and d4["lanes_k_x"] == 8 and d4["vec_y"] and d4["vec_c"] == 4
    odd = _plan(pkg, "C [a,7,b,5] += sum(c,3) * A [a,c] * B [c,b];").describe()
    assert not odd["vec_x"] and odd["vec_c"] == 1
    even = _plan(pkg, "C [a,6,b,5] += sum(c,3) * A [a,c] * B [c,b];").describe()
    assert even["vec_x"] and even["vec_c"] == 2


def test_tile_choices(pkg):
    d = [_plan(pkg, e, dt).describe() for e, dt, _ in CONFIGS]
    # fp64 with enough tiles: the persistent warp-specialised kernel (variant 2)
    assert d[1]["kernel"] == "dmma_ws_64x96" and d[1]["tiles"] == [13824, 1]   # N = 96 is exactly one tile wide
    assert d[2]["kernel"] == "dmma_ws_128x64" and d[2]["tiles"] == [32, 64]
    # output-bound fp64 (K = 40): the kernel that keeps the output tile resident in shared memory
    assert d[4]["kernel"] == "dmma_wc_128x64" and d[4]["tiles"] == [500, 1000] and d[4]["tma_ct"] and d[4]["mblock_w"] == 32
    longer = _plan(pkg, CONFIGS[4][0].replace("g,40", "g,96")).describe()
    assert longer["kernel"].startswith("dmma_w") and longer["estimate_us"] > 2 * d[4]["estimate_us"]   # pipe-bound: time follows K
    # a skinny right operand (one external index of 24): the 32-wide tile wastes a quarter of its columns, not five eighths
    skinny = _plan(pkg, "t3 [a,312,b,24,c,296] += sum(d,312) * t2 [d,c,a] * v2 [b,d];").describe()
    assert skinny["kernel"] == "dmma_ws_128x32" and skinny["tiles"] == [722, 1] and skinny["estimate_us"] > 0
    # fp32: 96 rows = 4 whole runs of the 24-long fastest output index; (a, bc) blocks leave as bulk chunks
    # (default: the tcgen05 form of the three-TF32 product as the persistent kernel; one CTA per tile or the mma.sync
    # form on request or for small problems)
    assert d[3]["math"] == "tf32x3_tcgen05" and d[3]["kernel"] == "tf32wt_96x128" and d[3]["ksplit"] == 1
    per_tile = _plan(pkg, CONFIGS[3][0], "float32", path=pkg.PATH_TCGEN05, tile=(96, 128), variant=1).describe()
    assert per_tile["kernel"] == "tf32tc_96x128"
    sync = _plan(pkg, CONFIGS[3][0], "float32", path=pkg.PATH_3XTF32).describe()
    assert sync["math"] == "tf32x3" and sync["kernel"] == "tf32_96x128"
    # a 96-wide N leaves a quarter of a 128-wide tcgen05 tile empty and every tile ragged: mma.sync form
    n96 = _plan(pkg, CONFIGS[1][0], "float32").describe()
    assert n96["math"] == "tf32x3" and n96["kernel"] == "tf32_96x128"
    ffma = _plan(pkg, CONFIGS[3][0], "float32", path=pkg.PATH_FFMA).describe()
    assert ffma["math"] == "ffma" and ffma["kernel"] == "ffma_96x128"
    assert d[3]["epi_run"] == 24 and d[3]["epi_n_span"] == 576
    assert d[0]["kernel"] == "dmma_64x64_w4"                                    # tiny problem: one CTA per tile
    # operands whose fastest index is contracted are staged contraction-major with 16-byte copies
    assert d[4]["kvec_x"] and d[4]["vec_y"] and not d[4]["vec_x"]
    assert d[2]["kvec_x"] and d[2]["vec_y"]
    # forcing a persistent kernel disables the K split
    forced = _plan(pkg, "C [a,33,b,17] += sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];", tile=(128, 64), variant=3).describe()
    assert forced["ksplit"] == 1 and forced["kernel"] == "dmma_ws_128x64"


def test_output_tensor_boxes(pkg):
    """Which outputs the persistent fp64 kernel may write as tiled TMA boxes (per warp batch / per tile)."""
    d = [_plan(pkg, e, dt).describe() for e, dt, _ in CONFIGS]
    # cfg2: (a, b) are contiguous in C although not in A: runs of 9216 hold the 64-row tiles; N = c alone
    assert d[1]["tma_c"] and d[1]["tma_ct"]
    # cfg5: M and N both fuse into one dimension
    assert d[4]["tma_c"] and d[4]["tma_ct"]
    # cfg3: the fastest M dimension (64) is shorter than the 128-row tile
    assert not d[2]["tma_c"] and not d[2]["tma_ct"]
    kw = dict(tile=(64, 96), variant=3)
    # N = (b: 32, d: 2): a batch of 16 rows stays inside b, a 96-row tile does not
    e = _plan(pkg, "C [a,128,b,32,c,3,d,2] += sum(e,24) * A [e,a,c] * B [b,d,e];", **kw).describe()
    assert e["tma_c"] and not e["tma_ct"]
    # N's fastest dimension 24 is not a multiple of 16 and N has a second dimension
    e = _plan(pkg, "C [a,128,b,24,c,3,d,4] += sum(e,16) * A [e,a,c] * B [b,d,e];", **kw).describe()
    assert not e["tma_c"]
    # ... but (b, c) contiguous in C count as one dimension of 96 whatever their order in B
    e = _plan(pkg, "C [a,128,b,24,c,4] += sum(e,16) * A [e,a] * B [b,e,c];", **kw).describe()
    assert e["tma_c"] and e["tma_ct"]
    # odd extent of the only N dimension: n cannot split into (parity, n / 2)
    e = _plan(pkg, "C [a,128,b,33] += sum(e,16) * A [e,a] * B [e,b];", **kw).describe()
    assert not e["tma_c"]
    # fp32 and the one-CTA-per-tile kernels never use them
    assert not d[3]["tma_c"] and not d[0]["tma_c"]


def test_k_split_plans(pkg):
    p = _plan(pkg, "C [a,33,b,17] += sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];")
    d = p.describe()
    assert d["ksplit"] > 1 and d["launches"] == 2 and d["workspace_bytes"] == d["ksplit"] * 64 * 64 * 8
    assert d["k_chunk"] % 16 == 0 and d["k_chunk"] * d["ksplit"] >= 9000
    assert _plan(pkg, "C [a,33,b,17] += sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];", split_k=1).describe()["ksplit"] == 1
    assert _plan(pkg, CONFIGS[1][0]).describe()["ksplit"] == 1


def test_extent_override_and_errors(pkg):
    p = _plan(pkg, "t3 [a,16,b,16,c,16] += sum(d,16) * t2 [d,c,a] * v2 [b,d];")
    p.set_extents({"a": 312, "b": 24, "c": 296, "d": 312})
    assert p.cost()[0] == 2.0 * 312 * 24 * 296 * 312
    with pytest.raises(pkg.TcError) as e:
        p.set_extents({"z": 3})
    assert e.value.status == 2
    with pytest.raises(pkg.TcError) as e:
        p.set_extents({"a": 0})
    assert e.value.status == 4
    with pytest.raises(pkg.TcError) as e:
        _plan(pkg, CONFIGS[0][0], tile=(48, 48)).describe()
    assert e.value.status == 3
    with pytest.raises(pkg.TcError) as e:
        _plan(pkg, CONFIGS[0][0], path=pkg.PATH_FFMA).describe()
    assert e.value.status == 2
    with pytest.raises(pkg.TcError) as e:
        _plan(pkg, CONFIGS[3][0], "float32", path=pkg.PATH_DMMA).describe()
    assert e.value.status == 2


def test_strided_views(pkg):
    p = _plan(pkg, "C [a,4,b,3] += sum(c,5) * A [c,a] * B [b,c];")
    p.set_strides(pkg.TENSOR_OUT, [1, 4]).set_strides(pkg.TENSOR_RIGHT, [1, 7])
    d = p.describe()
    assert d["N"][0]["s_in"] == 1 and d["N"][0]["s_out"] == 4
    with pytest.raises(pkg.TcError) as e:
        _plan(pkg, "C [a,4,b,3] += sum(c,5) * A [c,a] * B [b,c];").set_strides(pkg.TENSOR_OUT, [1, 2]).describe()
    assert e.value.status == 4  # output elements would alias
    with pytest.raises(pkg.TcError) as e:
        p.set_strides(pkg.TENSOR_OUT, [1])
    assert e.value.status == 2


def test_sizes_beyond_32_bit(pkg):
    # 4.096e9 output elements: offsets are 64-bit (the reference's int arithmetic cannot address this)
    d = _plan(pkg, CONFIGS[4][0]).describe()
    assert d["tiles"][0] * d["tiles"][1] == 500 * 1000
    assert d["N"][0]["s_out"] == 64000


def test_index_classes_reproduce_the_contraction(pkg, orc):
    """What the kernels are told -- the digits of M, N and K with their strides, the operand swap -- evaluated in numpy
    gives the checker's result for random expressions: the classes cover every element once, fusion, splitting and
    re-ordering of digits included."""
    import random

    import numpy as np

    from test_parser import _random_expr

    def flat(dims, key):
        # flattened index f = sum digit_i * prod(extent_j, j < i)  ->  offset
        off = np.zeros(1, dtype=np.int64)
        for d in dims:
            off = (np.arange(d["extent"], dtype=np.int64)[:, None] * d[key] + off[None, :]).reshape(-1)
        return off

    rng = random.Random(99)
    seen_split = 0
    for n in range(250):
        expr = _random_expr(rng, max_out=6, max_sum=3)
        p = orc.parse(expr)
        # extents from a set that triggers vector, fusion and digit-splitting rules
        ext = {i: rng.choice([1, 2, 3, 4, 4, 5, 8, 8, 12, 16]) for i in p["out_idx"] + p["sum_idx"]}
        expr = orc.with_extents(expr, ext)
        if np.prod([float(v) for v in ext.values()]) > 3e6:
            continue
        c0, a, b = orc.make_inputs(expr, n, "float64")
        want = orc.contract(expr, c0.copy(), a, b)
        d = _plan(pkg, expr).describe()
        x, y = (b, a) if d["swapped"] else (a, b)
        om_x, om_c = flat(d["M"], "s_in"), flat(d["M"], "s_out")
        on_y, on_c = flat(d["N"], "s_in"), flat(d["N"], "s_out")
        ok_x, ok_y = flat(d["K"], "s_in"), flat(d["K"], "s_out")
        assert len(om_x) == d["Mflat"] and len(on_y) == d["Nflat"] and len(ok_x) == d["Kflat"]
        prod = x[om_x[:, None] + ok_x[None, :]] @ y[on_y[:, None] + ok_y[None, :]].T
        where = (om_c[:, None] + on_c[None, :]).reshape(-1)
        assert len(np.unique(where)) == c0.size == where.size, expr      # every output element exactly once
        got = c0.copy()
        op = p["op"]
        got[where] = prod.reshape(-1) if op == "=" else got[where] + (prod.reshape(-1) if op == "+=" else -prod.reshape(-1))
        assert orc.rel_error(got, want) <= 1e-12, (expr, d["M"], d["N"], d["K"])
        seen_split += any(dd["extent"] == 4 and dd["s_out"] != 1 for dd in d["M"][1:2])
    assert seen_split > 0  # the digit re-ordering was exercised


def test_few_tiles_and_a_long_contraction(pkg):
    """fp64 problems that cannot fill the GPU with tiles: the persistent kernel with K slices where its tiles do not
    pad much more than small ones (or the small kernel would gather both operands by element), else one CTA per tile."""
    both_gathered = _plan(pkg, "t3 [a,312,b,296] += sum(c,312,d,312) * t2 [c,a,d] * v2 [d,c,b];").describe()
    assert both_gathered["kernel"] == "dmma_ws_128x64" and both_gathered["ksplit"] > 1 and both_gathered["tiles"] == [3, 5]
    assert both_gathered["workspace_bytes"] == both_gathered["ksplit"] * 15 * 128 * 64 * 8
    assert both_gathered["k_chunk"] % 16 == 0 and both_gathered["k_chunk"] >= 256
    one_vector = _plan(pkg, "t3 [a,312,b,296] += sum(c,296,d,312) * t2 [a,c,d] * v2 [d,b,c];").describe()
    assert one_vector["kernel"] == "dmma_64x64_w4" and one_vector["ksplit"] > 1
    narrow = _plan(pkg, "t3 [a,72,b,72,c,72] += sum(d,72,e,72) * t2 [a,d,e,c] * v2 [e,b,d];").describe()
    assert narrow["kernel"] == "dmma_ws_128x64" and narrow["ksplit"] > 1 and narrow["tiles"] == [41, 2]
    short = _plan(pkg, "C [a,312,b,296] += sum(c,40) * A [c,a] * B [c,b];").describe()
    assert short["kernel"] == "dmma_64x64_w4" and short["ksplit"] == 1
    # on request the persistent kernel slices K whatever the shape
    forced = _plan(pkg, "C [a,200,b,70] -= sum(c,1003) * A [c,a] * B [b,c];", tile=(128, 64), variant=3, split_k=5).describe()
    assert forced["kernel"] == "dmma_ws_128x64" and forced["ksplit"] == 5


def test_no_default_fp32_plan_runs_a_tensor_core_chain_longer_than_512(pkg):
    """fp32 on the tensor cores accumulates with truncation, so the planner bounds every accumulation chain:
    K slices where their scratch fits 1 GiB, sequential passes into C beyond that."""
    import random
    rng = random.Random(9)
    seen = set()
    for n in range(300):
        m = rng.choice([64, 96, 500, 4096, 20000, 60000])
        nn = rng.choice([64, 128, 1000, 4096, 30000])
        k = rng.choice([16, 500, 512, 513, 1024, 4100, 8192, 50000])
        expr = "C [a,%d,b,%d] %s sum(c,%d) * A [c,a] * B [c,b];" % (m, nn, rng.choice(["+=", "-=", "="]), k)
        for path in (pkg.PATH_AUTO, pkg.PATH_TCGEN05, pkg.PATH_3XTF32):
            d = _plan(pkg, expr, "float32", path=path).describe()
            assert d["math"].startswith("tf32x3")
            assert d["chain"] <= 512, (expr, d)
            assert d["passes"] == 1 or d["ksplit"] == 1
            assert d["workspace_bytes"] <= (1 << 30) + 128 * 128 * 4 * d["ksplit"] * 148, (expr, d)
            seen.add("passes" if d["passes"] > 1 else "slices" if d["ksplit"] > 1 else "single")
    assert seen == {"passes", "slices", "single"}
    # the caller may override the rule explicitly, and FFMA never needs it
    assert _plan(pkg, "C [a,4096,b,8192] += sum(c,8192) * A [c,a] * B [c,b];", "float32", split_k=1).describe()["chain"] == 8192
    assert _plan(pkg, "C [a,4096,b,8192] += sum(c,8192) * A [c,a] * B [c,b];", "float32", path=pkg.PATH_FFMA).describe()["passes"] == 1


def test_operands_that_are_matrices_are_marked_as_boxes(pkg):
    """An operand is a TMA box tensor when it is a plain matrix: contraction index fastest with the externals
    contiguous among themselves (tma_x / tma_y, fp64 and fp32), or the external class one contiguous run with the
    contraction index at a constant pitch (tma_xe / tma_ye, fp32).  Rows must be 16 bytes apart or more."""
    def flags(expr, dt):
        d = pkg.Plan(expr, dt).describe()
        return tuple(bool(d[k]) for k in ("tma_x", "tma_y", "tma_xe", "tma_ye"))
    assert flags("C [a,512,b,512] += sum(c,256) * A [c,a] * B [c,b];", pkg.F32) == (True, True, False, False)
    assert flags("C [a,512,b,512] += sum(c,256) * A [a,c] * B [b,c];", pkg.F32) == (False, False, True, True)
    assert flags("C [a,512,b,512] += sum(c,256) * A [c,a] * B [b,c];", pkg.F32) == (True, False, False, True)
    assert flags("C [a,512,b,512] += sum(c,256) * A [c,a] * B [b,c];", pkg.F64) == (True, False, False, False)
    # rows of 250 floats are not 16 bytes apart; 250 doubles are
    assert flags("C [a,512,b,512] += sum(c,250) * A [c,a] * B [c,b];", pkg.F32) == (False, False, False, False)
    assert flags("C [a,512,b,512] += sum(c,250) * A [c,a] * B [c,b];", pkg.F64) == (True, True, False, False)
    # fused externals stay a box while they are contiguous among themselves; a permuted pair is not
    assert flags("C [a,64,b,8,c,512] += sum(d,64) * A [d,a,b] * B [d,c];", pkg.F32)[0]
    assert not flags("C [a,64,b,8,c,512] += sum(d,64) * A [d,b,a] * B [d,c];", pkg.F32)[0]
    assert flags("C [a,64,b,8,c,512] += sum(d,64) * A [a,b,d] * B [d,c];", pkg.F32)[2]
