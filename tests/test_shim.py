"""The reference's generated entry point, sd_t_d2_fusion_, served by the library (drop-in boundary)."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "tests", "shim")


def _build_driver(pkg, tmp_path):
    exe = str(tmp_path / "k_shim")
    libdir = os.path.dirname(pkg.LIB_PATH)
    cmd = ["gcc", "-std=gnu89", "-w", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(SHIM, "driver.c"),
           os.path.join(SHIM, "entry.c"), "-L", libdir, "-ltc_b200", "-Wl,-rpath," + libdir, "-o", exe]
    subprocess.run(cmd, check=True)
    return exe


def test_driver_in_the_reference_style_links_against_the_shim(pkg, tmp_path):
    exe = _build_driver(pkg, tmp_path)  # compile + link only: no GPU needed
    out = subprocess.run(["nm", "-D", "--defined-only", pkg.LIB_PATH], capture_output=True, text=True).stdout
    assert " tc_sd_t_d2_fusion" in out
    assert "sd_t_d2_fusion_" in subprocess.run(["nm", exe], capture_output=True, text=True).stdout


@pytest.mark.gpu
def test_reference_style_driver_end_to_end(pkg, orc, tmp_path):
    exe = _build_driver(pkg, tmp_path)
    ext = {"a": 40, "b": 9, "c": 21, "d": 33}
    expr = orc.with_extents("t3 [a,16,b,16,c,16] += sum(d,16) * t2 [d,c,a] * v2 [b,d];", ext)
    c0, a, b = orc.make_inputs(expr, 55)
    ref = orc.contract(expr, c0.copy(), a, b)
    paths = [str(tmp_path / n) for n in ("c.bin", "a.bin", "b.bin", "out.bin")]
    for arr, p in zip((c0, a, b), paths):
        arr.tofile(p)
    r = subprocess.run([exe] + [str(ext[i]) for i in "abcd"] + paths, capture_output=True, text=True)
    assert r.returncode == 0 and r.stderr == "", r.stderr
    got = np.fromfile(paths[3])
    assert orc.rel_error(got, ref) <= 1e-12


@pytest.mark.gpu
def test_entry_through_the_c_abi_caches_plans(pkg, orc):
    for dt, tol, code in ((np.float64, 1e-12, 0), (np.float32, 1e-5, 1)):
        expr = "t3 [a,16,b,16,c,16,d,16] -= sum(e,16,f,16) * t2 [e,a,f,c] * v2 [b,f,d,e];"
        sizes = [6, 5, 7, 3, 9, 4]
        actual = orc.with_extents(expr, dict(zip("abcdef", sizes)))
        c0, a, b = orc.make_inputs(actual, 56, dt)
        ref = orc.contract(actual, c0.copy(), a, b)
        ref2 = orc.contract(actual, ref.copy(), a, b)
        c = c0.copy()
        pkg.sd_t_d2_fusion(expr, sizes, c, a, b, dtype=code)
        assert orc.rel_error(c, ref) <= tol
        pkg.sd_t_d2_fusion(expr, sizes, c, a, b, dtype=code)  # second call reuses the cached plan
        assert orc.rel_error(c, ref2) <= tol
    with pytest.raises(pkg.TcError) as e:
        pkg.sd_t_d2_fusion("t3 [a,16] += sum(d,16) * t2 [d,a] * v2 [d];", [4, 5, 6], np.zeros(4), np.zeros(20), np.zeros(5))
    assert e.value.status == 2


# ---------------------------------------- the reference's own drivers, unmodified ----
def _driver_report(stdout):
    """(passed, errors, total) from the report the reference's post_Correctness prints
    (cogent/drivers/tccg/code_main_tccg_02.c:154-155)."""
    import re
    ok = re.search(r">>> PASSED:\s*([\d,']+) among\s*([\d,']+)", stdout)
    bad = re.search(r">>> ERROR :\s*([\d,']+) among", stdout)
    num = lambda m, g: int(re.sub(r"[,']", "", m.group(g)))
    return num(ok, 1), num(bad, 1), num(ok, 2)


def _run_driver(orc, tag, sizes):
    exe = os.path.join(ROOT, "oracle", "_ref", "k_" + tag)
    r = subprocess.run([exe] + [str(x) for x in sizes], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stderr == "", (tag, r.stderr[-500:])
    return _driver_report(r.stdout)


@pytest.mark.gpu
def test_every_unmodified_reference_driver_passes_its_own_check(pkg, orc):
    """All 57 driver files of the reference (cogent/drivers/tccg, tccg-float), compiled unchanged with their
    correctness check switched on (-DDEBUG_CORRECTNESS) and linked against libtc_b200.so through the shim header:
    their own main() allocates with malloc, fills with rand(), calls sd_t_d2_fusion_ and compares with its CPU loop
    nest (epsilon 1e-8 fp64, 1e-5 fp32).  The executables are built where the reference tree is present."""
    if not orc.ref_available() or not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "k_f64_02")):
        pytest.skip("the reference's drivers are not built here (oracle/_ref absent)")
    rng = np.random.default_rng(5)
    for tag, info in sorted(orc.ref_table().items()):
        sizes = [int(rng.integers(5, 13)) for _ in info["size_args"]]
        passed, errors, total = _run_driver(orc, tag, sizes)
        assert errors == 0 and passed == total == int(np.prod(sizes[:len(sizes) - _n_sum(info)])), (tag, sizes, passed, errors, total)


def _n_sum(info):
    return len(info["expr"].split("sum(")[1].split(")")[0].split(",")) // 2


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["f64_02", "f64_05", "f64_31", "f64_40", "f32_40", "f32_48"])
def test_unmodified_reference_driver_at_the_reference_bench_sizes(pkg, orc, tag):
    """The same executables with the problem sizes the reference's bench script passes them (cogent/bench_tccg.sh:5-54)."""
    if not orc.ref_available() or not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "k_" + tag)):
        pytest.skip("the reference's drivers are not built here (oracle/_ref absent)")
    info = orc.ref_table()[tag]
    passed, errors, total = _run_driver(orc, tag, info["bench_sizes"])
    assert errors == 0 and passed == total > 0, (tag, passed, errors, total)
