"""Makes baseline/_ref/tccg_items.json: the reference's own benchmark list, read where it lies.

Per item (48 fp64 + the 9 fp32 repeats of items 40-48): the expression line of
cogent/input_strings/tccg/input_tccg_NN.in, the problem sizes cogent/bench_tccg.sh:5-54 (fp32:
cogent/bench_fb.sh) passes to its driver, and the kernel-only GFLOPS the reference publishes for its generated
kernels on V100 and P100 (cogent/expect_{v100,p100}_cogent_{tccg,fb}_results.txt; the fp32 files count ONE
operation per multiply-add, cogent/src/codes/kernels/tc_interface.py:304-307, so they are doubled here) and for
the NWChem-generated kernels (nwchem-tccg/expect_v100_nwchem_tccg_results.txt).
The list itself is the reference's; it is read from the reference tree and written to a folder git ignores.

Usage:  python baseline/make_tccg_table.py [--reference DIR]
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REF_DEFAULT = os.environ.get("TC_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _sizes(path):
    out = {}
    if os.path.exists(path):
        for m in re.finditer(r'"([\d ]+)"\s*\)?\s*#\s*(\d+)', open(path).read()):
            out[int(m.group(2))] = [int(x) for x in m.group(1).split()]
    return out


def _published(path, scale=1.0):
    out = {}
    if os.path.exists(path):
        for m in re.finditer(r"tccg-\s*(\d+)\s*>>.*?time\(ms\):\s*([\d.]+).*?GFLOPS:\s*([\d.]+)", open(path).read()):
            out[int(m.group(1))] = {"ms": float(m.group(2)), "gflops": float(m.group(3)) * scale}
    return out


def _line(path):
    for line in open(path):
        if line.strip() and not line.startswith("#"):
            return line.strip()
    return None


def build(reference=REF_DEFAULT):
    cg = os.path.join(reference, "cogent")
    if not os.path.isdir(cg):
        return None
    os.makedirs(OUT, exist_ok=True)
    s64, s32 = _sizes(os.path.join(cg, "bench_tccg.sh")), _sizes(os.path.join(cg, "bench_fb.sh"))
    pub = {
        "f64": {"cogent_v100": _published(os.path.join(cg, "expect_v100_cogent_tccg_results.txt")),
                "cogent_p100": _published(os.path.join(cg, "expect_p100_cogent_tccg_results.txt")),
                "nwchem_v100": _published(os.path.join(reference, "nwchem-tccg", "expect_v100_nwchem_tccg_results.txt"))},
        "f32": {"cogent_v100": _published(os.path.join(cg, "expect_v100_cogent_fb_results.txt"), 2.0),
                "cogent_p100": _published(os.path.join(cg, "expect_p100_cogent_fb_results.txt"), 2.0)},
    }
    items = []
    for dtype, sizes, nums in (("f64", s64, range(1, 49)), ("f32", s32, range(40, 49))):
        for n in nums:
            line = _line(os.path.join(cg, "input_strings", "tccg", "input_tccg_%02d.in" % n))
            if line is None or n not in sizes:
                continue
            tok = line.replace("[", "").replace("]", "").replace(";", "").split()
            names = tok[1].split(",")[0::2] + tok[3][4:-1].split(",")[0::2]
            if len(names) != len(sizes[n]):
                continue
            item = {"tag": "%s_%02d" % (dtype, n), "dtype": dtype, "line": line, "extents": dict(zip(names, sizes[n]))}
            for k, table in pub[dtype].items():
                if n in table:
                    item[k + "_gflops"] = table[n]["gflops"]
            items.append(item)
    path = os.path.join(OUT, "tccg_items.json")
    with open(path, "w") as f:
        json.dump(items, f, indent=1)
    return path


if __name__ == "__main__":
    ref = REF_DEFAULT
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build(ref))
