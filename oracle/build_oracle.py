"""Builds the checker libraries (test infrastructure, never the product path).

  oracle/liboracle.so          the C restatement in tc_oracle.c
  oracle/_ref/libref_nests.so  the reference's OWN loop nests, compiled from the
                               57 driver files where they lie in the reference
                               tree (cogent/drivers/tccg/*.c, tccg-float/*.c),
                               only when that tree is present
  oracle/_ref/ref_nests.json   what each compiled nest computes, recovered from
                               its code (not from its comments, which disagree
                               with the code in places), plus the problem sizes
                               the reference's bench script runs it with
  oracle/_ref/k_<tag>          the reference's UNMODIFIED drivers compiled with
                               -DDEBUG_CORRECTNESS (their own checker switched
                               on) and linked against the product library
                               through include/tc_b200_shim.h, so that the
                               drop-in symbol is exercised by the reference's
                               own main() and checked by its own report

No reference source is copied: every driver is compiled in place with its
`main`, `post_Correctness` and `pre_Initializing_Input_Tensors` renamed through
-D so that all of them fit in one shared object; the generated entry they call
(`sd_t_d2_fusion_`) is stubbed.  gcc is used directly (-std=gnu89: the drivers
rely on implicit declarations and K&R prototypes).

Usage: python oracle/build_oracle.py [--reference DIR]
"""
import json
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference tree sits beside the repository ("reference" next to the repository's folder) unless TC_REFERENCE_ROOT says otherwise
REF_DEFAULT = os.environ.get("TC_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
REF_OUT = os.path.join(HERE, "_ref")
LIB_ORACLE = os.path.join(HERE, "liboracle.so")
LIB_REF = os.path.join(REF_OUT, "libref_nests.so")
JSON_REF = os.path.join(REF_OUT, "ref_nests.json")


def build_oracle():
    src = os.path.join(HERE, "tc_oracle.c")
    if os.path.exists(LIB_ORACLE) and os.path.getmtime(LIB_ORACLE) >= os.path.getmtime(src):
        return LIB_ORACLE
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-std=c99", src, "-o", LIB_ORACLE]
    subprocess.run(cmd, check=True)
    return LIB_ORACLE


_IDX = re.compile(r"(?<!size_)idx_(\w+)")


def describe_driver(path):
    """Recovers (expression, size-argument order) from a driver's post_Correctness CODE."""
    text = open(path).read()
    body = text[text.rindex("void post_Correctness("):]  # the definition (the prototype comes first)
    sig = body[:body.index(")") + 1]
    is_float = "float* h_C" in sig or "float *h_C" in sig
    size_args = re.findall(r"int\s+size_idx_(\w+)", sig)
    loops = re.findall(r"for\s*\(\s*idx_(\w+)\s*=\s*0", body)
    m = re.search(r"tmp_r_idx\s*=\s*([^;]+);", body)
    out_idx = _IDX.findall(m.group(1))
    m = re.search(r"h_C_chk\[tmp_r_idx\]\s*([+-])=\s*h_A\[(.*?)\]\s*\*\s*h_B\[(.*?)\];", body, re.S)
    op = m.group(1) + "="
    a_idx = _IDX.findall(m.group(2))
    b_idx = _IDX.findall(m.group(3))
    sum_idx = [i for i in loops if i not in out_idx]
    assert loops[:len(out_idx)] == out_idx, (path, loops, out_idx)  # output loops outermost, in output order
    assert sorted(size_args) == sorted(out_idx + sum_idx), (path, size_args, out_idx, sum_idx)
    expr = "t3 [%s] %s sum(%s) * t2 [%s] * v2 [%s];" % (
        ",".join("%s,16" % i for i in out_idx), op, ",".join("%s,16" % i for i in sum_idx),
        ",".join(a_idx), ",".join(b_idx))
    return {"expr": expr, "size_args": size_args, "dtype": "f32" if is_float else "f64"}


def build_ref(reference=REF_DEFAULT):
    drivers = []
    for sub, tag in (("tccg", "f64"), ("tccg-float", "f32")):
        d = os.path.join(reference, "cogent", "drivers", sub)
        if not os.path.isdir(d):
            continue
        for f in sorted(os.listdir(d)):
            mm = re.match(r"code_main_tccg_(\d+)\.c$", f)
            if mm:
                drivers.append(("%s_%s" % (tag, mm.group(1)), os.path.join(d, f)))
    if not drivers:
        return None
    os.makedirs(REF_OUT, exist_ok=True)
    objs, table = [], {}
    for tag, path in drivers:
        info = describe_driver(path)
        info["symbol"] = "ref_post_" + tag
        info["source"] = os.path.relpath(path, reference)
        table[tag] = info
        obj = os.path.join(REF_OUT, tag + ".o")
        cmd = ["gcc", "-std=gnu89", "-O2", "-ffp-contract=off", "-w", "-fPIC", "-c", path, "-o", obj,
               "-Dmain=ref_main_" + tag, "-Dpost_Correctness=ref_post_" + tag,
               "-Dpre_Initializing_Input_Tensors=ref_pre_" + tag]
        subprocess.run(cmd, check=True)
        objs.append(obj)
    stub = os.path.join(REF_OUT, "stub.c")
    with open(stub, "w") as f:
        f.write("/* generated: the drivers' call into the generated GPU entry does nothing here */\n"
                "void sd_t_d2_fusion_() {}\n")
    subprocess.run(["gcc", "-std=gnu89", "-w", "-shared", "-fPIC", "-o", LIB_REF, stub] + objs, check=True)
    for o in objs:
        os.remove(o)
    with open(JSON_REF, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    return LIB_REF


def bench_sizes(reference):
    """Problem sizes per item from the reference's bench script (cogent/bench_tccg.sh:5-54): item number -> ints."""
    path = os.path.join(reference, "cogent", "bench_tccg.sh")
    if not os.path.exists(path):
        return {}
    out = {}
    for m in re.finditer(r'"([\d ]+)"\s*\)?\s*#\s*(\d+)', open(path).read()):
        out[int(m.group(2))] = [int(x) for x in m.group(1).split()]
    return out


def build_drivers(reference=REF_DEFAULT):
    """Links every reference driver, unchanged and with its own correctness check enabled, against the product
    library: one generated translation unit per driver defines sd_t_d2_fusion_ through the shim header."""
    if not os.path.exists(JSON_REF):
        return []
    root = os.path.dirname(HERE)
    libdir = os.path.join(root, "cgo2019-ae_b200")
    if not os.path.exists(os.path.join(libdir, "libtc_b200.so")):
        return []
    table = json.load(open(JSON_REF))
    sizes = bench_sizes(reference)
    built = []
    for tag, info in sorted(table.items()):
        src = os.path.join(reference, info["source"])
        n = len(info["size_args"])
        # the driver passes its sizes in the order of its own call; recover that order from the call site
        call = re.search(r"sd_t_d2_fusion_\(([^;]*?)\);", open(src).read(), re.S).group(1)
        order = re.findall(r"size_idx_(\w+)", call)
        p_out = re.findall(r"(\w+),16", info["expr"].split("sum(")[0])
        p_sum = re.findall(r"(\w+),16", info["expr"].split("sum(")[1].split(")")[0])
        assert order == p_out + p_sum, (tag, order, p_out, p_sum)  # output indices in written order, then sum(...)
        ctype, dt = ("float", "TC_F32") if info["dtype"] == "f32" else ("double", "TC_F64")
        unit = os.path.join(REF_OUT, "entry_%s.c" % tag)
        with open(unit, "w") as f:
            f.write('/* generated */\n#include "tc_b200_shim.h"\nTC_DEFINE_SD_T_D2_FUSION_%d("%s", %s, %s)\n'
                    % (n, info["expr"], ctype, dt))
        exe = os.path.join(REF_OUT, "k_" + tag)
        cmd = ["gcc", "-std=gnu89", "-w", "-O2", "-DDEBUG_CORRECTNESS", "-I", os.path.join(root, "include"), src, unit,
               "-L", libdir, "-ltc_b200", "-Wl,-rpath,$ORIGIN/../../cgo2019-ae_b200", "-o", exe]
        subprocess.run(cmd, check=True)
        os.remove(unit)
        info["driver"] = "k_" + tag
        num = int(tag.split("_")[1])
        if info["dtype"] == "f64" and num in sizes and len(sizes[num]) == n:
            info["bench_sizes"] = sizes[num]
        elif info["dtype"] == "f32" and num in sizes and len(sizes[num]) == n:
            info["bench_sizes"] = sizes[num]   # the fp32 items 40-48 run with the sizes of the fp64 items of the same number
        built.append(exe)
    with open(JSON_REF, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    return built


def build_all(reference=REF_DEFAULT):
    out = [build_oracle()]
    if os.path.isdir(reference):
        out.append(build_ref(reference))
        out += build_drivers(reference)
    return out


if __name__ == "__main__":
    ref = REF_DEFAULT
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build_all(ref))
