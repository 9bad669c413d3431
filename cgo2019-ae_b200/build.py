"""Builds libtc_b200.so (the C-ABI library with every sm_100a kernel) in-tree, and beside it
probes/libtc_probes.so (pipe-peak microbenchmarks the bench uses for roofline denominators; not part
of the product library).

Usage:  python build.py [--force] [--verbose]
Each .cu/.cpp under csrc/ is compiled to an object in csrc/_obj/ (in parallel,
only when older than its sources) and linked into ../libtc_b200.so next to this
file.  nvcc cross-compiles for sm_100a without a GPU.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libtc_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
COMMON += os.environ.get("TC_NVCC_FLAGS", "").split()
PROBES_SRC = os.path.join(HERE, "probes", "tc_probes.cu")
PROBES_LIB = os.path.join(HERE, "probes", "libtc_probes.so")


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _generate_kernel_units():
    """One translation unit per line of csrc/tc_kernel_list.h (written only when its text changes)."""
    import re
    text = open(os.path.join(CSRC, "tc_kernel_list.h")).read()
    units = []
    for m in re.finditer(r"^\s*X\((\w+),\s*(\w+),\s*(\w+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+)\)", text, re.M):
        name, t, math, bm, bn, wm, wn, st, minb, _variant = m.groups()
        body = ('// generated from tc_kernel_list.h by build.py\n#include "../tc_inst.cuh"\n'
                "%s(tc_inst_%s, %s, %s, %s, %s, %s, %s, %s, %s)\n"
                % ("TC_DEFINE_INST_KV" if math == "TC_MATH_TF32TC" else "TC_DEFINE_INST", name, t, math, bm, bn, wm, wn, st, minb))
        path = os.path.join(OBJ, "gen_%s.cu" % name)
        if not os.path.exists(path) or open(path).read() != body:
            with open(path, "w") as f:
                f.write(body)
        units.append(path)
    wt = text[text.index("#define TC_WT_KERNEL_LIST"):]
    for m in re.finditer(r"^\s*X\((\w+),\s*(\d+),\s*(\d+)\)", wt, re.M):
        name, bm, _variant = m.groups()
        body = ('// generated from tc_kernel_list.h by build.py\n#include "../tc_inst.cuh"\n'
                "TC_DEFINE_WT_INST(tc_inst_%s, %s)\n" % (name, bm))
        path = os.path.join(OBJ, "gen_%s.cu" % name)
        if not os.path.exists(path) or open(path).read() != body:
            with open(path, "w") as f:
                f.write(body)
        units.append(path)
    wc = text[text.index("#define TC_WC_KERNEL_LIST"):text.index("#define TC_WT_KERNEL_LIST")]
    for m in re.finditer(r"^\s*X\((\w+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+)\)", wc, re.M):
        name, bm, groups, wgm, wgn, st, _variant = m.groups()
        body = ('// generated from tc_kernel_list.h by build.py\n#include "../tc_inst.cuh"\n'
                "TC_DEFINE_WC_INST(tc_inst_%s, %s, %s, %s, %s, %s)\n" % (name, bm, groups, wgm, wgn, st))
        path = os.path.join(OBJ, "gen_%s.cu" % name)
        if not os.path.exists(path) or open(path).read() != body:
            with open(path, "w") as f:
                f.write(body)
        units.append(path)
    ws = text[text.index("#define TC_WS_KERNEL_LIST"):text.index("#define TC_WC_KERNEL_LIST")]
    for m in re.finditer(r"^\s*X\((\w+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+)\)", ws, re.M):
        name, bm, bn, st, _variant = m.groups()
        body = ('// generated from tc_kernel_list.h by build.py\n#include "../tc_inst.cuh"\n'
                "TC_DEFINE_WS_INST(tc_inst_%s, %s, %s, %s)\n" % (name, bm, bn, st))
        path = os.path.join(OBJ, "gen_%s.cu" % name)
        if not os.path.exists(path) or open(path).read() != body:
            with open(path, "w") as f:
                f.write(body)
        units.append(path)
    return units


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "tc_b200.h"))
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cpp"))]
    sources += _generate_kernel_units()
    jobs = []
    objs = []
    for path in sources:
        src = os.path.basename(path)
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if not force and _newer(obj, [path] + headers):
            continue
        cmd = [NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", path, "-o", obj]
        jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    failed = False
    with ThreadPoolExecutor(max_workers=max(1, os.cpu_count() or 1)) as ex:
        for src, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write("[%s]\n%s%s" % (src, r.stdout, r.stderr))
            failed = failed or r.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or jobs or not _newer(LIB, objs):
        cmd = [NVCC] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    if force or not _newer(PROBES_LIB, [PROBES_SRC]):
        cmd = [NVCC] + ARCH + COMMON + ["-shared", "-o", PROBES_LIB, PROBES_SRC, "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("probe library failed to build")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
