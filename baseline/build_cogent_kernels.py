"""Same-box GPU comparison: the reference's OWN generated CUDA kernels, compiled for sm_100.

For the benchmark configurations the reference generator can express (1-4; configuration 5 needs 64-bit
addressing, which its `int` index arithmetic does not have), this script
  1. copies the reference's generator (cogent/) into a scratch folder outside the repository,
  2. runs cogent/tc_code_generator.py there, exactly as cogent/tccg.sh:30-43 does, on the configuration's
     expression line with the tensors named t3 / t2 / v2 (the emitter hard-codes those names),
  3. compiles the emitted temp__NN.cu UNCHANGED with the flags of cogent/Makefile:7,16 (only the architecture
     becomes sm_100) into baseline/_ref/libcogent_<cfg>.so.
Timing: the emitted host wrapper does cudaMalloc / cudaMemcpy / launch / cudaMemcpy / cudaFree in one call.  A
header forced in front of it (-include) routes its cudaMemcpy calls through a wrapper that records a CUDA event
after the last host-to-device copy and before the device-to-host copy -- the kernel alone, what the reference's
own numbers count (nvprof kernel line, cogent/bench_tccg.sh:89-91) -- and silences its banner printfs.
Nothing of the reference is copied into the repository; baseline/_ref/ is built output and ignored by git.

Usage:  python baseline/build_cogent_kernels.py [--reference DIR]
"""
import json
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REF_DEFAULT = os.environ.get("TC_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

# the benchmark configurations in the reference's grammar, tensors renamed to what its emitter expects
CONFIGS = {
    "cfg1": ("t3 [i,64,j,48,k,32] += sum(l,40) * t2 [l,k,i] * v2 [j,l];", "DOUBLE"),
    "cfg2": ("t3 [a,96,b,96,c,96,d,96] += sum(e,96) * t2 [a,e,b,d] * v2 [e,c];", "DOUBLE"),
    "cfg3": ("t3 [a,64,b,64,c,64,d,64] += sum(e,64,f,64) * t2 [e,c,a,f] * v2 [b,f,d,e];", "DOUBLE"),
    "cfg4": ("t3 [a,24,b,24,c,24,i,24,j,24,k,24] += sum(l,24) * t2 [l,a,i,j] * v2 [b,c,k,l];", "FLOAT"),
}

PRELUDE = r'''
// Forced in front of the generated file: kernel-only timing and quiet banners.  Not part of the generated code.
#include <cuda_runtime.h>
#include <stdio.h>
static cudaEvent_t tc_ev0, tc_ev1;
static int tc_ev_ready = 0;
static float tc_kernel_ms = -1.f;
static inline cudaError_t tc_timed_memcpy(void* dst, const void* src, size_t n, cudaMemcpyKind kind) {
  if (!tc_ev_ready) { cudaEventCreate(&tc_ev0); cudaEventCreate(&tc_ev1); tc_ev_ready = 1; }
  if (kind == cudaMemcpyDeviceToHost) {
    cudaEventRecord(tc_ev1, 0);
    cudaEventSynchronize(tc_ev1);
    cudaEventElapsedTime(&tc_kernel_ms, tc_ev0, tc_ev1);
  }
  cudaError_t e = (cudaMemcpy)(dst, src, n, kind);
  if (kind == cudaMemcpyHostToDevice) cudaEventRecord(tc_ev0, 0);
  return e;
}
extern "C" float cogent_last_kernel_ms(void) { return tc_kernel_ms; }
extern "C" int cogent_last_error(void) { return (int)cudaGetLastError(); }
#define cudaMemcpy(dst, src, n, kind) tc_timed_memcpy(dst, src, n, kind)
#define printf(...) ((void)0)
'''


def build(reference=REF_DEFAULT, force=True):
    gen = os.path.join(reference, "cogent")
    if not os.path.isdir(gen):
        return []
    os.makedirs(OUT, exist_ok=True)
    libs = [os.path.join(OUT, "libcogent_%s.so" % name) for name in sorted(CONFIGS)]
    if not force and os.path.exists(os.path.join(OUT, "cogent_kernels.json")) and all(os.path.exists(x) for x in libs):
        return libs
    built, table = [], {}
    with tempfile.TemporaryDirectory(prefix="cogent_gen_") as scratch:
        work = os.path.join(scratch, "cogent")
        shutil.copytree(gen, work)
        prelude = os.path.join(scratch, "timing_prelude.h")
        with open(prelude, "w") as f:
            f.write(PRELUDE)
        for num, (name, (line, kind)) in enumerate(sorted(CONFIGS.items()), start=91):
            with open(os.path.join(work, "in_%s.in" % name), "w") as f:
                f.write(line + "\n")
            r = subprocess.run([sys.executable, "tc_code_generator.py", str(num), "in_%s.in" % name, "-1", "-1", kind],
                               cwd=work, capture_output=True, text=True)
            src = os.path.join(work, "temp__%d.cu" % num)
            if r.returncode != 0 or not os.path.exists(src):
                table[name] = {"error": "generator failed: " + (r.stderr or r.stdout)[-300:]}
                continue
            lib = os.path.join(OUT, "libcogent_%s.so" % name)
            cmd = [NVCC, "-O3", "-std=c++11", "-arch=sm_100", "--use_fast_math", "-Xptxas", "-dlcm=cg", "-include", prelude,
                   "-Xcompiler", "-fPIC", "-shared", "-o", lib, src, "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
            c = subprocess.run(cmd, capture_output=True, text=True)
            if c.returncode != 0:
                table[name] = {"error": "nvcc failed: " + c.stderr[-300:]}
                continue
            # the entry takes the sizes of the output indices in written order, then the contraction indices
            idx = [t.split(",")[0::2] for t in (line.split("[")[1].split("]")[0], line.split("sum(")[1].split(")")[0])]
            ext = [t.split(",")[1::2] for t in (line.split("[")[1].split("]")[0], line.split("sum(")[1].split(")")[0])]
            table[name] = {"lib": os.path.basename(lib), "dtype": "f32" if kind == "FLOAT" else "f64",
                           "sizes": [int(x) for x in ext[0] + ext[1]], "indices": idx[0] + idx[1], "expr": line}
            built.append(lib)
    with open(os.path.join(OUT, "cogent_kernels.json"), "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    return built


if __name__ == "__main__":
    ref = REF_DEFAULT
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build(ref))
