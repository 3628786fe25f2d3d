"""Build libwcn_b200.so in this folder with nvcc for sm_100a (no other architecture).

Usage: ``python -m warpconvnet_b200.csrc.build [--force] [--verbose]``
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["api.cu", "hash_kmap.cu", "brick_kmap.cu", "conv_explicit.cu", "conv_simt.cu", "conv_tcgen05.cu",
           "conv_wgrad_tcgen05.cu", "conv_rows_tcgen05.cu"]
HEADERS = ["wcn_common.cuh", "tcgen05_common.cuh", os.path.join("..", "..", "include", "wcn_b200.h")]
LIB = os.path.join(HERE, "libwcn_b200.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isfile(cand) or cand == "nvcc"):
            return cand
    return "nvcc"


def needs_build():
    if not os.path.isfile(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, ptxas_info=False):
    if not force and not needs_build():
        return LIB
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for s in SOURCES:
        obj = os.path.join(HERE, s.replace(".cu", ".o"))
        cmd = [_nvcc(), *flags, "-c", os.path.join(HERE, s), "-o", obj]
        if verbose:
            print(" ".join(cmd))
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for s, pr in procs:
        out, _ = pr.communicate()
        if out.strip() and (verbose or ptxas_info or pr.returncode != 0):
            print(out)
        if pr.returncode != 0:
            failed = True
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart", "-Xlinker", "-rpath=/usr/local/cuda/lib64"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_info="--ptxas" in sys.argv))
