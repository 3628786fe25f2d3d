"""Build recipe: compile the reference's self-contained kernel sources as host C++.

The three sources (hash table, kernel map, Morton code) only use a handful of
CUDA builtins, which ``ref_shim/cuda_cpu_shim.h`` supplies.  They are compiled
directly from where they lie in the reference tree; outputs go to
``oracle/_ref/`` only.  Test infrastructure: the product never loads these.

Usage: ``python -m oracle.ref_build [REFERENCE_ROOT]``
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SHIM = os.path.join(HERE, "ref_shim")

TARGETS = {
    "libref_hashmap.so": ("ref_hashmap_driver.cpp", "warpconvnet/csrc/hashmap_kernels.cu"),
    "libref_discrete.so": ("ref_discrete_driver.cpp", "warpconvnet/csrc/discrete_kernels.cu"),
    "libref_morton.so": ("ref_morton_driver.cpp", "warpconvnet/csrc/morton_code.cu"),
}


def default_reference_root():
    """Where the reference project is checked out: the WCN_REFERENCE_ROOT environment variable,
    else a directory named ``reference`` beside this repository if it holds the package.
    Neither means "not on this machine": nothing is built and the tests that need the compiled
    reference skip."""
    root = os.environ.get("WCN_REFERENCE_ROOT", "")
    if root:
        return root
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return sibling if os.path.isdir(os.path.join(sibling, "warpconvnet")) else ""


def build(reference_root=None, force=False, verbose=False):
    """Compile every target whose reference source exists. Returns the list built."""
    reference_root = reference_root or default_reference_root()
    built = []
    if not reference_root or not os.path.isdir(reference_root):
        return built
    os.makedirs(OUT, exist_ok=True)
    for lib, (driver, rel_src) in TARGETS.items():
        src = os.path.join(reference_root, rel_src)
        dst = os.path.join(OUT, lib)
        drv = os.path.join(SHIM, driver)
        if not os.path.isfile(src):
            continue
        if (not force and os.path.isfile(dst)
                and os.path.getmtime(dst) >= max(os.path.getmtime(src), os.path.getmtime(drv))):
            built.append(dst)
            continue
        cmd = ["g++", "-O2", "-shared", "-fPIC", "-x", "c++", "-I", SHIM,
               f'-DREF_SRC="{src}"', drv, "-o", dst]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
        built.append(dst)
    return built


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else None
    for p in build(root, force=True, verbose=True):
        print("built", p)
