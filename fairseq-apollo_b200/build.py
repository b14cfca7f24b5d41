"""Builds libmega_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python fairseq-apollo_b200/build.py [--force] [--verbose]

The library has no torch or Python dependency: plain ``extern "C"`` entry points declared in
``include/mega_b200.h``.  Objects and the shared library land next to the sources' package
directory (git-ignored) so they travel with a copy of the tree.
"""
import argparse
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libmega_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "-Xptxas", "-v"]
# Per-file additions.  The step loop of the segmented tensor-core forms lives at the register limit; with ptxas'
# most aggressive register usage level it runs 2.7 % faster (5.28 -> 5.14 ms on B=64, L=32768, D=2048), while the
# other forms of the same kernel are 3 % slower with it, hence a translation unit of their own.
# The forms with narrow tiles (mma_cl_narrow.cu) gain ~2 % from a low level instead (shards of 8 and 16 sequences).
FILE_FLAGS = {"mma_cl_seg.cu": ["-Xptxas", "--register-usage-level=10"],
              "mma_cl_narrow.cu": ["-Xptxas", "--register-usage-level=2"]}


def nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def newest_dep():
    deps = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(ROOT, "include", "mega_b200.h"))
    return max(os.path.getmtime(d) for d in deps)


def build(force=False, verbose=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= newest_dep():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    cc = nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [cc, "-c", src, "-o", obj, "-I", os.path.join(ROOT, "include"), "-I", CSRC] + ARCH + NVCC_FLAGS + \
            FILE_FLAGS.get(os.path.basename(src), [])
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for src, p in procs:
        out, _ = p.communicate()
        log.append("== %s\n%s" % (os.path.basename(src), out))
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError("nvcc failed on %s" % src)
    with open(os.path.join(OBJ, "ptxas.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    cmd = [cc, "-shared", "-o", LIB] + objs + ARCH + ["-Xcompiler", "-fPIC", "-cudart", "static"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
