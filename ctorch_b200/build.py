"""Builds libctorch_b200.so (CUDA kernels + C ABI + C++ front end) in-tree with nvcc for sm_100a.

    python -m ctorch_b200.build [--force] [--verbose]

Cross-compiles without a GPU.  The elementwise / reduction / row-wise files are compiled with
-fmad=false so that every product and sum is rounded on its own, as in the reference's chain of
single-op CPU kernels; intended fused multiply-adds are written as fmaf().
"""
import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OUT_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libctorch_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"),
          "-I", os.path.join(CSRC, "kernels", "CUDA"), "-I", os.path.join(CSRC, "host")]
NO_FMAD = {"elementwise.cu", "reduce.cu", "rowwise.cu"}


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built (there is no CPU fallback)")
    return exe


def sources():
    cu = sorted(os.path.join(CSRC, "kernels", "CUDA", f) for f in os.listdir(os.path.join(CSRC, "kernels", "CUDA")) if f.endswith(".cu"))
    host_dir = os.path.join(CSRC, "host")
    cpp = sorted(os.path.join(host_dir, f) for f in os.listdir(host_dir) if f.endswith(".cpp")) if os.path.isdir(host_dir) else []
    return cu + cpp


def _headers():
    hs = [os.path.join(ROOT, "include", "ctorch_b200.h")]
    for d in (os.path.join(CSRC, "kernels", "CUDA"), os.path.join(CSRC, "host")):
        if os.path.isdir(d):
            hs += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".h", ".cuh", ".hpp"))]
    return hs


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in sources() + _headers() + [os.path.abspath(__file__)])


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    jobs = []
    for src in sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        cmd = [nvcc] + ARCH + COMMON + ["-c", src, "-o", obj]
        if src.endswith(".cpp"):
            cmd = [nvcc] + ARCH + COMMON + ["-x", "cu", "-c", src, "-o", obj]
        if os.path.basename(src) in NO_FMAD:
            cmd.insert(1, "-fmad=false")
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        jobs.append((cmd, obj))

    def run(job):
        cmd, _ = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    link = [nvcc] + ARCH + ["-shared", "-o", LIB] + [o for _, o in jobs] + ["-ldl", "-lpthread"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(" ".join(link) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
