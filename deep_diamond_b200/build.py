"""Builds libdd_b200.so (the C-ABI library of hand-written sm_100a kernels) in-tree with nvcc.

Usage: python deep_diamond_b200/build.py [--force]
(run as a script: importing the package itself needs the built library).  The library has no
Python or torch dependency; it links the CUDA runtime statically.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libdd_b200.so")
OBJ = os.path.join(HERE, "_obj")
# `--tune` builds libdd_b200_tune.so with -DDD_TUNE (launch-plan overrides read from the environment,
# for parameter sweeps); the package loads it when DD_B200_LIBRARY names it.
if "--tune" in sys.argv:
    OUT = os.path.join(HERE, "libdd_b200_tune.so")
    OBJ = os.path.join(HERE, "_obj", "tune")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
] + (["-DDD_TUNE"] if "--tune" in sys.argv else [])


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    hdrs.append(os.path.join(HERE, "..", "include", "dd_b200.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src, force, hdr_mtime):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    srcp = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) > max(os.path.getmtime(srcp), hdr_mtime)):
        return obj
    cmd = [_nvcc()] + NVCC_FLAGS + ["-c", srcp, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return obj


def build(force=False, verbose=True):
    os.makedirs(OBJ, exist_ok=True)
    hdr_mtime = _deps_mtime()
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, hdr_mtime), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(OUT) or os.path.getmtime(OUT) < newest:
        tmp = OUT + ".partial"  # linked beside the target and renamed over it: a reader never sees half a file
        cmd = [_nvcc(), "-shared", "-o", tmp] + objs + [
            "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl",
            "-Xlinker", "--no-undefined",
        ]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
        os.replace(tmp, OUT)
    if verbose:
        print("built", OUT)
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv)
