"""Builds libflagattn_b200.so in-tree with nvcc for sm_100a.

Every .cu file under csrc/ is compiled to an object (in parallel, skipped when
the object is newer than all sources and headers) and linked into
flagattention_b200/lib/libflagattn_b200.so with the CUDA runtime linked
statically, so the library loads on a machine without a GPU or a CUDA
installation (symbol checks) and needs only the driver to run.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libflagattn_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; cannot build libflagattn_b200.so")
    return path


def _sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith(".cu"):
                out.append(os.path.join(root, f))
    return sorted(out)


def _headers_mtime():
    newest = 0.0
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    for f in os.listdir(INCLUDE):
        newest = max(newest, os.path.getmtime(os.path.join(INCLUDE, f)))
    return newest


def _compile_one(nvcc, src, obj, verbose):
    cmd = [nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, res.stdout, res.stderr))
    if verbose:
        print("compiled", os.path.relpath(src, PKG_DIR), flush=True)
    return obj


def build(force=False, verbose=False):
    """Compiles what is out of date and links the shared library. Returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = _headers_mtime()
    jobs, objs = [], []
    for src in _sources():
        rel = os.path.relpath(src, CSRC).replace(os.sep, "__")
        obj = os.path.join(OBJ_DIR, rel[:-3] + ".o")
        objs.append(obj)
        stale = (force or not os.path.exists(obj)
                 or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time))
        if stale:
            jobs.append((src, obj))
    if jobs:
        workers = max(1, min(len(jobs), os.cpu_count() or 1))
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, verbose) for s, o in jobs]
            for f in futs:
                f.result()
    need_link = (jobs or not os.path.exists(LIB_PATH)
                 or any(os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs))
    if need_link:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "static", "-o", LIB_PATH] + objs
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
        if verbose:
            print("linked", LIB_PATH, flush=True)
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
