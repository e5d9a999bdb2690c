"""Builds libtrain_station_b200.so in-tree with nvcc for sm_100a.

Usage: python train-station_b200/build.py [--force]
The shared library has a plain C ABI (include/train_station_b200.h) and depends only on
the CUDA runtime (linked statically) and NCCL.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtrain_station_b200.so")
SOURCES = ["runtime.cu", "elementwise.cu", "reduce.cu", "reduce_dims.cu", "softmax.cu", "transform.cu", "adam.cu", "sgemm.cu", "thin_gemm.cu", "gemm_tcgen05.cu", "engine.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the library cannot be built (there is no CPU fallback)")


STAMP = LIB + ".stamp"


def _source_digest() -> str:
    """Hash of everything the library is made from.  Contents, not timestamps: a copy of the tree to another
    machine keeps the binary valid whatever it does to modification times."""
    import hashlib
    h = hashlib.sha256()
    deps = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)) + [
        os.path.join(HERE, "..", "include", "train_station_b200.h"), os.path.abspath(__file__)]
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def needs_build() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(STAMP):
        return True
    with open(STAMP) as f:
        return f.read().strip() != _source_digest()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    import hashlib
    shared = b""
    for dep in (os.path.join(CSRC, "common.h"), os.path.join(HERE, "..", "include", "train_station_b200.h"), os.path.abspath(__file__)):
        with open(dep, "rb") as f:
            shared += f.read()
    procs, objs = [], []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        with open(os.path.join(CSRC, src), "rb") as f:
            digest = hashlib.sha256(shared + f.read()).hexdigest()
        stamp = obj + ".stamp"
        if not force and not verbose and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
            continue   # this translation unit and everything it includes are unchanged
        cmd = [nvcc, *ARCH, *CFLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, stamp, digest, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = None
    for src, stamp, digest, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = failed or f"nvcc failed on {src}:\n{out}"
            continue
        if verbose and out:
            print(out)
        with open(stamp, "w") as f:
            f.write(digest + "\n")
    if failed:
        raise RuntimeError(failed)
    # NCCL is opened with dlopen when data parallelism is first used (see engine.cu), so it is not linked here
    link = [nvcc, *ARCH, "-shared", "-o", LIB, *objs, "-ldl", "-Xcompiler", "-fPIC"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    with open(STAMP, "w") as f:
        f.write(_source_digest() + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
