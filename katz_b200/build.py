"""Build recipe for libkatz_b200.so: every .cu under csrc/ compiled for sm_100a with nvcc and linked into one
C-ABI shared library next to this file. Runs without a GPU (nvcc cross-compiles)."""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libkatz_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-I", INCLUDE, "-I", CSRC,
]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_digest():
    h = hashlib.sha256()
    for root in (CSRC, INCLUDE):
        for f in sorted(os.listdir(root)):
            if f.endswith((".cuh", ".h")):
                with open(os.path.join(root, f), "rb") as fh:
                    h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(verbose=False, force=False, ptxas_info=False):
    """Compile out-of-date objects and relink. Returns the library path."""
    os.makedirs(BUILD, exist_ok=True)
    dep = _deps_digest()
    jobs = []
    objs = []
    for src in _sources():
        obj = os.path.join(BUILD, os.path.basename(src)[:-3] + ".o")
        stamp = obj + ".stamp"
        with open(src, "rb") as fh:
            digest = hashlib.sha256(fh.read() + dep.encode()).hexdigest()
        objs.append(obj)
        fresh = (not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest)
        if not fresh:
            jobs.append((src, obj, stamp, digest))

    def compile_one(job):
        src, obj, stamp, digest = job
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
        if ptxas_info:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        if verbose or ptxas_info:
            sys.stderr.write(r.stderr)
        with open(stamp, "w") as fh:
            fh.write(digest)
        return obj

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not os.path.exists(LIB):
        tmp = LIB + ".linking"          # linked under another name and renamed: a reader never sees half a library
        cmd = [_nvcc(), "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv))
