"""In-tree build of the sm_100a kernel library (``libeasyllm_b200.so``) with nvcc.

Every ``csrc/*.cu`` is compiled for ``compute_100a/sm_100a`` (cross-compiles without a GPU)
and linked into one shared object beside this file, which ``ops.cuda`` loads with ctypes.
The entry points are plain ``extern "C"`` launchers taking raw device pointers and a CUDA
stream, so the library has no dependency on the PyTorch C++ ABI and builds in seconds.

    python -m easyllm_b200.ops.build [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(HERE, "libeasyllm_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest(path, flags):
    h = hashlib.sha1(" ".join(flags).encode())
    for p in [path] + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))):
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def build(force=False, verbose=False, extra_flags=()):
    """Compile stale objects in parallel and relink.  Returns the library path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    flags = NVCC_FLAGS + list(extra_flags)
    jobs, objs = [], []
    for src in sources():
        base = os.path.splitext(os.path.basename(src))[0]
        obj = os.path.join(OBJ_DIR, base + ".o")
        stamp = obj + ".sha1"
        dig = _digest(src, flags)
        objs.append(obj)
        fresh = os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig
        if force or not fresh:
            jobs.append((src, obj, stamp, dig))

    def compile_one(job):
        src, obj, stamp, dig = job
        cmd = [nvcc] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-I", CSRC, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        with open(stamp, "w") as f:
            f.write(dig)
        return src

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for done in ex.map(compile_one, jobs):
                if verbose:
                    print("compiled", done)
    if jobs or not os.path.exists(LIB_PATH):
        cmd = [nvcc, "-shared", "-cudart", "static", "-o", LIB_PATH] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
