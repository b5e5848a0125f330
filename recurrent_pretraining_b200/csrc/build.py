"""Build the sm_100a kernel library in-tree with nvcc (no JIT cache, no torch headers).

``python -m recurrent_pretraining_b200.csrc.build`` compiles every ``.cu`` file of this directory to an object
file and links ``recurrent_pretraining_b200/_lib/libb200ops.so``.  nvcc cross-compiles, so this works on a
machine without a GPU.  Objects are rebuilt only when a source or header changed.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_DIR = os.path.join(PKG, "_lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libb200ops.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def sources() -> list[str]:
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cu"))


def headers() -> list[str]:
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def build(verbose: bool = False, force: bool = False) -> str:
    nvcc = find_nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = headers()
    jobs, objs = [], []
    for src in sources():
        tag = _digest([src] + hdrs)
        obj = os.path.join(OBJ_DIR, f"{os.path.basename(src)[:-3]}.{tag}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append((src, obj))
    if verbose:
        NVCC_FLAGS_V = NVCC_FLAGS + ["-Xptxas", "-v"]
    else:
        NVCC_FLAGS_V = NVCC_FLAGS

    def compile_one(job):
        src, obj = job
        stem = os.path.basename(src)[:-3]
        for old in os.listdir(OBJ_DIR):
            if old.startswith(stem + ".") and old.endswith(".o"):
                os.remove(os.path.join(OBJ_DIR, old))
        r = subprocess.run([nvcc, *NVCC_FLAGS_V, "-c", src, "-o", obj], capture_output=True, text=True)
        return src, r

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(compile_one, jobs):
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed for {src}")
    link_tag = _digest(objs) if all(os.path.exists(o) for o in objs) else ""
    stamp = os.path.join(LIB_DIR, "link.stamp")
    old = open(stamp).read() if os.path.exists(stamp) else ""
    if jobs or force or not os.path.exists(LIB_PATH) or old != link_tag:
        r = subprocess.run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
        with open(stamp, "w") as f:
            f.write(link_tag)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
