"""Builds go-inference_b200/liblthn_cuda.so for sm_100a with nvcc (in-tree).

    python go-inference_b200/build.py [--force] [--verbose]

The shared library is the product: a plain C ABI (include/lthn_cuda.h) over the
hand-written kernels in csrc/. Sources are compiled one object per file so an
edit only recompiles what changed.

A second library, liblthn_cuda_hooks.so, is linked from the very same objects plus
csrc/test_hooks.cu: it adds the lthn_debug_* entry points the parity tests use to force
each kernel variant. The product library does not contain them."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "liblthn_cuda.so")
OUT_HOOKS = os.path.join(HERE, "liblthn_cuda_hooks.so")
HOOK_SOURCES = ("test_hooks.cu",)
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=default"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _newer(a, b):
    return (not os.path.exists(b)) or os.path.getmtime(a) > os.path.getmtime(b)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "lthn_cuda.h"))
    hdr_time = max(os.path.getmtime(h) for h in headers)
    jobs = []
    for src in sources():
        sp = os.path.join(CSRC, src)
        op = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        if force or _newer(sp, op) or hdr_time > os.path.getmtime(op):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", sp, "-o", op]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    for out, srcs in ((OUT, [s for s in sources() if s not in HOOK_SOURCES]), (OUT_HOOKS, sources())):
        objs = [os.path.join(OBJ, os.path.splitext(s)[0] + ".o") for s in srcs]
        if jobs or force or not os.path.exists(out):
            cmd = [NVCC, "-shared", "-o", out] + objs + ["-lcudart", "-ldl", "-lpthread"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
