"""Builds ``libjgpt_b200.so`` in-tree with nvcc for sm_100a (no torch, no JIT cache).

    python -m jgpt_b200.build [--force] [--verbose]

One object per ``csrc/*.cu`` (compiled in parallel), linked into ``jgpt_b200/lib/libjgpt_b200.so``
with the CUDA runtime linked statically, so the library depends on the driver only.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libjgpt_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
          "-Xcompiler", "-Wall", "-ccbin", "/usr/bin/g++"]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps_mtime():
    files = _sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(f) for f in files)


def _compile(src: str, verbose: bool, defines=(), tag: str = "") -> str:
    obj = os.path.join(LIBDIR, os.path.basename(src)[:-3] + tag + ".o")
    cmd = [NVCC, *ARCH, *CFLAGS, *[f"-D{d}" for d in defines], "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    elif r.stderr.strip():
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    if not os.path.exists(NVCC):
        raise RuntimeError(f"nvcc not found at {NVCC}; libjgpt_b200.so cannot be built")
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), _sources()))
    cmd = [NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-ccbin", "/usr/bin/g++", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


TRACE_LIB = os.path.join(LIBDIR, "libjgpt_b200_trace.so")


def build_trace() -> str:
    """The same library with in-kernel phase timing compiled into the decode-attention kernel
    (``-DJGPT_B200_DECODE_TRACE``): every CTA records when it started, when its first K/V slab arrived, when its block
    loop ended and when it left.  For ``bench.py --workload phases`` only; never the library a host should load."""
    os.makedirs(LIBDIR, exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, False, ("JGPT_B200_DECODE_TRACE",), ".trace"), _sources()))
    r = subprocess.run([NVCC, *ARCH, "-shared", "-o", TRACE_LIB, *objs, "-ccbin", "/usr/bin/g++", "-ldl"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    for o in objs:
        os.remove(o)
    return TRACE_LIB


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build_trace())
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
