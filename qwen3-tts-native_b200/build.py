"""Builds libqwen3_tts_cuda.so (sm_100a only) next to this file.

    python qwen3-tts-native_b200/build.py [--force] [--verbose]

Every .cu under csrc/ is compiled to an object with nvcc and the objects are linked into
one shared library that exports only the C ABI declared in include/*.h.  No GPU is needed
to build.  `-Xptxas -v` output (registers, spills, shared memory) goes to
csrc/_build/ptxas.log.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(CSRC, "_build")
LIB = os.path.join(HERE, "libqwen3_tts_cuda.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xptxas", "-v", "-Xcompiler", "-fPIC",
          "-Xcompiler", "-fvisibility=hidden", "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def headers_mtime():
    newest = 0.0
    for folder in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(folder):
            if f.endswith((".cuh", ".hpp", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(folder, f)))
    return newest


def compile_one(name, force, hdr_time):
    src = os.path.join(CSRC, name)
    obj = os.path.join(OUT_DIR, name[:-3] + ".o")
    if (not force and os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(src)
            and os.path.getmtime(obj) > hdr_time):
        return name, "", False
    cmd = [NVCC, *ARCH, *CFLAGS, "-c", src, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name}:\n{proc.stdout}\n{proc.stderr}")
    return name, proc.stderr, True


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    hdr_time = headers_mtime()
    names = sources()
    logs = []
    rebuilt = False
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(names))) as pool:
        for name, log, did in pool.map(lambda n: compile_one(n, force, hdr_time), names):
            rebuilt = rebuilt or did
            if did:
                logs.append(f"==== {name}\n{log}")
    if logs:
        with open(os.path.join(OUT_DIR, "ptxas.log"), "a" if not force else "w") as f:
            f.write("\n".join(logs))
    if rebuilt or not os.path.exists(LIB):
        objs = [os.path.join(OUT_DIR, n[:-3] + ".o") for n in names]
        cmd = [NVCC, *ARCH, "-shared", "-o", LIB, *objs]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print("\n".join(logs))
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv or True)
