"""In-tree build of libschedforge_b200.so (sm_100a only).

    python -m schedforge_b200.build [--force] [--verbose]

Every source under csrc/ is compiled with nvcc to an object under csrc/_obj/ (rebuilt
only when the source or a header is newer) and linked into
schedforge_b200/libschedforge_b200.so.  The CUDA runtime is linked statically and the
driver API is reached through cudaGetDriverEntryPoint, so the library loads on a
machine without a GPU (it then fails at the first compute call).
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(PKG, "libschedforge_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++20", "-O3", "-lineinfo", *os.environ.get("SFB_EXTRA_NVCC", "").split(),
    "-Xcompiler", "-fPIC,-fvisibility=default,-pthread",
    "--expt-relaxed-constexpr",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found")
    return path


def host_compiler():
    # The distribution g++ links libstdc++ dynamically; see oracle/Makefile for why that matters.
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def sources():
    found = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    return found


def headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "host", "*.hpp")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))


def _compile(src, obj, verbose):
    cmd = [nvcc(), "-ccbin", host_compiler(), *NVCC_FLAGS, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{result.stdout}\n{result.stderr}")
    return result.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    newest_header = max((os.path.getmtime(h) for h in headers()), default=0.0)
    jobs, objects = [], []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src).rsplit(".", 1)[0] + ".o")
        objects.append(obj)
        stale = force or not os.path.exists(obj) or \
            os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header)
        if stale:
            jobs.append((src, obj))
    logs = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for log in pool.map(lambda job: _compile(job[0], job[1], verbose), jobs):
                logs.append(log)
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc(), "-ccbin", host_compiler(), "-shared", "-o", LIB, *objects,
               "-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    if verbose:
        print("\n".join(logs))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
