"""In-tree build of the CUDA library (nvcc, sm_100a only).

`python -m fuse_b200.build` compiles every translation unit under fuse_b200/csrc into
fuse_b200/libfuse_b200.so.  Objects are rebuilt only when a source or header is newer."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfuse_b200.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header() -> float:
    stamps = [os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    stamps += [os.path.getmtime(os.path.join(INCLUDE, f)) for f in os.listdir(INCLUDE)]
    return max(stamps)


def build(verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    header_stamp = _newest_header()
    jobs = []
    objects = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if (not os.path.exists(obj) or os.path.getmtime(obj) < os.path.getmtime(src)
                or os.path.getmtime(obj) < header_stamp or ptxas_info):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or ptxas_info or result.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + result.stdout + result.stderr)
        if result.returncode != 0:
            raise RuntimeError("nvcc failed: " + cmd[-3])

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        link = [nvcc, "-shared", "-o", LIB, *objects, "-gencode", "arch=compute_100a,code=sm_100a",
                "-lcudart"]
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
