"""Build ``libfqla_sm100.so`` (the C-ABI library of the CUDA kernels) in-tree with nvcc.

    python -m flashqla_b200.build            # incremental
    python -m flashqla_b200.build --force    # rebuild everything

Only sm_100a code is generated.  Objects go to ``flashqla_b200/csrc/_obj`` and the shared
library next to this file, so that a copy of the source tree carries the built library with it.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libfqla_sm100.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(os.path.dirname(HERE), "include", "fqla.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src: str, force: bool, hdr_mtime: float) -> tuple[str, str]:
    obj = os.path.join(OBJ, src[:-3] + ".o")
    path = os.path.join(CSRC, src)
    if (
        not force
        and os.path.exists(obj)
        and os.path.getmtime(obj) > max(os.path.getmtime(path), hdr_mtime)
    ):
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return obj, res.stderr


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr_mtime = _deps_mtime()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(lambda s: _compile(s, force, hdr_mtime), _sources()))
    objs = [o for o, _ in results]
    logs = "".join(log for _, log in results)
    if logs:
        with open(os.path.join(OBJ, "ptxas.log"), "a") as f:
            f.write(logs)
    if verbose and logs:
        print(logs, file=sys.stderr)
    if force or not os.path.exists(LIB) or any(
        os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs
    ):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
