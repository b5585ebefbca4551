"""Build the sm_100a shared library in-tree with nvcc.

    python litespark-inference_b200/build.py [--force] [--verbose]

Produces ``litespark-inference_b200/_lspk_sm100.so`` from every ``csrc/*.cu``.  Objects are
cached under ``csrc/_obj`` and rebuilt when a source or header is newer.  nvcc cross-compiles
for sm_100a, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = CSRC / "_obj"
LIB = HERE / "_lspk_sm100.so"
INCLUDE = HERE.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _host_compiler_args() -> list:
    # A CC/CXX pointing at a wrapper toolchain without OpenMP specs is irrelevant here, but nvcc
    # needs a g++ it supports; prefer the system one when present.
    for cxx in ("/usr/bin/g++",):
        if Path(cxx).exists():
            return ["-ccbin", cxx]
    return []


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    newest_header = max((h.stat().st_mtime for h in headers), default=0.0)
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header)
        if stale:
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        extra = os.environ.get("LSPK_NVCC_FLAGS", "").split()        # e.g. -DLSPK_LINEAR_MIN_BLOCKS=3 for experiments
        cmd = [_nvcc(), *_host_compiler_args(), *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = OBJ / (src.stem + ".ptxas.log")
        log.write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return src.name

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name in ex.map(compile_one, jobs):
                print(f"[build] compiled {name}")
    objs = [str(OBJ / (s.stem + ".o")) for s in sources]
    need_link = force or bool(jobs) or not LIB.exists()
    if need_link:
        cmd = [_nvcc(), *_host_compiler_args(), "-shared", "-o", str(LIB), *objs,
               "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        print(f"[build] linked {LIB.name}")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
