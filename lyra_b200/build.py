"""Builds the native libraries in-tree.

* ``lyra_b200/_lib/liblyra_b200_kernels.so`` - every ``.cu`` under ``csrc/`` compiled by nvcc for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a``), exported as plain C symbols.
* ``lyra_b200/_lib/liblyra_b200_io.so`` - the host runtime (``csrc/io/*.cpp``): ArrayRecord
  reader/writer, prefetching block loader, checkpoint chunk I/O.

Objects are cached by source mtime so a rebuild after one edit takes seconds. The libraries are
loaded with ctypes (see ``lyra_b200/ops/native.py``); there is no JIT step at import time.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-Wall"]


def _newer(src: Path, out: Path, extra: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *extra])


def _run(cmd: list[str], log: Path | None = None) -> None:
    res = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("build failed: " + " ".join(cmd))


def build_kernels(verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))
    sources = sorted(CSRC.rglob("*.cu"))
    objs: list[Path] = []
    jobs = []
    for src in sources:
        obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(obj)
        if _newer(src, obj, headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        _run(["nvcc", *NVCC_FLAGS, "-c", str(src), "-o", str(obj)], log=obj.with_suffix(".ptxas.log"))
        if verbose:
            print(f"[build] nvcc {src.relative_to(ROOT)}")

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(compile_one, jobs))
    out = LIB / "liblyra_b200_kernels.so"
    if jobs or not out.exists():
        _run(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(out), *map(str, objs)])
    return out


def build_io(verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted((CSRC / "io").glob("*.cpp"))
    headers = list((CSRC / "io").glob("*.h"))
    out = LIB / "liblyra_b200_io.so"
    if not sources:
        return out
    if any(_newer(s, out, headers) for s in sources):
        _run(["g++", *CXX_FLAGS, "-shared", "-o", str(out), *map(str, sources), "-ldl"])
        if verbose:
            print("[build] g++ io runtime")
    return out


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose)
    build_io(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
    print("built:", *(p.name for p in LIB.glob("*.so")))
