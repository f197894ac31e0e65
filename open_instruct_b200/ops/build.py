"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``libb200ops.so``  - every ``csrc/*.cu`` kernel file, compiled by ``nvcc`` for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``), exporting a plain C ABI used through ``ctypes``.
* ``libb200host.so`` - the C++ host runtime in ``csrc/host/*.cpp`` (packer, block manager,
  scheduler), compiled with ``g++``.

The kernels do not include torch headers, so a full rebuild takes seconds and cross-compiles
on a machine without a GPU.  ``python -m open_instruct_b200.ops.build`` rebuilds what changed.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
OPS_LIB = HERE / "libb200ops.so"
HOST_LIB = HERE / "libb200host.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-Wall"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    return cand


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile_cu(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ / (src.stem + ".ptxas.txt")).write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stderr}")
    if verbose:
        spills = [ln for ln in res.stderr.splitlines() if "spill" in ln and "0 bytes spill stores, 0 bytes spill loads" not in ln]
        print(f"[build] {src.name}: ok" + (f" ({len(spills)} kernels spill)" if spills else ""))
    return obj


def build_ops(force: bool = False, verbose: bool = True) -> Path:
    """Compile all kernels into ``libb200ops.so`` (no-op when sources are unchanged)."""
    OBJ.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    stamp = OBJ / "ops.sha256"
    digest = _digest(srcs + hdrs, " ".join(NVCC_FLAGS))
    if not force and OPS_LIB.exists() and stamp.exists() and stamp.read_text() == digest:
        return OPS_LIB
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_cu(s, verbose), srcs))
    cmd = [_nvcc(), "-shared", "-o", str(OPS_LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr}")
    stamp.write_text(digest)
    if verbose:
        print(f"[build] linked {OPS_LIB.name} from {len(objs)} objects")
    return OPS_LIB


def build_host(force: bool = False, verbose: bool = True) -> Path | None:
    """Compile the C++ host runtime into ``libb200host.so``."""
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    if not srcs:
        return None
    OBJ.mkdir(exist_ok=True)
    hdrs = sorted((CSRC / "host").glob("*.h"))
    stamp = OBJ / "host.sha256"
    digest = _digest(srcs + hdrs, " ".join(CXX_FLAGS))
    if not force and HOST_LIB.exists() and stamp.exists() and stamp.read_text() == digest:
        return HOST_LIB
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, *CXX_FLAGS, "-I", str(CSRC / "host"), "-o", str(HOST_LIB), *map(str, srcs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{res.stderr}")
    stamp.write_text(digest)
    if verbose:
        print(f"[build] linked {HOST_LIB.name} from {len(srcs)} sources")
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = True) -> None:
    build_ops(force, verbose)
    build_host(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
