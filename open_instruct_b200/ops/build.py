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


def ptxas_digest() -> str:
    """Markdown table of registers, stack and spills per kernel, from the ``*.ptxas.txt`` files the last build left beside the
    objects (``ptxas -v`` output, one file per source)."""
    import re

    rows, mangled = [], set()
    pat = re.compile(r"Function properties for (\S+)\n\s+(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads\n"
                     r"ptxas info\s+: Used (\d+) registers")
    for path in sorted(OBJ.glob("*.ptxas.txt")):
        for m in pat.finditer(path.read_text()):
            rows.append((path.name.replace(".ptxas.txt", ".cu"), m.group(1), *map(int, m.groups()[1:])))
            mangled.add(m.group(1))
    names = sorted(mangled)
    plain = subprocess.run(["c++filt"], input="\n".join(names), capture_output=True, text=True).stdout.split("\n") if shutil.which("c++filt") else names
    short = {n: re.sub(r"\(.*$", "", d).replace("void ", "").replace("b200::", "") for n, d in zip(names, plain)}
    out = ["# Registers, stack and spills of every kernel (`nvcc " + " ".join(NVCC_FLAGS[:5]) + " -Xptxas -v`)", "",
           "Made by `python -m open_instruct_b200.ops.build --force && python -m open_instruct_b200.ops.build --ptxas-digest > profiles/ptxas_registers.md`.",
           "Kernel entry points only, template arguments kept.  A kernel with a non-zero spill column reads and writes local memory.", "",
           "| source | kernel | registers | stack B | spill stores B | spill loads B |", "|---|---|---|---|---|---|"]
    seen, spilled = set(), set()
    for src, name, stack, sst, sld, regs in rows:
        key = (src, short[name])
        if key in seen:
            continue
        seen.add(key)
        out.append(f"| `{src}` | `{short[name]}` | {regs} | {stack} | {sst} | {sld} |")
        if sst or sld:
            spilled.add(f"`{short[name]}` ({sst} / {sld} B)")
    out += ["", f"{len(seen)} kernels; {len(spilled)} with spills" + (": " + ", ".join(sorted(spilled)) if spilled else "") + "."]
    return "\n".join(out) + "\n"


def main() -> None:
    if "--ptxas-digest" in sys.argv:
        sys.stdout.write(ptxas_digest())
        return
    build_all(force="--force" in sys.argv)


if __name__ == "__main__":
    main()
