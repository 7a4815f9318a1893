"""Build the C-ABI shared library `subspec_b200/lib/libsubspec_b200.so` with nvcc.

sm_100a only.  The library is built in-tree so that it travels with the source
tree; nothing is JIT-compiled at import time.  Run `python -m subspec_b200.build`
(add `-v` for the ptxas register / shared-memory report).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libsubspec_b200.so"
STAMP = LIBDIR / "libsubspec_b200.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the subspec_b200 CUDA library cannot be built")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "subspec_b200.h"]):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ and link them into one shared library."""
    LIBDIR.mkdir(exist_ok=True)
    digest = _digest()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
        return LIB
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = LIBDIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(PKG.parent / "include"), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src.name} ---\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- {src.name} ---\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    link = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcuda",
            "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(link, check=True)
    STAMP.write_text(digest)
    return LIB


if __name__ == "__main__":
    path = build(force="-f" in sys.argv or "-v" in sys.argv, verbose="-v" in sys.argv)
    print(path)
