"""In-tree build of the CUDA library (``libvmoe.so``) for sm_100a with plain nvcc.

``python sm120_moe_bench_b200/build.py`` (or ``build_library()``; run it as a script, because
importing the package needs the finished library) compiles every ``csrc/*.cu``
into one shared object next to this file.  nvcc cross-compiles without a GPU.  No fast-math:
the SwiGLU and the scale divisions need IEEE ``expf`` and division (the reference builds
without it for the same reason, fused-moe/verdict_moe.py:67-76).
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
LIB = PKG / "libvmoe.so"
STAMP = PKG / "csrc" / ".build_stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]
if os.environ.get("VMOE_PROFILE", "0") == "1":     # role cycle counters in the tcgen05 kernels (development aid)
    NVCC_FLAGS.append("-DVMOE_PROFILE")
if os.environ.get("VMOE_TIMELINE", "0") == "1":    # %globaltimer marks in the small-batch kernels (development aid)
    NVCC_FLAGS.append("-DVMOE_TIMELINE")


def _sources():
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "vmoe.h"]):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    digest = _digest()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
        return LIB
    if not os.path.exists(nvcc):
        if LIB.exists():
            return LIB          # prebuilt library shipped with the tree, no compiler on this host
        raise RuntimeError("nvcc not found and no prebuilt libvmoe.so")
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src in _sources():
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    log = []
    for src, p in procs:
        out, _ = p.communicate()
        log.append(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(LIB), *objs, "-lcudart"], check=True)
    (objdir / "ptxas.log").write_text("\n".join(log))
    STAMP.write_text(digest)
    if verbose:
        print("\n".join(log))
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
