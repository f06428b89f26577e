"""Test infrastructure, not part of the product: builds ``oracle/_ref/libref_host.so`` from the reference's own
host C++ reference (``fused-moe/csrc/verdict_fused_independent.cu``), compiled in place through the wrapper
``oracle/ref_host.cu``.  Needs the reference checkout and nvcc (the file carries sm_120a kernels, which are
compiled but never launched).  Where the checkout is absent the previously built library is used as is."""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "libref_host.so"
REFERENCE_ROOT = Path(os.environ.get("VMOE_REFERENCE_ROOT", "/root/reference"))
SOURCE = REFERENCE_ROOT / "fused-moe" / "csrc" / "verdict_fused_independent.cu"


def build(force: bool = False) -> Path | None:
    """Returns the library path, or None when it neither exists nor can be built here."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not SOURCE.exists() or not os.path.exists(nvcc):
        return OUT if OUT.exists() else None
    wrapper = HERE / "ref_host.cu"
    if not force and OUT.exists() and OUT.stat().st_mtime >= max(wrapper.stat().st_mtime, SOURCE.stat().st_mtime):
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = [nvcc, f"-I{REFERENCE_ROOT}", "-gencode", "arch=compute_120a,code=sm_120a", "-O2", "-shared",
           "-Xcompiler", "-fPIC", "-o", str(OUT), str(wrapper)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building the reference host library failed:\n" + res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
