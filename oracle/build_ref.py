"""Test infrastructure, not part of the product: builds the libraries under ``oracle/_ref/`` from the reference's
own sources, compiled where they lie.  Nothing of the reference is copied into this repository; the outputs are
shared objects only.

* ``libref_host.so``   -- the host C++ reference of ``fused-moe/csrc/verdict_fused_independent.cu`` (codec,
  block quantiser, one-token expert pipeline) through the wrapper ``oracle/ref_host.cu``;
* ``libref_tables.so`` -- ``build_group_tables`` of ``fused-moe/csrc/verdict_fused_grouped.cu:655-691`` through
  the wrapper ``oracle/ref_tables.cu``;
* ``libref_router.so`` -- ``moe_topk_select`` of ``fused-moe/csrc/megakernel_v1.cu:491-537``.  That function is
  device code whose body is one sequential thread; the rest of its file does not compile for a host.  Its text
  is read from the reference file at build time (found by name, up to the matching brace), and piped to g++
  behind a few lines that define the device keywords away -- no intermediate file is written.

The first two need nvcc (the files carry sm_120a kernels, compiled but never launched), the third g++.  The
reference checkout is looked for at ``$VMOE_REFERENCE_ROOT``, else in a directory ``reference`` beside this
repository.  Where it is absent the previously built libraries are used as they are."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OUT = OUT_DIR / "libref_host.so"
OUT_TABLES = OUT_DIR / "libref_tables.so"
OUT_ROUTER = OUT_DIR / "libref_router.so"


def reference_root(arg: str | None = None) -> Path | None:
    cand = arg or os.environ.get("VMOE_REFERENCE_ROOT") or str(HERE.parent.parent / "reference")
    p = Path(cand)
    return p if (p / "fused-moe" / "csrc").is_dir() else None


def _newer(out: Path, *deps: Path) -> bool:
    return out.exists() and out.stat().st_mtime >= max(d.stat().st_mtime for d in deps)


def _nvcc_wrapper(root: Path, wrapper: Path, source: Path, out: Path, force: bool) -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return out
    if not force and _newer(out, wrapper, source):
        return out
    cmd = [nvcc, f"-I{root}", "-gencode", "arch=compute_120a,code=sm_120a", "-O2", "-shared",
           "-Xcompiler", "-fPIC", "-o", str(out), str(wrapper)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {out.name} failed:\n" + res.stdout + res.stderr)
    return out


def _function_text(source: Path, signature: str) -> str:
    """The text of one function of ``source``: from the line holding ``signature`` to its matching brace."""
    text = source.read_text()
    start = text.index(signature)
    start = text.rfind("\n", 0, start) + 1
    depth, i = 0, text.index("{", start)
    while True:
        c = text[i]
        if c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                return text[start:i + 1]
        i += 1


_ROUTER_PRELUDE = """
#include <math.h>
#define __device__
struct ThreadIdxStub { int x; };
static ThreadIdxStub threadIdx = {0};       /* the function's work is done by thread 0 */
static inline void __syncthreads() {}
"""
_ROUTER_WRAPPER = """
extern "C" void ref_topk_select(const float* logits, int num_experts, int top_k, int* ids, float* wts, float* scratch) {
    for (int e = 0; e < num_experts; ++e) scratch[e] = logits[e];     /* the function overwrites its input */
    moe_topk_select(ids, wts, scratch, num_experts, top_k);
}
"""


def _router(root: Path, out: Path, force: bool) -> Path:
    source = root / "fused-moe" / "csrc" / "megakernel_v1.cu"
    gxx = shutil.which("g++")
    if gxx is None or not source.exists():
        return out
    if not force and _newer(out, source, Path(__file__)):
        return out
    body = _function_text(source, "void moe_topk_select(")
    res = subprocess.run([gxx, "-x", "c++", "-O2", "-shared", "-fPIC", "-o", str(out), "-"],
                         input=_ROUTER_PRELUDE + body + _ROUTER_WRAPPER, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building libref_router.so failed:\n" + res.stdout + res.stderr)
    return out


def build(force: bool = False, root: str | None = None) -> Path | None:
    """Builds what can be built here.  Returns the path of ``libref_host.so``, or None when it neither exists
    nor can be built."""
    ref = reference_root(root)
    if ref is not None:
        OUT_DIR.mkdir(exist_ok=True)
        csrc = ref / "fused-moe" / "csrc"
        _nvcc_wrapper(ref, HERE / "ref_host.cu", csrc / "verdict_fused_independent.cu", OUT, force)
        _nvcc_wrapper(ref, HERE / "ref_tables.cu", csrc / "verdict_fused_grouped.cu", OUT_TABLES, force)
        _router(ref, OUT_ROUTER, force)
    return OUT if OUT.exists() else None


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("-")]
    print(build(force=True, root=args[0] if args else None))
