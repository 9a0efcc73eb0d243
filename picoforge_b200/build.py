"""Builds the native parts in-tree: the CUDA product library (sm_100a only), the synthetic
weight generator, and (test infrastructure) the CPU oracle.

    python -m picoforge_b200.build            # build what is out of date
    python -m picoforge_b200.build --force

nvcc cross-compiles without a GPU.  The outputs stay beside the sources so that they travel
with the tree; they are git-ignored.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "picoforge_b200"
CSRC = PKG / "csrc"
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
GCC = shutil.which("gcc") or "gcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    newest = max(s.stat().st_mtime for s in sources)
    return target.stat().st_mtime < newest


def _run(cmd: list[str]) -> None:
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True)


def build_product(force: bool = False) -> Path:
    out = PKG / "libqwen4_moe_b200.so"
    cu_sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [ROOT / "include" / "qwen4_moe_b200.h"]
    host = CSRC / "moe_host.c"
    build_dir = PKG / "build"
    build_dir.mkdir(exist_ok=True)
    objects = []
    for src in cu_sources:
        obj = build_dir / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            _run([NVCC, *ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-c", src, "-o", obj])
        objects.append(obj)
    for host in (host, CSRC / "gguf_slice.c", CSRC / "verify_stack.c"):
        host_obj = build_dir / (host.stem + ".o")
        if force or _stale(host_obj, [host] + headers):
            _run([GCC, "-std=c11", "-O2", "-fPIC", "-Wall", "-Wextra", "-fvisibility=default", "-D_DEFAULT_SOURCE", f"-I{ROOT / 'include'}",
                  "-c", host, "-o", host_obj])
        objects.append(host_obj)
    if force or _stale(out, objects):
        _run([NVCC, *ARCH, "-shared", "-Xlinker", "-Bsymbolic", "-o", out, *objects, "-lm"])
    return out


def build_synth(force: bool = False) -> Path:
    out = PKG / "libqw4synth.so"
    src = CSRC / "synth.c"
    if force or _stale(out, [src, CSRC / "iq2xxs_codebook.h"]):
        _run([GCC, "-std=c11", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", src, "-lm", "-lpthread", "-o", out])
    return out


def build_oracle() -> None:
    """Compiles oracle/ (and the reference's own objects when its sources are mounted).
    Building the checker is not using it: nothing in the package imports it."""
    _run(["make", "-C", ROOT / "oracle", "--no-print-directory"])


def build_all(force: bool = False) -> None:
    build_product(force)
    build_synth(force)
    build_oracle()


if __name__ == "__main__":
    build_all("--force" in sys.argv)
