"""Builds ``libnomos_attn.so`` in-tree with nvcc for sm_100a.

    python -m nomos_nvfp4_b200.build [--force] [--verbose-ptxas]

The shared object lands beside this file (``nomos_nvfp4_b200/libnomos_attn.so``) so
it travels with a snapshot of the tree; nothing is written outside the package.
nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_obj"
LIB = PKG / "libnomos_attn.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
          "--expt-relaxed-constexpr"]
# Per-file extra flags.  The codecs must not contract a*b+c into an FMA: their
# bytes are compared bit-for-bit with a CPU restatement of the reference.
EXTRA = {"kv_quant.cu": ["-fmad=false"], "kv_producer.cu": ["-fmad=false"]}
SOURCES = ["abi.cu", "kv_quant.cu", "kv_producer.cu", "kv_ring.cu", "attn_fused.cu", "attn_dense.cu"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; libnomos_attn.so cannot be built")
    return exe


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose_ptxas: bool = False, extra_flags=(), out: Path | None = None,
          obj_dir: Path | None = None) -> Path:
    """Compile and link.  `extra_flags` (e.g. -DNOMOS_NWARP=3) with `out`/`obj_dir` build a variant
    beside the default library without touching it."""
    global OBJ, LIB
    OBJ, LIB = (obj_dir or PKG / "_obj"), (out or PKG / "libnomos_attn.so")
    OBJ.mkdir(exist_ok=True, parents=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "nomos_attn.h", Path(__file__)]
    objs = []
    procs = []
    for name in SOURCES:
        src = CSRC / name
        obj = OBJ / (name + ".o")
        objs.append(obj)
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc(), *ARCH, *COMMON, *EXTRA.get(name, []), *extra_flags, "-c", str(src), "-o", str(obj)]
            if verbose_ptxas:
                cmd += ["-Xptxas", "-v"]
            procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for name, p in procs:
        log, _ = p.communicate()
        if verbose_ptxas or p.returncode != 0:
            sys.stderr.write(f"--- {name}\n{log}\n")
        if p.returncode != 0:
            failed.append(name)
    if failed:
        raise RuntimeError(f"nvcc failed for {failed}")
    if force or procs or _stale(LIB, objs):
        cmd = [nvcc(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose_ptxas="--verbose-ptxas" in sys.argv)
    print(path, os.path.getsize(path), "bytes")
