"""Build libdnet_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
SRC = ROOT / "csrc" / "dn_api.cu"
# the batched sequence-mixer step is a library of its own: a process that serves such a model compiles and loads
# only this one
SEQ_SRC = ROOT / "csrc" / "dn_seq.cu"
_SEQ_ONLY = [*sorted((ROOT / "csrc").glob("dn_seq*.cu*")), ROOT.parent / "include" / "dnet_b200_seq.h"]
SEQ_DEPS = [*_SEQ_ONLY, *sorted((ROOT / "csrc").glob("*.cuh"))]      # it shares the tcgen05 GEMM of dn_gemm_tc.cuh
SEQ_OUT = ROOT / "lib" / "libdnet_b200_seq.so"
DEPS = [d for d in [*sorted((ROOT / "csrc").glob("*.cu*")), ROOT.parent / "include" / "dnet_b200.h"] if d not in _SEQ_ONLY]
OUT = ROOT / "lib" / "libdnet_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-cudart", "static",
]


def needs_build(out: Path = OUT, deps=None) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in (DEPS if deps is None else deps))


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(OUT), str(SRC)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return OUT


def build_seq(force: bool = False, verbose: bool = False) -> Path:
    """libdnet_b200_seq.so; concurrent first calls build into private files and rename."""
    if not force and not needs_build(SEQ_OUT, SEQ_DEPS):
        return SEQ_OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    SEQ_OUT.parent.mkdir(parents=True, exist_ok=True)
    tmp = SEQ_OUT.with_name(f".{SEQ_OUT.name}.{os.getpid()}")
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(tmp), str(SEQ_SRC)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
        print(" ".join(cmd), file=sys.stderr)
    try:
        subprocess.run(cmd, check=True, stdout=sys.stderr)
        os.replace(tmp, SEQ_OUT)
    finally:
        if tmp.exists():
            tmp.unlink()
    return SEQ_OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_seq(force="--force" in sys.argv, verbose="-v" in sys.argv))
