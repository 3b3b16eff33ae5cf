"""In-tree build of libmgbs_b200.so for sm_100a with nvcc.

The reference JIT-builds its extension with torch.utils.cpp_extension.load (beam_engine.py:112-157); here the
library has no torch or Python dependency, so a plain nvcc invocation is enough.  Usage:
    python -m multigpubeamsearch_b200.build [--force]
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
ROOT = PKG.parent
LIB = PKG / "libmgbs_b200.so"
SOURCES = ["mgbs_step.cu", "mgbs_engine.cu", "mgbs_scorer.cu", "mgbs_transformer.cu", "mgbs_nvfp4.cu"]
HEADERS = ["mgbs_device.cuh", "mgbs_internal.cuh", "mgbs_tc.cuh", "mgbs_nvfp4.cuh"]


def _nccl_include() -> str:
    purelib = Path(sysconfig.get_paths()["purelib"])
    cand = purelib / "nvidia" / "nccl" / "include"
    if (cand / "nccl.h").exists():
        return str(cand)
    for p in ("/usr/include", "/usr/local/cuda/include"):
        if (Path(p) / "nccl.h").exists():
            return p
    raise FileNotFoundError("nccl.h not found")


def nccl_library_path() -> str:
    """Path of the libnccl.so.2 that torch uses (handed to mgbs_engine_init_nccl)."""
    purelib = Path(sysconfig.get_paths()["purelib"])
    cand = purelib / "nvidia" / "nccl" / "lib" / "libnccl.so.2"
    return str(cand) if cand.exists() else "libnccl.so.2"


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES if (CSRC / s).exists()] + [CSRC / h for h in HEADERS] + [ROOT / "include" / "mgbs.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    cmd = [
        nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC",
        "-I", str(ROOT / "include"), "-I", str(CSRC), "-I", _nccl_include(),
        "-o", str(LIB), *srcs, "-ldl",
    ]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
