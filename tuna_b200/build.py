"""In-tree build of libtuna_b200.so (nvcc, sm_100a only).

The shared library is the product's only native artefact: hand-written CUDA
kernels behind a C ABI (include/tuna_b200.h).  It is built next to the sources
so that it travels with the tree; nothing is JIT-compiled at import time.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libtuna_b200.so"
SOURCES = ["tuna_api.cu", "host_util.cu", "dequant_sm100a.cu", "quantize_sm100a.cu", "gemm_stream_sm100a.cu", "gemm_tstream_sm100a.cu", "gemm_umma_sm100a.cu", "exchange_sm100a.cu", "ref_symbols.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel source for sm_100a and link the shared library."""
    from . import make_configs

    make_configs.generate()
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.inc")) + [
        HERE.parent / "include" / "tuna_b200.h"
    ]
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str):
        obj = objdir / (src + ".o")
        if force or _stale(obj, [CSRC / src] + headers):
            extra = os.environ.get("TUNA_EXTRA_NVCC_FLAGS", "").split()
            cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(CSRC / src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    if force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB)] + [str(o) for o in objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
