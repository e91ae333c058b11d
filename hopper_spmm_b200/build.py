"""In-tree build of libb200spmm.so (nvcc, sm_100a only)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200spmm.so")
CLI = os.path.join(HERE, "spmm_test")  # spmm_test <matrix.mtx> <feature_dim> [fp16|tf32]
SOURCES = ["capi.cu", "kat.cu", "convert_gpu.cu", "compress_gpu.cu", "tall_gpu.cu", "sharded.cu", "formats_ext.cu", "capi_formats.cpp", "format.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",  # -arch=sm_100a would add a generic PTX pass that rejects tcgen05
    "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-ldl",
]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps += [os.path.join(HERE, "..", "include", f) for f in os.listdir(os.path.join(HERE, "..", "include"))]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not _stale():
        return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + SOURCES
    subprocess.run(cmd, cwd=CSRC, check=True)
    # the command-line run of the reference's main, linked against the library next to it
    cli = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-o", CLI, "spmm_test.cu",
           "-L" + HERE, "-lb200spmm", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    subprocess.run(cli, cwd=CSRC, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
