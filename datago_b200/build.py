"""Compile the CUDA library in-tree: datago_b200/libdatago_b200.so, sm_100a only."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libdatago_b200.so")
SOURCES = ["api.cu", "kernels_jpeg.cu", "kernels_resize.cu", "host_logic.cpp", "jpeg_header.cpp", "feeder.cpp"]
HEADERS = ["desc.h", "host.h", "host_pool.h", "kernels.h", os.path.join("..", "..", "include", "datago_b200.h")]


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--shared",
           "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3", "-o", OUT]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("DATAGO_B200_NVCC_FLAGS", "").split()
    cmd += [os.path.join(CSRC, f) for f in SOURCES]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
