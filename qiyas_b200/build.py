"""Builds libqiyas_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBRARY = os.path.join(HERE, "libqiyas_b200.so")
SOURCES = ["api.cu", "gemv.cu", "codecs.cu", "matmul.cu"]
HEADERS = ["common.cuh", "launch.h", os.path.join("..", "..", "include", "qiyas_b200.h")]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--compiler-options", "-fPIC",
         "-shared", "-Xptxas", "-v"]


def stale():
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > built for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compiles every .cu of the package into one shared library; returns its path."""
    if not force and not stale():
        return LIBRARY
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + FLAGS + os.environ.get("QB200_NVCC_FLAGS", "").split() + ["-o", LIBRARY] + SOURCES
    out = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose or out.returncode:
        print(out.stdout + out.stderr)
    if out.returncode:
        raise RuntimeError("nvcc failed building libqiyas_b200.so")
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True, verbose=True))
