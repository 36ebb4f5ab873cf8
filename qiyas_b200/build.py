"""Builds libqiyas_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Every .cu is compiled to an object of its own (in parallel; an object is rebuilt only when its source or a header is
newer) and the objects are linked into the one shared library.
"""
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIBRARY = os.path.join(HERE, "libqiyas_b200.so")
SOURCES = ["api.cu", "gemv.cu", "codecs.cu", "matmul.cu", "shard.cu"]
HEADERS = ["common.cuh", "launch.h", "encode_blocks.cuh", os.path.join("..", "..", "include", "qiyas_b200.h")]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--compiler-options", "-fPIC",
         "-Xptxas", "-v"]


def _newest_header():
    return max(os.path.getmtime(os.path.join(CSRC, h)) for h in HEADERS)


def _flags():
    return FLAGS + os.environ.get("QB200_NVCC_FLAGS", "").split()


def _stamp():
    return " ".join(_flags())


def _object(src):
    return os.path.join(OBJ, src.replace(".cu", ".o"))


def _stale_object(src, headers_time):
    obj = _object(src)
    if not os.path.exists(obj):
        return True
    built = os.path.getmtime(obj)
    return os.path.getmtime(os.path.join(CSRC, src)) > built or headers_time > built


def stale():
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > built for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compiles every .cu of the package and links the shared library; returns its path."""
    if not force and not stale():
        return LIBRARY
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    stamp_file = os.path.join(OBJ, "flags.txt")
    same_flags = os.path.exists(stamp_file) and open(stamp_file).read() == _stamp()
    headers_time = _newest_header()
    todo = [s for s in SOURCES if force or not same_flags or _stale_object(s, headers_time)]

    def compile_one(src):
        cmd = [nvcc] + _flags() + ["-c", "-o", _object(src), src]
        return src, subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, todo))
    log = "".join(f"---- {src}\n{out.stdout}{out.stderr}" for src, out in results)
    if verbose or any(out.returncode for _, out in results):
        print(log)
    if any(out.returncode for _, out in results):
        raise RuntimeError("nvcc failed building libqiyas_b200.so")
    with open(stamp_file, "w") as f:
        f.write(_stamp())
    link = subprocess.run([nvcc, "-shared", "-o", LIBRARY] + [_object(s) for s in SOURCES], cwd=CSRC, capture_output=True, text=True)
    if verbose or link.returncode:
        print(link.stdout + link.stderr)
    if link.returncode:
        raise RuntimeError("nvcc failed linking libqiyas_b200.so")
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True, verbose=True))
