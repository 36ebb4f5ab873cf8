"""Compiles the C oracle (``qiyas_oracle.c``) into ``libqiyas_oracle.so`` beside it.

``-ffp-contract=off`` keeps every f32 multiply and add a separate rounding unless the source
writes ``fmaf``: the reference's CPU order (src/BlockProducts.cs:50) is unfused, its device
order (src/BlockProducts.cs:158-161) is fused, and the oracle restates both.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "qiyas_oracle.c")
LIBRARY = os.path.join(HERE, "libqiyas_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIBRARY) and os.path.getmtime(LIBRARY) >= os.path.getmtime(SOURCE):
        return LIBRARY
    cmd = ["gcc", "-O3", "-std=c11", "-ffp-contract=off", "-mavx2", "-fPIC", "-shared", "-fvisibility=hidden",
           "-Wall", "-Wextra", "-o", LIBRARY, SOURCE, "-lpthread", "-lm"]
    subprocess.run(cmd, check=True)
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True))
