"""Builds the C twin of the oracle (oracle/ref_kernels.c) into oracle/_build/libref_kernels.so.

TEST / BENCH INFRASTRUCTURE: only tests/, the smoke check and bench.py's CPU-baseline leg load it.
The reference itself (Zig on MLX) needs a Zig toolchain and the MLX libraries, so no build of its
own sources exists next to this twin.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")
LIB = os.path.join(OUT, "libref_kernels.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "ref_kernels.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        # AVX2+FMA is a safe floor for the hosts this runs on; -march=native would tie the
        # binary to the build machine.
        cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-shared", "-fPIC", "-o", LIB, src, "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"gcc failed:\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force=True))
