"""Builds the C restatement of the Lloyd iteration (test infrastructure only):

    python -m oracle.build

The reference itself is pure Python on the numba_dpex / dpctl stack and has no C or C++
sources to compile, so there is no `oracle/_ref` binary: the oracle is this port.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "lloyd_oracle.c")
LIB = os.path.join(HERE, "liboracle_lloyd.so")


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found")
    # x86-64-v3 (AVX2) without FMA contraction: multiply and add stay separate roundings
    cmd = [gcc, "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
           SRC, "-o", LIB, "-lm"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force=True))
