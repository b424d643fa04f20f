"""Build the CPU oracle (test infrastructure) into oracle/libgs_oracle.so.

    python oracle/build.py            # g++ -O3 -march=native -fopenmp

-ffp-contract=off keeps the compiler from fusing a*b+c on its own, so the fp32 key arithmetic
in philox.h is the exact sequence of IEEE operations the CUDA kernels spell with intrinsics.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "gs_oracle.cc")
OUT = os.path.join(HERE, "libgs_oracle.so")


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(HERE, "philox.h")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    cmd = ["g++", "-std=c++17", "-O3", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off", "-fPIC",
           "-shared", "-fvisibility=hidden", "-Wall", "-Wextra", "-o", OUT, SRC]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
