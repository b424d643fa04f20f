"""Builds the sm_100a kernel library (graph_sampling_b200/lib/libgsb200.so) with nvcc.

    python -m graph_sampling_b200.build [--force] [--verbose]

The library has no torch dependency: it is plain CUDA C++ behind the C ABI of include/gsb200.h.
nvcc cross-compiles for sm_100a, so this also runs on a machine without a GPU.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "_obj")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libgsb200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler",
              "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(PKG), "include", "gsb200.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    hm = _headers_mtime()
    jobs = []
    for s in sources():
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hm):
            cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources()]
    if jobs or not os.path.exists(LIB):
        subprocess.check_call(["nvcc", "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB] + objs + ["-lcudart"])
    return LIB


GLUE_SRC = os.path.join(CSRC, "glue", "gs_glue.cc")
GLUE_LIB = os.path.join(LIBDIR, "libgs.so")


def build_glue(force: bool = False) -> str:
    """Builds lib/libgs.so: the TorchScript front end (gs_classes.Graph, gs_ops.*) over the C ABI.  Needs the
    torch headers; links against libgsb200.so (found next to it through $ORIGIN) and torch."""
    build(force=False)
    deps = [GLUE_SRC, os.path.join(os.path.dirname(PKG), "include", "gsb200.h")]
    if not force and os.path.exists(GLUE_LIB) and all(os.path.getmtime(GLUE_LIB) >= os.path.getmtime(d) for d in deps):
        return GLUE_LIB
    import sysconfig
    import torch
    tdir = os.path.dirname(torch.__file__)
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-w",
           "-I", os.path.join(tdir, "include"), "-I", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           "-I", sysconfig.get_paths()["include"], "-I", "/usr/local/cuda/include", GLUE_SRC, "-o", GLUE_LIB,
           "-L", LIBDIR, "-lgsb200", "-Wl,-rpath,$ORIGIN", "-L", os.path.join(tdir, "lib"), "-ltorch", "-ltorch_cpu",
           "-ltorch_cuda", "-lc10", "-lc10_cuda", "-Wl,-rpath," + os.path.join(tdir, "lib"),
           "-L", "/usr/local/cuda/lib64", "-lcudart"]
    subprocess.check_call(cmd)
    return GLUE_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--glue" in sys.argv:
        print(build_glue(force="--force" in sys.argv))
