"""In-tree build of libmimfer_b200.so (sm_100a only).

Host C (gcc, C11) : csrc/core, csrc/pack, csrc/plan, csrc/engine, csrc/cuda
CUDA   (nvcc)     : csrc/kernels, compiled with
                    -gencode arch=compute_100a,code=sm_100a -lineinfo

Run:  python -m mimfer_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.environ.get("MMB_BUILD_LIB", os.path.join(PKG, "libmimfer_b200.so"))
OBJ = os.environ.get("MMB_BUILD_OBJ", OBJ)
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

C_SOURCES = ["core/core.c", "pack/pack.c", "plan/select.c", "engine/engine.c", "model/weights.c",
             "cuda/rt.c", "cuda/kx_gemm_f4.c"]
CU_SOURCES = ["kernels/rowwarp.cu", "kernels/stream.cu", "kernels/mx.cu", "kernels/mxg.cu", "kernels/umma.cu",
              "kernels/silu_mul.cu", "kernels/add_rmsnorm.cu", "kernels/tp_barrier.cu", "kernels/host_gather.cu"]
HEADERS = ["core/core.h", "kernels/launch.h", "kernels/ptx.cuh", "kernels/fp4.cuh", "kernels/mx.cuh",
           "../../include/mimfer_abi.h", "../../include/mimfer_b200.h"]

CFLAGS = ["-std=c11", "-O2", "-fPIC", "-fopenmp", "-Wall", "-Wextra", "-Werror",
          "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CUDA_HOME, "include"),
          *os.environ.get("MMB_EXTRA_DEFS", "").split()]
NVFLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
           "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"),
           *os.environ.get("MMB_EXTRA_NVFLAGS", "").split(), *os.environ.get("MMB_EXTRA_DEFS", "").split()]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.normpath(os.path.join(CSRC, h)) for h in HEADERS]
    objs = []
    for rel in C_SOURCES + CU_SOURCES:
        src = os.path.join(CSRC, rel)
        obj = os.path.join(OBJ, rel.replace("/", "_") + ".o")
        objs.append(obj)
        if not force and not _stale(obj, [src] + headers):
            continue
        if rel.endswith(".cu"):
            cmd = [NVCC, *NVFLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj]
        else:
            cmd = ["gcc", *CFLAGS, "-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if force or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fopenmp", "-lm"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
