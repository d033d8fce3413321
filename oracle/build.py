"""Build recipe for the CPU oracle (test infrastructure, not product code).

  liboracle.so            plain-C restatement of the reference algorithm
                          (oracle/nvfp4_oracle.c)
  _ref/integration_main   the reference's dispatcher, CUDA shim and core linked with
                          this library's objects (build_integration): the link
                          recipe of the integration notes, executed
  _ref/libmimfer_ref.so   the reference's own CPU kernel, compiled from the
                          sources where they lie in the read-only reference
                          tree (src/kernels/cpu/cx.c + src/core/mimfer.c) plus
                          oracle/ref_driver.c and oracle/ref_driver_norm.c.  Only built when that tree is
                          mounted; the prebuilt file is used otherwise.

Run:  python oracle/build.py
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.environ.get("MIMFER_REFERENCE", os.path.join(os.sep, "root", "reference"))   # the reference tree, where mounted

ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libmimfer_ref.so")

# -std=c11: ISO mode keeps -ffp-contract=off, so gcc forms no FMA; no
# -march=native.  These are the flags that matter for bit-identity with the
# reference host build (reference Makefile:8-11,32,41-46).
CFLAGS = ["-std=c11", "-O2", "-fPIC", "-shared", "-fopenmp", "-Wall", "-Wextra"]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.exists(s) and os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = [os.path.join(HERE, "nvfp4_oracle.c")]
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    subprocess.check_call(["gcc", *CFLAGS, *src, "-lm", "-o", ORACLE_SO])
    return ORACLE_SO


def reference_available():
    return os.path.isfile(os.path.join(REF, "src", "kernels", "cpu", "cx.c"))


def build_ref(force=False):
    """Returns the path of the reference library, or None if it can be neither
    built (no reference tree) nor found prebuilt."""
    if not reference_available():
        return REF_SO if os.path.exists(REF_SO) else None
    src = [os.path.join(REF, "src", "kernels", "cpu", "cx.c"),
           os.path.join(REF, "src", "core", "mimfer.c"),
           os.path.join(HERE, "ref_driver.c"),
           os.path.join(HERE, "ref_driver_norm.c")]
    if not force and _newer(REF_SO, src):
        return REF_SO
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    inc = ["-I" + os.path.join(REF, "include"),
           "-I" + os.path.join(REF, "src", "kernels"),
           "-I" + os.path.join(REF, "src", "model"),
           "-I" + os.path.join(ROOT, "include")]
    # the reference sources are compiled without -Wextra noise control: they are not ours
    flags = [f for f in CFLAGS if f not in ("-Wall", "-Wextra")]
    subprocess.check_call(["gcc", *flags, *inc, *src, "-lm", "-o", REF_SO])
    return REF_SO


INTEGRATION_EXE = os.path.join(HERE, "_ref", "integration_main")


def build_integration(force=False):
    """The link recipe a maintainer of the reference tree would run, executed: the
    reference's own dispatcher (src/kernels/kx.c), CUDA runtime shim
    (src/cuda/cuda_rt.c, -DMM_WITH_CUDA) and core (src/core/mimfer.c), compiled where
    they lie, linked with this library's objects MINUS csrc/cuda/rt.c and
    csrc/core/core.c (csrc/core/core_shim.c instead), the launcher built with
    -DMMB_NO_DISPATCHER, stubs for the launchers the library does not own
    (tests/c/integration_stubs.c) and a driver written against the reference headers
    (tests/c/integration_main.c).  Returns the program's path, or None when it can be
    neither built (no reference tree) nor found prebuilt."""
    if not reference_available():
        return INTEGRATION_EXE if os.path.exists(INTEGRATION_EXE) else None
    sys.path.insert(0, ROOT)
    from mimfer_b200 import build as lib_build
    lib_build.build()                                        # the kernels' objects
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    csrc, objdir = lib_build.CSRC, lib_build.OBJ
    ref_src = [os.path.join(REF, "src", "kernels", "kx.c"), os.path.join(REF, "src", "cuda", "cuda_rt.c"),
               os.path.join(REF, "src", "core", "mimfer.c"),
               os.path.join(ROOT, "tests", "c", "integration_stubs.c"),
               os.path.join(ROOT, "tests", "c", "integration_main.c")]
    own_src = [os.path.join(csrc, "core", "core_shim.c"), os.path.join(csrc, "plan", "select.c"),
               os.path.join(csrc, "cuda", "kx_gemm_f4.c")]
    kernels = [os.path.join(objdir, rel.replace("/", "_") + ".o") for rel in lib_build.CU_SOURCES]
    deps = ref_src + own_src + kernels
    if not force and _newer(INTEGRATION_EXE, deps):
        return INTEGRATION_EXE
    out = os.path.join(HERE, "_ref", "integration_obj")
    os.makedirs(out, exist_ok=True)
    objs = []
    ref_inc = ["-I" + os.path.join(REF, "include"), "-I" + os.path.join(REF, "src", "kernels"),
               "-I" + os.path.join(cuda, "include")]
    for src in ref_src:
        obj = os.path.join(out, "ref_" + os.path.basename(src) + ".o")
        subprocess.check_call(["gcc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", "-O2", "-DMM_WITH_CUDA=1", *ref_inc,
                               "-c", src, "-o", obj])
        objs.append(obj)
    for src in own_src:
        obj = os.path.join(out, "own_" + os.path.basename(src) + ".o")
        subprocess.check_call(["gcc", "-std=c11", "-O2", "-fopenmp", "-DMMB_NO_DISPATCHER",
                               "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(cuda, "include"),
                               "-c", src, "-o", obj])
        objs.append(obj)
    subprocess.check_call([os.path.join(cuda, "bin", "nvcc"), "-o", INTEGRATION_EXE, *objs, *kernels,
                           "-Xcompiler", "-fopenmp", "-lm"])
    return INTEGRATION_EXE


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_integration(force="--force" in sys.argv))
