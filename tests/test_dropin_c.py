"""The operator ABI driven from C, as mimfer's own host code would."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, fnv1a64

SRC = os.path.join(ROOT, "tests", "c", "dropin_main.c")
REF = os.environ.get("MIMFER_REFERENCE", os.path.join(os.sep, "root", "reference"))   # the reference tree, where mounted
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
LIBDIR = os.path.join(ROOT, "mimfer_b200")


def _build(tmp_path, flags):
    exe = str(tmp_path / "dropin_main")
    cmd = ["gcc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", "-O1", *flags, "-I" + os.path.join(CUDA, "include"),
           SRC, "-o", exe, "-L" + LIBDIR, "-lmimfer_b200", "-L" + os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + LIBDIR, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    subprocess.check_call(cmd)
    return exe


def test_links_against_unmodified_reference_headers(lib, tmp_path):
    """A translation unit written against the reference's own headers compiles
    and links against this library: same types, same symbols."""
    if not os.path.isdir(os.path.join(REF, "include", "mimfer")):
        pytest.skip("reference headers not mounted")
    exe = _build(tmp_path, ["-DUSE_REFERENCE_HEADERS", "-I" + os.path.join(REF, "include")])
    assert os.path.exists(exe)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N", [(1, 5120, 512), (16, 17408, 1024), (300, 512, 264), (3, 48, 9)])
def test_c_host_matches_python_path_and_oracle(rt, lib, oracle, tmp_path, M, K, N):
    import mimfer_b200 as mm
    from conftest import REL_L2_TOL, row_rel_l2
    exe = _build(tmp_path, ["-I" + os.path.join(ROOT, "include")])
    out = subprocess.check_output([exe, str(M), str(K), str(N)], timeout=300).decode().split()[-1]
    w = mm.make_weight(N, K, seed=0).to_device(rt.device)
    xb = mm.make_activations(M, K, seed=1)
    y = rt.from_device_bf16(rt.gemm_f4(rt.to_device_bf16(xb), w))
    assert int(out, 16) == fnv1a64(np.ascontiguousarray(y))          # the C host's output, bit for bit
    assert row_rel_l2(y, oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL
