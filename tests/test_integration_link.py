"""The link recipe of the integration notes, executed: mimfer's own dispatcher
(src/kernels/kx.c), CUDA runtime shim (src/cuda/cuda_rt.c, -DMM_WITH_CUDA) and core
(src/core/mimfer.c), compiled from the reference tree, linked with this library's
objects minus csrc/cuda/rt.c and csrc/core/core.c (oracle/build.py: build_integration).
On a GPU one OP_GEMM_F4 then goes through the reference's mm_kx_invoke into this
library's kx_op_gemm_f4 and is compared with the oracle."""
import os
import subprocess

import numpy as np
import pytest

from conftest import REL_L2_TOL, row_rel_l2


def _exe():
    from oracle import build
    return build.build_integration()


def test_reference_dispatcher_links_against_the_library(lib):
    from oracle import build
    if not build.reference_available():
        pytest.skip("reference tree not mounted")
    exe = _exe()
    assert exe and os.path.exists(exe)
    syms = subprocess.check_output(["nm", "--defined-only", exe]).decode().split("\n")
    defined = [line.split()[-1] for line in syms if line.strip()]
    for name in ("mm_kx_invoke", "mm_cuda_stream_raw", "mm_cuda_capturing", "mm_status_str", "mm_log", "mmb_log",
                 "kx_op_gemm_f4", "kx_op_qkv", "kx_op_lmhead", "kx_op_silu_mul", "kx_op_add_rmsnorm",
                 "kx_op_rope", "kx_cuda_oppref", "mm_f4_select"):
        assert defined.count(name) == 1, name
    # the runtime shim and the core of this library stayed out
    for name in ("mmb_event_pool_reserve", "mm_time_begin", "mm_lin_engine_create"):
        assert name not in defined, name


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N", [(1, 5120, 512), (16, 2048, 1000), (300, 512, 264), (3, 48, 9)])
def test_op_through_the_reference_dispatcher(rt, oracle, tmp_path, M, K, N):
    import mimfer_b200 as mm
    exe = _exe()
    if not exe or not os.path.exists(exe):
        pytest.skip("integration program not built (no reference tree where the library was built)")
    w = mm.make_weight(N, K, seed=5)
    xb = mm.make_activations(M, K, seed=6)
    paths = [str(tmp_path / n) for n in ("x.bin", "payload.bin", "scales.bin", "y.bin")]
    for a, p in zip((xb, w.payload, w.scales), paths):
        np.ascontiguousarray(a).tofile(p)
    out = subprocess.run([exe, str(M), str(K), str(N), repr(float(w.gs)), *paths], capture_output=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr.decode()[-2000:]
    y = np.fromfile(paths[3], dtype=np.uint16).reshape(M, N)
    assert row_rel_l2(y, oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL
    # and bit for bit what the library gives through its own entry point
    assert np.array_equal(y, rt.from_device_bf16(rt.gemm_f4(rt.to_device_bf16(xb), w.to_device(rt.device))))
