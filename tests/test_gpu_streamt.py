"""STREAM-T: the decode kernel that dequantises into tensor memory and runs the
multiply on tcgen05 (variant 3), against the CPU oracle."""
import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import V_STREAMT
from conftest import REL_L2_TOL, row_rel_l2
from test_gpu_parity import check, run

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M", [1, 2, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("K,N", [(256, 256), (512, 40), (1024, 600), (5120, 1024)])
def test_streamt_shapes(rt, oracle, M, K, N):
    check(rt, oracle, M, K, N, V_STREAMT, seed=K + N + M)


@pytest.mark.parametrize("M", [1, 16, 32])
def test_streamt_long_k_split(rt, oracle, M):
    plan = mm.select_plan(M, 17408, 5120, ws_bytes=rt.lib.mm_f4_workspace_bytes(), variant=V_STREAMT)
    assert plan.split_k > 1
    check(rt, oracle, M, 17408, 5120, V_STREAMT, seed=5)


def test_streamt_gate_up(rt, oracle):
    check(rt, oracle, 4, 5120, 34816, V_STREAMT, seed=0)


@pytest.mark.parametrize("M", [1, 16, 32])
def test_streamt_activation_range_picks_operand_format(rt, oracle, M):
    K, N = 2048, 512
    w = mm.make_weight(N, K, seed=3)
    xf = mm.linear.fill_normal(M, K, 4)
    xf[0, 5] = 3.0e-9
    xf[M - 1, 700] = 2.5e5
    xf[0, 1300:1310] = 0.0
    xf[M // 2, 1800] = -1.0e-30
    x = mm.linear.f32_to_bf16(xf)
    y = run(rt, x, w, V_STREAMT)
    assert row_rel_l2(y, oracle.gemm_f4(x, w.payload, w.scales, w.gs)) <= REL_L2_TOL
    x2 = mm.linear.f32_to_bf16(xf * np.float32(1.0e-7))
    y2 = run(rt, x2, w, V_STREAMT)
    assert row_rel_l2(y2, oracle.gemm_f4(x2, w.payload, w.scales, w.gs)) <= REL_L2_TOL


def test_streamt_random_bytes_and_determinism(rt, oracle):
    rng = np.random.Generator(np.random.PCG64(6))
    M, K, N = 5, 1024, 300
    w = mm.NvFp4Weight(rng.integers(0, 256, (N, K // 2), dtype=np.uint8),
                       rng.integers(0, 256, (N, K // 16), dtype=np.uint8), 1.0, N, K)
    x = mm.make_activations(M, K, seed=8)
    a = run(rt, x, w, V_STREAMT)
    assert row_rel_l2(a, oracle.gemm_f4(x, w.payload, w.scales, 1.0)) <= REL_L2_TOL
    assert np.array_equal(run(rt, x, w, V_STREAMT), a)
