"""GPU parity of OP_ADD_RMSNORM (res += delta in place, y = rmsnorm(res) * gain)
against the CPU oracle, through the dispatcher and inside an op list behind the
down projection, where the reference planner emits it (src/plan/plan.c:440-449).

Bar: the in-place sum is bit-exact; the normalised output is within the op's
relative L2 bar and never more than one bf16 step from the oracle (the sum of
squares is added in another order than the reference's left-to-right loop)."""
import ctypes as C
import os

import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import _lib as L
from conftest import GOLDEN, REL_L2_TOL, row_rel_l2, bf16_bits_to_f32

pytestmark = pytest.mark.gpu


def bf16_steps(a, b):
    """largest distance between two bf16 arrays in units of the larger value's step"""
    fa, fb = bf16_bits_to_f32(a).astype(np.float64), bf16_bits_to_f32(b).astype(np.float64)
    big = np.maximum(np.abs(fa), np.abs(fb))
    step = np.where(big > 0, 2.0 ** (np.floor(np.log2(np.where(big > 0, big, 1.0))) - 7), 1.0)
    return float((np.abs(fa - fb) / step).max())


def run_norm(rt, res, delta, gain, via_dispatch=True):
    t_res, t_delta = rt.to_device_bf16(res), rt.to_device_bf16(delta)
    t_gain = rt.to_device_bf16(gain.reshape(1, -1))
    y = rt.torch.zeros(res.shape, dtype=rt.torch.bfloat16, device=rt.device)
    M, H = res.shape
    if via_dispatch:
        d = L.MmOpDesc()
        d.op, d.layer = L.OP_ADD_RMSNORM, -1
        d.a, d.b, d.c, d.d = t_res.data_ptr(), t_delta.data_ptr(), y.data_ptr(), t_gain.data_ptr()
        d.n0, d.n1, d.n2 = M, H, 0
        kc = L.MmKcall(C.pointer(d), C.c_void_p(1), None)
        L.check(rt.lib.mm_kx_invoke(C.byref(kc)), "mm_kx_invoke(OP_ADD_RMSNORM)")
    else:
        L.check(rt.lib.mm_add_rmsnorm(t_res.data_ptr(), t_delta.data_ptr(), y.data_ptr(), t_gain.data_ptr(),
                                      M, H, None), "mm_add_rmsnorm")
        rt.sync()
    assert rt.device_status() == 0
    return rt.from_device_bf16(t_res), rt.from_device_bf16(y)


@pytest.mark.parametrize("M,H", [(1, 64), (3, 1000), (4, 5120), (16, 5120), (2, 17408), (5, 77), (32, 8192 + 256)])
def test_add_rmsnorm_matches_the_oracle(rt, oracle, M, H):
    res = mm.make_activations(M, H, seed=H + M, std=2.0)
    delta = mm.make_activations(M, H, seed=H + M + 1)
    gain = mm.make_activations(1, H, seed=H + 2, std=0.2)[0]
    want_res, want_y = oracle.add_rmsnorm(res, delta, gain, rt.lib.mm_norm_eps_get())
    got_res, got_y = run_norm(rt, res, delta, gain, via_dispatch=(M % 2 == 1))
    assert np.array_equal(got_res, want_res)
    assert row_rel_l2(got_y, want_y) <= REL_L2_TOL
    assert bf16_steps(got_y, want_y) <= 1.0


def test_add_rmsnorm_reference_fixture(rt):
    """Outputs of the reference's own kernel (tests/golden/add_rmsnorm.npz)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    g = np.load(os.path.join(GOLDEN, "add_rmsnorm.npz"))
    assert rt.lib.mm_norm_eps_set(mg.ADD_RMSNORM_EPS) == L.MM_OK
    for (M, H) in mg.ADD_RMSNORM_SHAPES:
        res, delta, gain = mg.add_rmsnorm_inputs(M, H)
        got_res, got_y = run_norm(rt, res, delta, gain)
        assert np.array_equal(got_res, g[f"res_{M}x{H}"])
        assert bf16_steps(got_y, g[f"y_{M}x{H}"]) <= 1.0
        assert row_rel_l2(got_y, g[f"y_{M}x{H}"]) <= REL_L2_TOL


def test_epsilon_is_the_registered_value(rt, oracle):
    res = mm.make_activations(2, 512, seed=5, std=1.0e-3)       # small rows: epsilon matters
    delta = mm.make_activations(2, 512, seed=6, std=1.0e-3)
    gain = mm.make_activations(1, 512, seed=7)[0]
    try:
        for eps in (1.0e-5, 1.0e-6):
            assert rt.lib.mm_norm_eps_set(eps) == L.MM_OK
            _, want = oracle.add_rmsnorm(res, delta, gain, eps)
            _, got = run_norm(rt, res, delta, gain)
            assert bf16_steps(got, want) <= 1.0
        rt.lib.mm_log_set_level(-1)
        assert rt.lib.mm_norm_eps_set(-1.0) == L.MM_ERR_RANGE
        rt.lib.mm_log_set_level(1)
    finally:
        rt.lib.mm_norm_eps_set(1.0e-6)


def test_down_then_add_rmsnorm_in_one_graph(rt, oracle):
    """down projection -> residual add + norm, as the planner emits them, captured
    and replayed: the norm reads the projection's output, so it must wait for it."""
    torch = rt.torch
    M, K, N = 4, 2048, 1024
    w = mm.make_weight(N, K, seed=9).to_device(rt.device)
    xb = mm.make_activations(M, K, seed=10)
    resb = mm.make_activations(M, N, seed=11)
    gainb = mm.make_activations(1, N, seed=12, std=0.2)[0]
    x = rt.to_device_bf16(xb)
    delta = torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device)
    res = rt.to_device_bf16(resb)
    gain = rt.to_device_bf16(gainb.reshape(1, -1))
    y = torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device)
    want_delta = oracle.gemm_f4(xb, w.payload, w.scales, w.gs)
    want_res, want_y = oracle.add_rmsnorm(resb, want_delta, gainb, rt.lib.mm_norm_eps_get())
    for overlap in (0, 2):
        eng = mm.LinearEngine(rt, max_ops=4)
        eng.overlap(overlap)
        eng.add(x, w, delta)
        eng.add_add_rmsnorm(res, delta, y, gain)
        eng.capture()
        res.copy_(rt.to_device_bf16(resb))
        rt.sync()
        rt.torch.cuda.synchronize()
        eng.launch()
        rt.sync()
        assert rt.device_status() == 0
        got_delta = rt.from_device_bf16(delta)
        assert row_rel_l2(got_delta, want_delta) <= REL_L2_TOL
        # the oracle on the projection the device produced: the norm itself is then held to one step
        _, y_on_dev = oracle.add_rmsnorm(resb, got_delta, gainb, rt.lib.mm_norm_eps_get())
        assert bf16_steps(rt.from_device_bf16(y), y_on_dev) <= 1.0
        assert row_rel_l2(rt.from_device_bf16(y), want_y) <= REL_L2_TOL
        eng.close()
