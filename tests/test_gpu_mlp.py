"""The MLP front half on the GPU: the fused gate/up/silu kernel
(mm_f4_mlp_gate_up), the unfused SILU_MUL op, the engine's fusion of the
reference planner's three-op sequence, and OP_LMHEAD, against the CPU oracle."""
import ctypes as C
import os

import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import _lib as L
from conftest import GOLDEN, REL_L2_TOL, bf16_bits_to_f32, row_rel_l2

pytestmark = pytest.mark.gpu


def _pair(rt, K, inter, seed, order="gate_first"):
    wg = mm.make_weight(inter, K, seed=seed, std=0.02)
    wu = mm.make_weight(inter, K, seed=seed + 100, std=0.02)
    keep = mm.place_weights([wg, wu] if order == "gate_first" else [wu, wg], rt.device)
    return wg, wu, keep


def _exact_fraction(a, b):
    return float(np.mean(a == b))


# (M, K, inter): decode shapes; tails in inter (not a multiple of 128), split-K on and off
DECODE = [(1, 1024, 384), (5, 2048, 200), (8, 5120, 128), (16, 1024, 1000), (17, 512, 256),
          (32, 4096, 136), (2, 256, 17408)]


@pytest.mark.parametrize("M,K,inter", DECODE)
@pytest.mark.parametrize("order", ["gate_first", "up_first"])
@pytest.mark.parametrize("kernel", ["block_scaled", "streaming"])
def test_gate_up_decode(rt, oracle, M, K, inter, order, kernel):
    rt.lib.mm_f4_tune(5, 1 if kernel == "block_scaled" else 0)
    try:
        _gate_up_decode(rt, oracle, M, K, inter, order, L.V_MX if kernel == "block_scaled" else L.V_STREAM)
    finally:
        rt.lib.mm_f4_tune(5, 1)


def _gate_up_decode(rt, oracle, M, K, inter, order, variant):
    wg, wu, keep = _pair(rt, K, inter, seed=M + inter, order=order)
    xb = mm.make_activations(M, K, seed=3)
    x = rt.to_device_bf16(xb)
    y = rt.torch.full((M, inter), 7.0, dtype=rt.torch.bfloat16, device=rt.device)
    if variant == L.V_MX:                                   # the selector's default for a decode pair
        assert mm.select_plan(M, K, inter, ws_bytes=rt.lib.mm_f4_workspace_bytes() // 8, glu=True).variant == variant
    rt.mlp_gate_up_async(x, wg, wu, y)
    rt.sync()
    assert rt.device_status() == 0
    got = rt.from_device_bf16(y)
    ref = oracle.mlp_gate_up(xb, wg, wu)
    assert row_rel_l2(got, ref) <= REL_L2_TOL
    assert _exact_fraction(got, ref) > 0.9
    # deterministic: a second run is bitwise equal (split-K sums in slice order)
    y2 = rt.torch.zeros_like(y)
    rt.mlp_gate_up_async(x, wg, wu, y2)
    rt.sync()
    assert np.array_equal(got, rt.from_device_bf16(y2))


PREFILL = [(64, 512, 256), (200, 1024, 392), (300, 256, 128), (129, 768, 1000), (520, 512, 264)]


@pytest.mark.parametrize("M,K,inter", PREFILL)
def test_gate_up_prefill(rt, oracle, M, K, inter):
    wg, wu, keep = _pair(rt, K, inter, seed=M, order="gate_first" if M % 2 == 0 else "up_first")
    xb = mm.make_activations(M, K, seed=4)
    x = rt.to_device_bf16(xb)
    y = rt.torch.full((M, inter), 7.0, dtype=rt.torch.bfloat16, device=rt.device)
    plan = mm.select_plan(M, K, inter, glu=True)
    assert plan.variant == L.V_UMMA and plan.tile_n == 256
    rt.mlp_gate_up_async(x, wg, wu, y)
    rt.sync()
    assert rt.device_status() == 0
    got = rt.from_device_bf16(y)
    ref = oracle.mlp_gate_up(xb, wg, wu)
    assert row_rel_l2(got, ref) <= REL_L2_TOL
    assert _exact_fraction(got, ref) > 0.9


def test_gate_up_matches_three_ops_on_device(rt, oracle):
    """Fused kernel against the same library's gate GEMM, up GEMM and SILU_MUL, and both
    against the oracle's three ops."""
    torch = rt.torch
    for (M, K, inter) in [(4, 5120, 1024), (96, 1024, 512)]:
        wg, wu, keep = _pair(rt, K, inter, seed=11)
        xb = mm.make_activations(M, K, seed=5)
        x = rt.to_device_bf16(xb)
        g = torch.empty((M, inter), dtype=torch.bfloat16, device=rt.device)
        u = torch.empty_like(g)
        y3 = torch.empty_like(g)
        y1 = torch.empty_like(g)
        rt.linear_async(x, wg, g)
        rt.linear_async(x, wu, u)
        rt.silu_mul_async(g, u, y3)
        rt.mlp_gate_up_async(x, wg, wu, y1)
        rt.sync()
        assert rt.device_status() == 0
        a, b = rt.from_device_bf16(y1), rt.from_device_bf16(y3)
        assert _exact_fraction(a, b) > 0.99           # same epilogue arithmetic; K slices may differ
        assert row_rel_l2(a, b) <= 2.0 ** -10
        want = oracle.mlp_gate_up(xb, wg, wu)
        assert row_rel_l2(a, want) <= REL_L2_TOL and row_rel_l2(b, want) <= REL_L2_TOL
        assert _exact_fraction(a, want) > 0.9


def test_gate_up_rejects_what_it_cannot_fuse(rt):
    torch = rt.torch
    wg, wu, keep = _pair(rt, 272, 64, seed=1)                # K % 256 != 0
    x = rt.to_device_bf16(mm.make_activations(2, 272, seed=1))
    y = torch.empty((2, 64), dtype=torch.bfloat16, device=rt.device)
    with pytest.raises(L.MimferError) as e:
        rt.mlp_gate_up_async(x, wg, wu, y)
    assert e.value.status == L.MM_ERR_UNSUPPORTED
    # payload and scale tensors in opposite address order
    wa, wb, keep2 = _pair(rt, 256, 128, seed=2)
    wa.dev_scales, wb.dev_scales = wb.dev_scales, wa.dev_scales
    x = rt.to_device_bf16(mm.make_activations(2, 256, seed=1))
    y = torch.empty((2, 128), dtype=torch.bfloat16, device=rt.device)
    with pytest.raises(L.MimferError) as e:
        rt.mlp_gate_up_async(x, wa, wb, y)
    assert e.value.status == L.MM_ERR_UNSUPPORTED


def test_silu_mul_all_gate_patterns(rt, oracle):
    """Every bf16 gate value (the golden fixture's inputs): NaN where the
    reference gives NaN, otherwise within one bf16 step, almost always equal."""
    gate = np.arange(65536, dtype=np.uint16)
    up = np.random.Generator(np.random.PCG64(5)).integers(0, 65536, 65536, dtype=np.uint16)
    ref = np.load(os.path.join(GOLDEN, "silu_mul.npz"))["y"]
    g, u = rt.to_device_bf16(gate), rt.to_device_bf16(up)
    y = rt.torch.empty_like(g)
    rt.silu_mul_async(g, u, y)
    rt.sync()
    got = rt.from_device_bf16(y)
    rf, gf = bf16_bits_to_f32(ref), bf16_bits_to_f32(got)
    nan = np.isnan(rf)
    assert np.array_equal(nan, np.isnan(gf))
    ok = ~nan
    assert _exact_fraction(got[ok], ref[ok]) > 0.995
    # differing results are neighbours: same sign, adjacent bit patterns
    d = np.abs(got[ok].astype(np.int32) - ref[ok].astype(np.int32))
    assert d.max() <= 1


@pytest.mark.parametrize("n,offset", [(1, 0), (7, 0), (4099, 0), (1 << 20, 0), (1000, 1)])
def test_silu_mul_sizes(rt, oracle, n, offset):
    gb = mm.make_activations(1, n + offset, seed=9, std=3.0)[0]
    ub = mm.make_activations(1, n + offset, seed=10)[0]
    g, u = rt.to_device_bf16(gb), rt.to_device_bf16(ub)
    y = rt.torch.zeros_like(g)
    rt.silu_mul_async(g[offset:], u[offset:], y[offset:])       # offset 1: no 16-byte alignment
    rt.sync()
    got = rt.from_device_bf16(y)[offset:]
    ref = oracle.silu_mul(gb[offset:], ub[offset:])
    assert _exact_fraction(got, ref) > 0.99
    assert row_rel_l2(got[None, :], ref[None, :]) <= REL_L2_TOL


def _mlp_engine(rt, x, wg, wu, g, u, y, fuse):
    eng = mm.LinearEngine(rt)
    eng.fuse_mlp(fuse)
    eng.add(x, wg, g, note=b"gate")
    eng.add(x, wu, u, note=b"up")
    eng.add_silu_mul(g, u, y)
    return eng


@pytest.mark.parametrize("M,K,inter", [(4, 1024, 512), (80, 512, 256)])
def test_engine_fuses_the_planner_sequence(rt, oracle, M, K, inter):
    torch = rt.torch
    wg, wu, keep = _pair(rt, K, inter, seed=21)
    xb = mm.make_activations(M, K, seed=6)
    x = rt.to_device_bf16(xb)
    ref = oracle.mlp_gate_up(xb, wg, wu)
    for fuse, n_ops in ((False, 3), (True, 1)):
        g = torch.full((M, inter), 5.0, dtype=torch.bfloat16, device=rt.device)
        u = torch.full_like(g, 5.0)
        y = torch.zeros_like(g)
        eng = _mlp_engine(rt, x, wg, wu, g, u, y, fuse)
        assert eng.n_ops() == n_ops
        for captured in (False, True):
            if captured:
                eng.capture()
            y.zero_()
            eng.launch()
            rt.sync()
            assert row_rel_l2(rt.from_device_bf16(y), ref) <= REL_L2_TOL
        if fuse:                                 # the gate and up buffers are never written
            assert float(g.float().min()) == 5.0 and float(u.float().max()) == 5.0
        eng.close()


def test_engine_keeps_three_ops_when_fusion_is_impossible(rt, oracle):
    torch = rt.torch
    M, K, inter = 3, 272, 96                      # K % 256 != 0: fallback kernel
    wg, wu, keep = _pair(rt, K, inter, seed=31)
    xb = mm.make_activations(M, K, seed=7)
    x = rt.to_device_bf16(xb)
    g = torch.empty((M, inter), dtype=torch.bfloat16, device=rt.device)
    u, y = torch.empty_like(g), torch.zeros_like(g)
    eng = _mlp_engine(rt, x, wg, wu, g, u, y, True)
    assert eng.n_ops() == 3
    eng.launch()
    rt.sync()
    assert row_rel_l2(rt.from_device_bf16(y), oracle.mlp_gate_up(xb, wg, wu)) <= REL_L2_TOL
    eng.close()


def test_lmhead_opcode_routes_to_the_fp4_kernels(rt, oracle):
    M, K, N = 3, 512, 1000
    w = mm.make_weight(N, K, seed=41).to_device(rt.device)
    xb = mm.make_activations(M, K, seed=8)
    x = rt.to_device_bf16(xb)
    y = rt.torch.zeros((M, N), dtype=rt.torch.bfloat16, device=rt.device)
    d = rt.op_desc(x, w, y, op=L.OP_LMHEAD, note=b"lmhead")
    kc = L.MmKcall(C.pointer(d), C.c_void_p(1), None)
    L.check(rt.lib.mm_kx_invoke(C.byref(kc)), "mm_kx_invoke(OP_LMHEAD)")
    assert row_rel_l2(rt.from_device_bf16(y), oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL
    d.d = None                                    # bf16 head: not served
    assert rt.lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_UNSUPPORTED
    assert rt.lib.kx_cuda_oppref(L.OP_LMHEAD) == 1 and rt.lib.kx_cuda_oppref(L.OP_SILU_MUL) == 1
