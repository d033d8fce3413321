"""GPU parity of the block-scaled decode path (tcgen05 kind::mxf4nvf4 on the packed
weights, activations as e2m1 digit planes): single ops, the gated pair, the digit
planes themselves, and group launches, against the CPU oracle through the C-ABI.

Bar: per-row relative L2 <= 2^-8 after bf16 rounding; products of single
(nibble, scale) pairs bit-exact."""
import ctypes as C
import os

import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import V_MX, V_STREAM, _lib as L
from conftest import GOLDEN, REL_L2_TOL, row_rel_l2

pytestmark = pytest.mark.gpu

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def run(rt, x_bits, w, variant=V_MX):
    if w.dev_payload is None:
        w.to_device(rt.device)
    x = rt.to_device_bf16(x_bits)
    y = rt.gemm_f4(x, w, variant=variant)
    assert rt.device_status() == 0
    return rt.from_device_bf16(y)


def check(rt, oracle, M, K, N, seed=0, x=None, w=None, variant=V_MX):
    w = w or mm.make_weight(N, K, seed=seed)
    x = x if x is not None else mm.make_activations(M, K, seed=seed + 1)
    y = run(rt, x, w, variant)
    err = row_rel_l2(y, oracle.gemm_f4(x, w.payload, w.scales, w.gs))
    assert err <= REL_L2_TOL, f"M={M} K={K} N={N}: rel L2 {err}"
    return y


def test_decode_shapes_take_this_path_by_default(rt):
    for (M, K, N) in ((1, 5120, 5120), (16, 5120, 34816), (16, 17408, 5120), (32, 5120, 1024)):
        x = rt.torch.zeros((M, K), dtype=rt.torch.bfloat16, device=rt.device)
        plan = mm.select_plan(M, K, N, ws_bytes=rt.lib.mm_f4_workspace_bytes() // 8)
        assert plan.variant == V_MX
        del x


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("K,N", [(256, 256), (512, 40), (1024, 600), (5120, 1024)])
def test_shapes(rt, oracle, M, K, N):
    check(rt, oracle, M, K, N, seed=K + N + M)


@pytest.mark.parametrize("M,K,N", [(1, 5120, 5120), (8, 2048, 1000), (17, 512, 264), (16, 17408, 5120),
                                   (5, 17408, 5120), (1, 256, 8), (32, 256, 1)])
def test_split_k_ragged_tiles_and_long_k(rt, oracle, M, K, N):
    check(rt, oracle, M, K, N, seed=M + N)


@pytest.mark.parametrize("rows,split", [(256, 1), (236, 0), (128, 3), (48, 0), (32, 2), (16, 1)])
@pytest.mark.parametrize("M", [1, 16])
def test_rows_per_cta_and_forced_split(rt, oracle, M, rows, split):
    """Any tile height that is a multiple of 4 (idle second MMA half, ragged last tile)
    and any K split give the oracle's result."""
    rt.lib.mm_f4_tune(2, rows)
    rt.lib.mm_f4_tune(3, split)
    try:
        check(rt, oracle, M, 2048, 1000, seed=31)
    finally:
        rt.lib.mm_f4_tune(2, 0)
        rt.lib.mm_f4_tune(3, 0)


def test_deterministic_and_close_to_the_streaming_kernel(rt, oracle):
    w = mm.make_weight(5120, 17408, seed=2).to_device(rt.device)
    x = mm.make_activations(8, 17408, seed=3)
    a = run(rt, x, w)
    for _ in range(3):
        assert np.array_equal(run(rt, x, w), a)
    b = run(rt, x, w, V_STREAM)
    assert row_rel_l2(a, b) <= REL_L2_TOL / 4
    assert (a == b).mean() > 0.99


def test_every_scale_code(rt):
    """All 256 scale bytes (subnormals, negative scales, 0x7f / 0xff which decode to 0)
    and all payload bytes, against the reference's own output."""
    g = np.load(os.path.join(GOLDEN, "random_bytes.npz"))
    K = g["x"].shape[1]
    w = mm.NvFp4Weight(g["payload"], g["scales"], 1.0, g["payload"].shape[0], K)
    assert row_rel_l2(run(rt, g["x"], w), g["y"]) <= REL_L2_TOL


def test_single_products_are_bit_exact(rt, oracle):
    """A one-hot activation row picks one (nibble, scale) product per output: the tensor
    path must return exactly the oracle's bf16 for every one of them."""
    K, N = 256, 256
    rng = np.random.Generator(np.random.PCG64(7))
    pay = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    sc = rng.integers(0, 256, (N, K // 16), dtype=np.uint8)
    w = mm.NvFp4Weight(pay, sc, 1.0, N, K)
    for k, bits in ((0, 0x3F80), (1, 0xBF80), (17, 0x4049), (100, 0x3F80), (255, 0x0080), (64, 0x7F00)):
        x = np.zeros((1, K), np.uint16)
        x[0, k] = bits
        assert np.array_equal(run(rt, x, w), oracle.gemm_f4(x, pay, sc, 1.0)), (k, hex(bits))


@pytest.mark.parametrize("M", [1, 16])
def test_activation_range(rt, oracle, M):
    K, N = 2048, 512
    w = mm.make_weight(N, K, seed=3)
    xf = mm.linear.fill_normal(M, K, 4)
    xf[0, 5] = 3.0e-9
    xf[M - 1, 700] = 2.5e5
    xf[0, 1300:1310] = 0.0
    xf[M // 2, 1800] = -1.0e-30
    check(rt, oracle, M, K, N, x=mm.linear.f32_to_bf16(xf), w=w)
    check(rt, oracle, M, K, N, x=mm.linear.f32_to_bf16(xf * np.float32(1.0e-7)), w=w)
    check(rt, oracle, M, K, N, x=mm.linear.f32_to_bf16(xf * np.float32(1.0e25)), w=w)   # products stay below 2^128
    zero = np.zeros((M, K), np.uint16)
    assert not run(rt, zero, w).view(np.uint16).astype(np.uint32).__and__(0x7FFF).any()


def test_inf_or_nan_rows_give_nan_and_leave_other_rows_alone(rt, oracle):
    K, N = 512, 128
    w = mm.make_weight(N, K, seed=8)
    x = mm.make_activations(4, K, seed=9)
    good = run(rt, x, w)
    bad = x.copy()
    bad[1, 7] = 0x7F80            # +inf
    bad[3, 300] = 0x7FC1          # NaN
    y = run(rt, bad, w)
    f = (y.astype(np.uint32) << 16).view(np.float32)
    assert np.isnan(f[1]).all() and np.isnan(f[3]).all()
    assert np.array_equal(y[0], good[0]) and np.array_equal(y[2], good[2])


# ---------------------------------------------------------------- digit planes
def ue4m3(b):
    b = b.astype(np.int64)
    e, m = (b >> 3) & 15, b & 7
    return np.where(e == 0, m * 2.0 ** -9, (1 + m / 8.0) * 2.0 ** (e - 7.0))


@pytest.mark.parametrize("M,K", [(1, 256), (5, 1024), (16, 5120), (32, 2048)])
def test_digit_planes_reconstruct_the_activations(rt, M, K):
    """mm_f4_xslice: planes x scales x row factors give back x.  A block's unit is 2^U,
    U = max(E_block - 16, E_row - 19) with E the exponent of the largest magnitude: values
    that are multiples of the unit come back exactly (all within 2^9 of the block's largest,
    in blocks within 2^3 of the row's largest), the others rounded to nearest."""
    torch = rt.torch
    xf = mm.linear.fill_normal(M, K, 21)
    xf[0, :16] *= np.float32(2.0 ** -12)          # a block far below the row's largest
    xf[M - 1, 40] = 3.0e3
    xf[M // 2, 100:116] = 0.0
    xf[0, 200] = 2.0 ** -20                        # far below its own block's largest
    xb = mm.linear.f32_to_bf16(xf)
    x = rt.to_device_bf16(xb)
    n = rt.lib.mm_f4_xslice_bytes(M, K)
    assert n > 0
    scratch = torch.zeros(n, dtype=torch.uint8, device=rt.device)
    L.check(rt.lib.mm_f4_xslice(x.data_ptr(), M, K, scratch.data_ptr(), n, None), "xslice")
    rt.sync()
    assert rt.device_status() == 0
    s = scratch.cpu().numpy()
    R = 6 * ((M + 3) // 4 * 4)
    f = s[:8 * M].view(np.float32).astype(np.float64).reshape(M, 2)
    planes = s[16384:16384 + R * (K // 2)].reshape(R, K // 2)
    scales = s[16384 + R * (K // 2):16384 + R * (K // 2) + R * (K // 16)].reshape(R, K // 16)
    codes = np.empty((R, K), np.uint8)
    codes[:, 0::2] = planes & 15
    codes[:, 1::2] = planes >> 4
    val = E2M1[codes] * np.repeat(ue4m3(scales), 16, axis=1)
    got = val.reshape(R // 6, 6, K).sum(axis=1)[:M] * (f[:, 0] * f[:, 1])[:, None]
    want = mm.linear.bf16_to_f32(xb).astype(np.float64)
    assert not val[6 * M:].any()                    # padding rows
    bmax = np.abs(want).reshape(M, K // 16, 16).max(axis=2).repeat(16, axis=1)
    rmax = np.abs(want).max(axis=1, keepdims=True)
    with np.errstate(divide="ignore"):
        e_b = np.floor(np.log2(np.where(bmax > 0, bmax, 1.0)))
        e_row = np.floor(np.log2(rmax))
        e_v = np.floor(np.log2(np.where(want != 0, np.abs(want), 1.0)))
    unit = 2.0 ** np.maximum(e_b - 16, e_row - 19)
    exact = (want == 0) | (e_v - 7 >= np.log2(unit))        # bf16: 8 significant bits
    assert exact.mean() > 0.5
    assert np.array_equal(got[exact], want[exact])
    assert (np.abs(got - want) <= unit / 2).all()
    # the scales are powers of two the tensor core takes as they are
    live = scales[:6 * M]
    assert (((live & 7) == 0) | ((live >> 3) == 0)).all() and (live <= 0x78).all()
    sub = live[(live >> 3) == 0]
    assert np.isin(sub, (0, 1, 2, 4)).all()


def test_xslice_refuses_what_it_cannot_take(rt):
    torch = rt.torch
    x = torch.zeros((4, 512), dtype=torch.bfloat16, device=rt.device)
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device=rt.device)
    assert rt.lib.mm_f4_xslice_bytes(33, 512) == 0 and rt.lib.mm_f4_xslice_bytes(4, 272) == 0
    assert rt.lib.mm_f4_xslice(x.data_ptr(), 33, 512, buf.data_ptr(), 1 << 20, None) == 4       # MM_ERR_SHAPE
    assert rt.lib.mm_f4_xslice(x.data_ptr(), 4, 512, buf.data_ptr() + 16, 1 << 19, None) == 4
    assert rt.lib.mm_f4_xslice(x.data_ptr(), 4, 512, buf.data_ptr(), 1024, None) != 0           # too small


# ---------------------------------------------------------------- gated pair
@pytest.mark.parametrize("M,K,inter", [(1, 512, 128), (4, 1024, 384), (16, 5120, 1024), (7, 1024, 1000)])
def test_gate_up_fused(rt, oracle, M, K, inter):
    full = mm.make_weight(2 * inter, K, seed=11)
    wg, wu = full.rows(0, inter), full.rows(inter, 2 * inter)
    keep = mm.place_weights([wg, wu], rt.device)
    plan = mm.select_plan(M, K, inter, ws_bytes=rt.lib.mm_f4_workspace_bytes() // 8, glu=True)
    assert plan.variant == V_MX
    xb = mm.make_activations(M, K, seed=12)
    x = rt.to_device_bf16(xb)
    y = rt.torch.empty((M, inter), dtype=rt.torch.bfloat16, device=rt.device)
    rt.mlp_gate_up_async(x, wg, wu, y)
    rt.sync()
    assert rt.device_status() == 0
    # silu(g) * u of two bf16-rounded GEMMs (the reference's three ops) against one fp32 epilogue:
    # twice the single-op bar
    assert row_rel_l2(rt.from_device_bf16(y), oracle.mlp_gate_up(xb, wg, wu)) <= 2 * REL_L2_TOL
    del keep


def test_gate_up_with_up_below_gate_in_memory(rt, oracle):
    M, K, inter = 4, 1024, 256
    full = mm.make_weight(2 * inter, K, seed=13)
    wu, wg = full.rows(0, inter), full.rows(inter, 2 * inter)          # up first in the arena
    keep = mm.place_weights([wu, wg], rt.device)
    xb = mm.make_activations(M, K, seed=14)
    y = rt.torch.empty((M, inter), dtype=rt.torch.bfloat16, device=rt.device)
    rt.mlp_gate_up_async(rt.to_device_bf16(xb), wg, wu, y)
    rt.sync()
    assert row_rel_l2(rt.from_device_bf16(y), oracle.mlp_gate_up(xb, wg, wu)) <= 2 * REL_L2_TOL
    del keep


# ---------------------------------------------------------------- group launch
GROUP_SHAPES = [(4, 1024, 600), (4, 1024, 300), (8, 2048, 1000), (1, 5120, 1024), (16, 5120, 1024), (3, 512, 40),
                (16, 17408, 512), (2, 256, 128), (32, 1024, 256)]


def group_case(rt):
    ws = [mm.make_weight(N, K, seed=i).to_device(rt.device) for i, (M, K, N) in enumerate(GROUP_SHAPES)]
    xb = [mm.make_activations(M, K, seed=50 + i) for i, (M, K, N) in enumerate(GROUP_SHAPES)]
    xb[1] = xb[0]                                   # two ops on the same activations
    xs = [rt.to_device_bf16(v) for v in xb]
    xs[1] = xs[0]
    ys = [rt.torch.zeros((M, N), dtype=rt.torch.bfloat16, device=rt.device) for (M, K, N) in GROUP_SHAPES]
    return ws, xb, xs, ys


@pytest.mark.parametrize("captured", [False, True])
def test_group_launch_matches_the_oracle(rt, oracle, captured):
    ws, xb, xs, ys = group_case(rt)
    eng = mm.LinearEngine(rt, max_ops=16)
    try:
        for x, w, y in zip(xs, ws, ys):
            eng.add(x, w, y)
        if captured:
            eng.capture()
        for _ in range(3 if captured else 1):          # replays reuse counters and scratch
            for y in ys:
                y.zero_()
            eng.launch()
            rt.sync()
            assert rt.device_status() == 0
            assert eng.n_group_launches() == 1 and eng.n_independent() == len(GROUP_SHAPES) - 1
            for i in range(len(GROUP_SHAPES)):
                want = oracle.gemm_f4(xb[i], ws[i].payload, ws[i].scales, ws[i].gs)
                assert row_rel_l2(rt.from_device_bf16(ys[i]), want) <= REL_L2_TOL, GROUP_SHAPES[i]
    finally:
        eng.close()


def test_group_launch_can_be_switched_off(rt, oracle):
    ws, xb, xs, ys = group_case(rt)
    eng = mm.LinearEngine(rt, max_ops=16)
    try:
        eng.group(False)
        for x, w, y in zip(xs, ws, ys):
            eng.add(x, w, y)
        eng.launch()
        rt.sync()
        assert eng.n_group_launches() == 0 and rt.device_status() == 0
        for i in range(len(GROUP_SHAPES)):
            want = oracle.gemm_f4(xb[i], ws[i].payload, ws[i].scales, ws[i].gs)
            assert row_rel_l2(rt.from_device_bf16(ys[i]), want) <= REL_L2_TOL
    finally:
        eng.close()


def test_dependent_ops_do_not_share_a_group(rt, oracle):
    """down reads what gate+up writes: two launches, the second after the first."""
    M, K, inter = 4, 1024, 512
    full = mm.make_weight(2 * inter, K, seed=21)
    wg, wu = full.rows(0, inter), full.rows(inter, 2 * inter)
    wd = mm.make_weight(K, inter, seed=22)
    keep = mm.place_weights([wg, wu, wd], rt.device)
    xb = mm.make_activations(M, K, seed=23)
    x = rt.to_device_bf16(xb)
    torch = rt.torch
    g = torch.zeros((M, inter), dtype=torch.bfloat16, device=rt.device)
    u = torch.zeros_like(g)
    h = torch.zeros_like(g)
    y = torch.zeros((M, K), dtype=torch.bfloat16, device=rt.device)
    eng = mm.LinearEngine(rt, max_ops=8)
    try:
        eng.fuse_mlp(True)
        eng.add(x, wg, g)
        eng.add(x, wu, u)
        eng.add_silu_mul(g, u, h)
        eng.add(h, wd, y)
        eng.capture()
        eng.launch()
        rt.sync()
        assert rt.device_status() == 0 and eng.n_group_launches() == 2
        hb = rt.from_device_bf16(h)
        assert row_rel_l2(hb, oracle.mlp_gate_up(xb, wg, wu)) <= 2 * REL_L2_TOL
        want = oracle.gemm_f4(hb, wd.payload, wd.scales, wd.gs)           # down on the hidden the GPU produced
        assert row_rel_l2(rt.from_device_bf16(y), want) <= REL_L2_TOL
    finally:
        eng.close()
    del keep


def test_more_ops_than_one_launch_holds(rt, oracle):
    """60 small ops: the op list of a launch holds 48, so the engine makes two."""
    M, K, N = 2, 512, 96
    ws = [mm.make_weight(N, K, seed=100 + i).to_device(rt.device) for i in range(6)]
    xb = [mm.make_activations(M, K, seed=200 + i) for i in range(60)]
    xs = [rt.to_device_bf16(v) for v in xb]
    ys = [rt.torch.zeros((M, N), dtype=rt.torch.bfloat16, device=rt.device) for _ in range(60)]
    eng = mm.LinearEngine(rt, max_ops=64)
    try:
        for i in range(60):
            eng.add(xs[i], ws[i % 6], ys[i])
        eng.launch()
        rt.sync()
        assert rt.device_status() == 0 and eng.n_group_launches() == 2
        for i in range(60):
            w = ws[i % 6]
            assert row_rel_l2(rt.from_device_bf16(ys[i]), oracle.gemm_f4(xb[i], w.payload, w.scales, w.gs)) <= REL_L2_TOL
    finally:
        eng.close()


def test_group_launch_of_tensor_parallel_ops(rt, oracle):
    """mm_lin_engine_add_tp: three linears, each the second of two N-shards, every output tile
    stored at its column offset into two full-width buffers (what two ranks would hold), all
    in one group launch; the other shard's columns stay untouched."""
    torch = rt.torch
    shapes = [(4, 1024, 1200), (16, 2048, 512), (1, 5120, 2048)]
    ws = [mm.make_weight(N, K, seed=70 + i) for i, (M, K, N) in enumerate(shapes)]
    xb = [mm.make_activations(M, K, seed=80 + i) for i, (M, K, N) in enumerate(shapes)]
    xs = [rt.to_device_bf16(v) for v in xb]
    shards = [w.rows(w.N // 2, w.N).to_device(rt.device) for w in ws]
    outs = [[torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for _ in range(2)] for (M, K, N) in shapes]
    torch.cuda.synchronize()
    eng = mm.LinearEngine(rt, max_ops=8)
    try:
        keep = []
        for x, sh, (a, b), w in zip(xs, shards, outs, ws):
            ptrs = (C.c_void_p * 2)(a.data_ptr(), b.data_ptr())
            keep.append(ptrs)
            eng.add_tp(x, sh, a, ptrs, 2, w.N // 2)
        eng.capture()
        for _ in range(2):
            eng.launch()
        rt.sync()
        assert rt.device_status() == 0 and eng.n_group_launches() == 1
        for i, w in enumerate(ws):
            a, b = rt.from_device_bf16(outs[i][0]), rt.from_device_bf16(outs[i][1])
            assert np.array_equal(a, b)
            h = w.N // 2
            assert not a[:, :h].any()
            want = oracle.gemm_f4(xb[i], w.payload, w.scales, w.gs, n_begin=h, n_end=w.N)
            assert row_rel_l2(a[:, h:], want) <= REL_L2_TOL, shapes[i]
    finally:
        eng.close()


@pytest.mark.parametrize("seed", range(12))
def test_random_groups(rt, oracle, seed):
    """Seeded random groups: 1 to 14 ops of random decode shapes (ragged N, K from 256 to 8192,
    M from 1 to 32, some sharing activations), captured and replayed twice, every output
    against the oracle.  Exercises the planner's K-split search, the unit hand-out and the
    split-K exchange on launches of very different lengths."""
    torch = rt.torch
    rng = np.random.Generator(np.random.PCG64(1000 + seed))
    n_ops = int(rng.integers(1, 15))
    ws, xb, xs, ys, shapes = [], [], [], [], []
    for i in range(n_ops):
        M = int(rng.choice([1, 2, 3, 4, 7, 8, 16, 17, 32]))
        K = 256 * int(rng.choice([1, 2, 4, 8, 20, 32]))
        N = int(rng.choice([8, 40, 136, 256, 600, 1000, 1024, 2048, 3000]))
        if i and rng.random() < 0.3 and shapes[-1][1] == K:      # reads the activations of the op in front
            M = shapes[-1][0]
            xb.append(xb[-1])
            xs.append(xs[-1])
        else:
            xb.append(mm.make_activations(M, K, seed=int(rng.integers(1 << 30))))
            xs.append(rt.to_device_bf16(xb[-1]))
        shapes.append((M, K, N))
        ws.append(mm.make_weight(N, K, seed=int(rng.integers(1 << 30))).to_device(rt.device))
        ys.append(torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device))
    torch.cuda.synchronize()
    eng = mm.LinearEngine(rt, max_ops=16)
    try:
        for x, w, y in zip(xs, ws, ys):
            eng.add(x, w, y)
        eng.capture()
        first = None
        for _ in range(2):
            eng.launch()
            rt.sync()
            assert rt.device_status() == 0
            got = [rt.from_device_bf16(y) for y in ys]
            if first is not None:
                assert all(np.array_equal(a, b) for a, b in zip(first, got))       # replays give the same bits
            first = got
        assert eng.n_group_launches() >= 1
        for i, w in enumerate(ws):
            want = oracle.gemm_f4(xb[i], w.payload, w.scales, w.gs)
            assert row_rel_l2(first[i], want) <= REL_L2_TOL, (seed, i, shapes[i])
    finally:
        eng.close()
