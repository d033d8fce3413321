"""GPU parity: every kernel family against the CPU oracle, through the C-ABI.

Bar: nibble/scale decode bit-exact; outputs within per-row relative L2 <= 2^-8
of the oracle after bf16 rounding (conftest.REL_L2_TOL)."""
import ctypes as C
import glob
import os

import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import V_ROWWARP, V_STREAM, V_UMMA, _lib as L
from conftest import GOLDEN, REL_L2_TOL, row_rel_l2

pytestmark = pytest.mark.gpu


def run(rt, x_bits, w, variant=None):
    if w.dev_payload is None:
        w.to_device(rt.device)
    x = rt.to_device_bf16(x_bits)
    y = rt.gemm_f4(x, w, variant=variant)
    assert rt.device_status() == 0
    return rt.from_device_bf16(y)


def check(rt, oracle, M, K, N, variant, seed=0, gs=None, sample_rows=None):
    w = mm.make_weight(N, K, seed=seed)
    if gs is not None:
        w.gs = gs
    x = mm.make_activations(M, K, seed=seed + 1)
    y = run(rt, x, w, variant)
    rows = None if sample_rows is None else sorted(set(sample_rows))
    want = oracle.gemm_f4(x, w.payload, w.scales, w.gs, rows=rows)
    got = y if rows is None else y[rows]
    err = row_rel_l2(got, want)
    assert err <= REL_L2_TOL, f"M={M} K={K} N={N} variant={variant}: rel L2 {err}"
    return y


# ---------------------------------------------------------------- decode
def test_decode_is_bit_exact(rt, oracle):
    bf16_form, f32, f16_form = rt.decode_probe()
    table = oracle.decode_table()
    assert not (bf16_form == 0xDEADBEEF).any(), "nibble positions of a word disagree"
    assert not (f16_form == 0xDEADBEEF).any(), "fp16 form: nibble positions or column order disagree"
    assert np.array_equal(f32, table)
    assert np.array_equal(bf16_form, table)
    assert np.array_equal(f16_form, table)


def test_decode_matches_reference_fixture(rt):
    gold = np.load(os.path.join(GOLDEN, "decode_products.npz"))
    ref = (gold["low_nibble_col0"].astype(np.uint32) << 16).view(np.float32)
    for form in rt.decode_probe():
        assert np.array_equal(form.view(np.float32), ref)


# ---------------------------------------------------------------- row-warp
@pytest.mark.parametrize("M,K,N", [(1, 16, 1), (1, 48, 7), (3, 528, 33), (5, 1024, 96), (17, 272, 100),
                                   (2, 5120, 64), (40, 256, 20)])
def test_rowwarp(rt, oracle, M, K, N):
    check(rt, oracle, M, K, N, V_ROWWARP, seed=M + N)


# ---------------------------------------------------------------- stream (decode)
@pytest.mark.parametrize("M", [1, 2, 3, 4, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("K,N", [(256, 256), (512, 40), (1024, 600), (5120, 1024)])
def test_stream_shapes(rt, oracle, M, K, N):
    check(rt, oracle, M, K, N, V_STREAM, seed=K + N + M)


def test_stream_config1(rt, oracle):
    check(rt, oracle, 1, 5120, 5120, None)


@pytest.mark.parametrize("M", [1, 16])
def test_stream_long_k_split(rt, oracle, M):
    plan = mm.select_plan(M, 17408, 5120, ws_bytes=rt.lib.mm_f4_workspace_bytes(), variant=V_STREAM)
    assert plan.variant == V_STREAM and plan.split_k > 1
    check(rt, oracle, M, 17408, 5120, V_STREAM, seed=5)


@pytest.mark.parametrize("rows,split", [(256, 1), (240, 0), (128, 3), (48, 0), (16, 2)])
@pytest.mark.parametrize("M", [1, 16])
def test_stream_rows_per_cta(rt, oracle, M, rows, split):
    """The decode kernel with any multiple of 16 weight rows per CTA (idle consumer
    warps, ragged last tile) and a forced K split: same result as the oracle, and
    bit-for-bit the 256-row result when the K split is the same."""
    K, N = 2048, 1000
    want = check(rt, oracle, M, K, N, V_STREAM, seed=31)
    base = mm.select_plan(M, K, N, ws_bytes=rt.lib.mm_f4_workspace_bytes(), variant=V_STREAM)
    assert base.split_k == 2                   # K / 256 = 8 steps, at least 4 per slice
    rt.lib.mm_f4_tune(2, rows)
    rt.lib.mm_f4_tune(3, split)
    try:
        got = check(rt, oracle, M, K, N, V_STREAM, seed=31)
    finally:
        rt.lib.mm_f4_tune(2, 0)
        rt.lib.mm_f4_tune(3, 0)
    if split != 1:                             # every other case ends up with two K slices too
        assert np.array_equal(got, want)


def test_stream_without_workspace(rt, oracle):
    ws = rt.workspace
    rt.sync()
    L.check(rt.lib.mm_f4_workspace_set(None, 0), "clear workspace")
    try:
        check(rt, oracle, 4, 4096, 512, V_STREAM, seed=9)
    finally:
        L.check(rt.lib.mm_f4_workspace_set(ws.data_ptr(), ws.numel()), "restore workspace")


@pytest.mark.parametrize("M", [1, 8, 16, 32])
def test_stream_activation_range_picks_operand_format(rt, oracle, M):
    """K steps whose activations do not convert to fp16 exactly (tiny, huge)
    take the bf16 operand path; both paths share the accumulators."""
    K, N = 2048, 512
    w = mm.make_weight(N, K, seed=3)
    xf = mm.linear.fill_normal(M, K, 4)
    xf[0, 5] = 3.0e-9            # step 0: below 2^-17
    xf[M - 1, 700] = 2.5e5       # step 2: above 2^16
    xf[0, 1300:1310] = 0.0       # zeros are exact in both formats
    xf[M // 2, 1800] = -1.0e-30  # step 7
    x = mm.linear.f32_to_bf16(xf)
    y = run(rt, x, w, V_STREAM)
    assert row_rel_l2(y, oracle.gemm_f4(x, w.payload, w.scales, w.gs)) <= REL_L2_TOL
    # all steps out of range
    x2 = mm.linear.f32_to_bf16(xf * np.float32(1.0e-7))
    y2 = run(rt, x2, w, V_STREAM)
    assert row_rel_l2(y2, oracle.gemm_f4(x2, w.payload, w.scales, w.gs)) <= REL_L2_TOL


def test_stream_is_deterministic(rt, oracle):
    w = mm.make_weight(5120, 17408, seed=2).to_device(rt.device)
    x = mm.make_activations(8, 17408, seed=3)
    a = run(rt, x, w)
    for _ in range(3):
        assert np.array_equal(run(rt, x, w), a)


# ---------------------------------------------------------------- umma (prefill)
@pytest.mark.parametrize("M,K,N", [(128, 256, 128), (256, 256, 256), (33, 512, 136), (300, 1024, 520),
                                   (512, 2048, 1024), (1000, 768, 264)])
def test_umma_shapes(rt, oracle, M, K, N):
    check(rt, oracle, M, K, N, V_UMMA, seed=M + N)


@pytest.mark.parametrize("tile", [(256, 256), (128, 256), (128, 128)])
def test_umma_every_tile_shape(rt, oracle, tile):
    # shapes chosen so the selector lands on each tile
    shapes = {(256, 256): (8192, 256, 8192), (128, 256): (128, 512, 37888), (128, 128): (128, 256, 128)}
    M, K, N = shapes[tile]
    plan = mm.select_plan(M, K, N)
    assert (plan.tile_m, plan.tile_n) == tile, plan.as_dict()
    rows = [0, 1, 127, 128, M // 2, M - 1] if M > 512 else None
    check(rt, oracle, M, K, N, V_UMMA, seed=1, sample_rows=rows)


@pytest.mark.parametrize("M,K,N", [(512, 2048, 1024), (300, 1024, 520), (2048, 6144, 5120), (512, 5120, 1024)])
def test_umma_tail_split_matches_whole_tiles(rt, oracle, M, K, N):
    """Tiles of the last wave cut into K slices (partial sums through the workspace, added
    in slice order by the tail kernel) against the same op with whole tiles: both within the
    op's tolerance of the oracle, the split result the same bits on every run."""
    plan = mm.select_plan(M, K, N, ws_bytes=rt.lib.mm_f4_workspace_bytes() // 8)
    assert plan.variant == V_UMMA and plan.split_k > 1 and plan.m_tiles > 0
    w = mm.make_weight(N, K, seed=17).to_device(rt.device)
    x = mm.make_activations(M, K, seed=18)
    rows = None if M * N <= 1 << 20 else [0, 127, 128, 255, 256, M - 1]
    want = oracle.gemm_f4(x, w.payload, w.scales, w.gs, rows=rows)
    a = run(rt, x, w)
    assert np.array_equal(run(rt, x, w), a)
    assert rt.lib.mm_f4_tune(8, 0) == 1
    try:
        b = run(rt, x, w)
    finally:
        rt.lib.mm_f4_tune(8, 1)
    for y in (a, b):
        assert row_rel_l2(y if rows is None else y[rows], want) <= REL_L2_TOL
    assert row_rel_l2(a, b) <= REL_L2_TOL / 4          # two roundings of different fp32 sums


@pytest.mark.parametrize("seed", range(8))
def test_umma_random_shapes(rt, oracle, seed):
    """Seeded random prefill shapes (ragged M and N, short and long K, tail split or not),
    sampled rows against the oracle."""
    rng = np.random.Generator(np.random.PCG64(500 + seed))
    M = int(rng.choice([33, 100, 129, 300, 700, 1500, 3000]))
    K = 256 * int(rng.choice([1, 2, 4, 12, 20, 32]))
    N = 8 * int(rng.integers(1, 700))
    assert mm.select_plan(M, K, N, ws_bytes=rt.lib.mm_f4_workspace_bytes() // 8).variant == V_UMMA
    rows = sorted(set([0, M - 1, M // 2] + [int(v) for v in rng.integers(0, M, 5)]))
    check(rt, oracle, M, K, N, None, seed=seed, sample_rows=rows)


def test_umma_prefill_gate_up_sampled(rt, oracle):
    M, K, N = 2048, 5120, 34816
    check(rt, oracle, M, K, N, None, seed=0, sample_rows=[0, 255, 256, 1023, 2047])


def test_umma_is_deterministic(rt, oracle):
    w = mm.make_weight(1024, 1024, seed=2).to_device(rt.device)
    x = mm.make_activations(512, 1024, seed=3)
    a = run(rt, x, w)
    assert np.array_equal(run(rt, x, w), a)


# ---------------------------------------------------------------- fixtures, edge cases
@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "seeded_*.npz"))),
                         ids=lambda p: os.path.basename(p)[:-4])
def test_seeded_reference_fixtures(rt, path):
    g = np.load(path)
    M, K, N = (int(v) for v in os.path.basename(path)[7:-4].split("x"))
    w = mm.make_weight(N, K, seed=0)
    w.gs = 1.0                                   # the reference has no global scale
    x = mm.make_activations(M, K, seed=1)
    assert row_rel_l2(run(rt, x, w), g["y"]) <= REL_L2_TOL


@pytest.mark.parametrize("variant", [V_ROWWARP, V_STREAM])
def test_random_bytes_fixture(rt, variant):
    """All 256 scale codes: NaN codes decode to 0, negative scales keep their sign."""
    g = np.load(os.path.join(GOLDEN, "random_bytes.npz"))
    M, K = g["x"].shape
    w = mm.NvFp4Weight(g["payload"], g["scales"], 1.0, g["payload"].shape[0], K)
    assert row_rel_l2(run(rt, g["x"], w, variant), g["y"]) <= REL_L2_TOL


def test_random_bytes_umma(rt, oracle):
    rng = np.random.Generator(np.random.PCG64(5))
    M, K, N = 130, 512, 264
    w = mm.NvFp4Weight(rng.integers(0, 256, (N, K // 2), dtype=np.uint8),
                       rng.integers(0, 256, (N, K // 16), dtype=np.uint8), 1.0, N, K)
    x = mm.make_activations(M, K, seed=8)
    want = oracle.gemm_f4(x, w.payload, w.scales, 1.0)
    assert row_rel_l2(run(rt, x, w, V_UMMA), want) <= REL_L2_TOL


@pytest.mark.parametrize("gs", [1.0, 0.25, 3.0517578125e-05, 4.0530e-05, 7.0])
@pytest.mark.parametrize("variant,M", [(V_ROWWARP, 2), (V_STREAM, 2), (V_UMMA, 128)])
def test_global_scale(rt, oracle, gs, variant, M):
    check(rt, oracle, M, 512, 256, variant, seed=4, gs=gs)


def test_output_canaries(rt, oracle):
    """Nothing is written outside y[M][N]."""
    torch = rt.torch
    for (M, K, N, v) in [(3, 512, 40, V_STREAM), (5, 272, 33, V_ROWWARP), (130, 512, 264, V_UMMA)]:
        w = mm.make_weight(N, K, seed=1).to_device(rt.device)
        x = rt.to_device_bf16(mm.make_activations(M, K, seed=2))
        pad = 4096
        buf = torch.full((pad + M * N + pad,), 0x7B7B, dtype=torch.int16, device=rt.device)
        y = buf[pad:pad + M * N].view(torch.bfloat16).view(M, N)
        rt.gemm_f4(x, w, y, variant=v)
        assert (buf[:pad] == 0x7B7B).all() and (buf[pad + M * N:] == 0x7B7B).all()
        want = oracle.gemm_f4(mm.make_activations(M, K, seed=2), w.payload, w.scales, w.gs)
        assert row_rel_l2(rt.from_device_bf16(y), want) <= REL_L2_TOL


def test_error_statuses_on_device(rt):
    rt.lib.mm_log_set_level(-1)
    w = mm.make_weight(8, 256, seed=1).to_device(rt.device)
    x = rt.to_device_bf16(mm.make_activations(1, 256, seed=2))
    y = rt.torch.empty((1, 8), dtype=rt.torch.bfloat16, device=rt.device)
    d = rt.op_desc(x, w, y)
    d.n1 = 24
    kc = L.MmKcall(C.pointer(d), 1, None)
    assert rt.lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_SHAPE
    d.n1, d.b = 256, None
    assert rt.lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_STATE
    rt.lib.mm_log_set_level(1)


def test_qkv_routes_to_fp4_kernel(rt, oracle):
    w = mm.make_weight(512, 512, seed=1).to_device(rt.device)
    xb = mm.make_activations(2, 512, seed=2)
    x = rt.to_device_bf16(xb)
    y = rt.torch.empty((2, 512), dtype=rt.torch.bfloat16, device=rt.device)
    d = rt.op_desc(x, w, y, op=L.OP_QKV, note=b"qkv")
    kc = L.MmKcall(C.pointer(d), 1, None)
    assert rt.lib.mm_kx_invoke(C.byref(kc)) == L.MM_OK
    assert row_rel_l2(rt.from_device_bf16(y), oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL


# ---------------------------------------------------------------- engine / graph
def test_engine_graph_equals_direct_dispatch(rt, oracle):
    torch = rt.torch
    shapes = [(5120, 6144), (5120, 1024), (6144, 5120), (5120, 2048), (2048, 5120)]
    M = 4
    ws = [mm.make_weight(N, K, seed=i).to_device(rt.device) for i, (K, N) in enumerate(shapes)]
    xs = [rt.to_device_bf16(mm.make_activations(M, K, seed=50 + i)) for i, (K, N) in enumerate(shapes)]
    ys = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for (K, N) in shapes]
    eng = mm.LinearEngine(rt)
    for x, w, y in zip(xs, ws, ys):
        eng.add(x, w, y)
    eng.launch()                                           # direct dispatch
    rt.sync()
    direct = [rt.from_device_bf16(y).copy() for y in ys]
    for y in ys:
        y.zero_()
    torch.cuda.synchronize()
    eng.capture()
    for _ in range(2):
        eng.launch()
    rt.sync()
    assert rt.device_status() == 0
    for i, (y, d) in enumerate(zip(ys, direct)):
        assert np.array_equal(rt.from_device_bf16(y), d)
        want = oracle.gemm_f4(mm.make_activations(M, shapes[i][0], seed=50 + i), ws[i].payload,
                              ws[i].scales, ws[i].gs)
        assert row_rel_l2(d, want) <= REL_L2_TOL
    eng.close()


def test_engine_host_step(rt, oracle):
    """mm_lin_engine_launch_host: host activations in, graph replay, host outputs out."""
    torch = rt.torch
    shapes = [(2, 1024, 512), (5, 512, 1000), (1, 2048, 256)]
    ws = [mm.make_weight(N, K, seed=i).to_device(rt.device) for i, (M, K, N) in enumerate(shapes)]
    xb = [mm.make_activations(M, K, seed=70 + i) for i, (M, K, N) in enumerate(shapes)]
    xd = [torch.zeros((M, K), dtype=torch.bfloat16, device=rt.device) for (M, K, N) in shapes]
    yd = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for (M, K, N) in shapes]
    xh = [torch.from_numpy(b.view(np.int16)).view(torch.bfloat16).pin_memory() for b in xb]
    yh = [torch.zeros((M, N), dtype=torch.bfloat16).pin_memory() for (M, K, N) in shapes]
    eng = mm.LinearEngine(rt)
    for x, w, y in zip(xd, ws, yd):
        eng.add(x, w, y)
    for captured in (False, True):
        if captured:
            eng.capture()
        for t in yh:
            t.zero_()
        eng.launch_host(xh, [yh[0], None, yh[2]])          # None: output stays on the device
        for i in (0, 2):
            got = yh[i].view(torch.int16).numpy().view(np.uint16)
            assert row_rel_l2(got, oracle.gemm_f4(xb[i], ws[i].payload, ws[i].scales, ws[i].gs)) <= REL_L2_TOL
        assert not yh[1].view(torch.int16).numpy().any()
        assert row_rel_l2(rt.from_device_bf16(yd[1]),
                          oracle.gemm_f4(xb[1], ws[1].payload, ws[1].scales, ws[1].gs)) <= REL_L2_TOL
    eng.close()


@pytest.mark.parametrize("upload_kernel", [True, False])
@pytest.mark.parametrize("overlap", [False, True])
def test_engine_bound_host_step(rt, oracle, overlap, upload_kernel):
    """mm_lin_engine_bind_host + mm_lin_engine_step_bound: the uploads and downloads are nodes
    of the captured graph; refilling the same pinned buffers changes the next step's result."""
    torch = rt.torch
    shapes = [(2, 1024, 512), (16, 5120, 768), (5, 512, 1000), (1, 2048, 256)]
    ws = [mm.make_weight(N, K, seed=i).to_device(rt.device) for i, (M, K, N) in enumerate(shapes)]
    xd = [torch.zeros((M, K), dtype=torch.bfloat16, device=rt.device) for (M, K, N) in shapes]
    yd = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for (M, K, N) in shapes]
    xh = [torch.zeros((M, K), dtype=torch.bfloat16).pin_memory() for (M, K, N) in shapes]
    yh = [torch.zeros((M, N), dtype=torch.bfloat16).pin_memory() for (M, K, N) in shapes]
    eng = mm.LinearEngine(rt)
    eng.overlap(overlap)
    for x, w, y in zip(xd, ws, yd):
        eng.add(x, w, y)
    eng.upload_kernel(upload_kernel)                        # one gather kernel per group, or copy nodes
    eng.upload_group(3)
    eng.bind_host(xh, [yh[0], yh[1], None, yh[3]])          # None: output stays on the device
    eng.capture()
    with pytest.raises(mm.MimferError):                     # that graph already carries the copies
        eng.launch_host(xh, yh)
    for step in range(2):
        xb = [mm.make_activations(M, K, seed=90 + 10 * step + i) for i, (M, K, N) in enumerate(shapes)]
        for t, b in zip(xh, xb):
            t.copy_(torch.from_numpy(b.view(np.int16)).view(torch.bfloat16))
        for t in yh:
            t.zero_()
        eng.step_bound()
        for i in (0, 1, 3):
            got = yh[i].view(torch.int16).numpy().view(np.uint16)
            assert row_rel_l2(got, oracle.gemm_f4(xb[i], ws[i].payload, ws[i].scales, ws[i].gs)) <= REL_L2_TOL
        assert not yh[2].view(torch.int16).numpy().any()
        assert row_rel_l2(rt.from_device_bf16(yd[2]),
                          oracle.gemm_f4(xb[2], ws[2].payload, ws[2].scales, ws[2].gs)) <= REL_L2_TOL
    eng.close()


def test_host_buffer_call(rt, oracle):
    torch = rt.torch
    M, K, N = 4, 1024, 512
    w = mm.make_weight(N, K, seed=3).to_device(rt.device)
    xb = mm.make_activations(M, K, seed=4)
    x_host = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).pin_memory()
    y_host = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty((M, K), dtype=torch.bfloat16, device=rt.device)
    y_dev = torch.empty((M, N), dtype=torch.bfloat16, device=rt.device)
    rt.linear_host(x_host, x_dev, w, y_dev, y_host)
    got = y_host.view(torch.int16).numpy().view(np.uint16)
    assert row_rel_l2(got, oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL


# ---------------------------------------------------------------- failure detection
def test_bounded_wait_expires_and_device_stays_usable(rt, oracle):
    """A wait on a barrier that nothing completes gives up after its limit, the
    kernel returns, the launcher reports MM_ERR_TIMEOUT, and the next op is fine."""
    done = rt.torch.zeros(1, dtype=rt.torch.int32, device=rt.device)
    rt.torch.cuda.synchronize()
    rt.lib.mm_log_set_level(-1)
    st = rt.lib.mm_f4_wait_selftest(done.data_ptr())
    rt.lib.mm_log_set_level(1)
    assert st == L.MM_ERR_TIMEOUT
    assert int(done.item()) == 1
    assert rt.device_status() == 0                       # the launcher cleared the word
    check(rt, oracle, 4, 512, 256, None, seed=3)         # the context is healthy


def test_tp_barrier_signals_waits_and_gives_up(rt, oracle):
    """mm_f4_tp_barrier on one GPU, both flag blocks local: with the peer's arrival already
    written the kernel passes and leaves its own arrival in the peer's block; with no peer it
    gives up after its limit (about two seconds), raises the timeout bit, and the device stays usable."""
    import ctypes as C
    torch = rt.torch
    blocks = torch.zeros((2, 16), dtype=torch.int32, device=rt.device)
    ptrs = (C.c_void_p * 2)(blocks[0].data_ptr(), blocks[1].data_ptr())
    blocks[0, 1] = 1                                       # rank 1 "arrived" at epoch 1
    torch.cuda.synchronize()
    L.check(rt.lib.mm_f4_tp_barrier(ptrs, 2, 0, None), "mm_f4_tp_barrier")
    rt.sync()
    assert rt.device_status() == 0
    got = blocks.cpu().numpy()
    assert got[0, 0] == 1 and got[1, 0] == 1 and got[0, 8] == 1      # own slots and the epoch word
    # epoch 2: nobody signals for rank 1
    L.check(rt.lib.mm_f4_tp_barrier(ptrs, 2, 0, None), "mm_f4_tp_barrier")
    rt.sync()
    assert rt.device_status() == 1                         # MMB_DEV_TIMEOUT, cleared by the read
    assert blocks.cpu().numpy()[1, 0] == 2
    check(rt, oracle, 4, 512, 256, None, seed=3)           # the context is healthy
    assert rt.lib.mm_f4_tp_barrier(ptrs, 9, 0, None) == L.MM_ERR_RANGE
