"""Parity at the benchmark's full sizes, through the C-ABI, on sampled rows and column
windows of the CPU oracle (the whole output where the oracle takes seconds).

Shapes: the decode sweep (gate+up 5120 -> 34816 and down 17408 -> 5120 at every
M of {1, 2, 4, 8, 16}), the fused gate/up pair at full size, the prefill chunk on
every projection, the LM head (5120 -> 151936), and the N-shards the
tensor-parallel form gives each rank at 2, 4 and 8 ranks (run here rank after rank
on one GPU, every rank's kernel storing its slice into two full-width outputs)."""
import ctypes as C

import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import V_MX, V_UMMA, _lib as L
from conftest import REL_L2_TOL, row_rel_l2

pytestmark = pytest.mark.gpu

SHAPES = {"gate_up": (5120, 34816), "down": (17408, 5120), "q": (5120, 6144), "k": (5120, 1024),
          "v": (5120, 1024), "o": (6144, 5120), "lm_head": (5120, 151936)}
_weights = {}


def weight(rt, name):
    """seed-0 N(0, 0.02) weight of a benchmark shape, packed once per session and resident."""
    if name not in _weights:
        K, N = SHAPES[name]
        _weights[name] = mm.make_weight(N, K, seed=0, std=0.02).to_device(rt.device)
    return _weights[name]


def windows(N, width=256):
    """column windows of the output: both ends, tile boundaries of 236/240/256-row tiles, the middle"""
    starts = {0, 236 - 8, 256 - 8, N // 2 - width // 2, (N // 3) // 8 * 8, N - width}
    return sorted((max(0, min(s, N - width)), max(0, min(s, N - width)) + min(width, N)) for s in starts)


def check_windows(oracle, xb, w, y, rows=None, width=256):
    for (a, b) in windows(w.N, width):
        want = oracle.gemm_f4(xb, w.payload, w.scales, w.gs, rows=rows, n_begin=a, n_end=b)
        got = (y if rows is None else y[rows])[:, a:b]
        err = row_rel_l2(got, want)
        assert err <= REL_L2_TOL, f"columns [{a}, {b}): rel L2 {err}"


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("name", ["gate_up", "down"])
def test_decode_sweep_shapes(rt, oracle, name, M):
    w = weight(rt, name)
    K, N = SHAPES[name]
    assert mm.select_plan(M, K, N, ws_bytes=rt.lib.mm_f4_workspace_bytes() // 8).variant == V_MX
    xb = mm.make_activations(M, K, seed=1)
    y = rt.from_device_bf16(rt.gemm_f4(rt.to_device_bf16(xb), w))
    assert rt.device_status() == 0
    if name == "down":                                   # 5120 outputs: the whole result
        assert row_rel_l2(y, oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL
    else:
        check_windows(oracle, xb, w, y)


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_gate_up_pair_full_size_every_m(rt, oracle, M):
    """The fused gate/up kernel on 2 x 17408 rows at every M of the decode sweep, on column
    windows of the oracle's three ops."""
    K, inter = 5120, 17408
    full = weight(rt, "gate_up")
    host = mm.NvFp4Weight(full.payload, full.scales, full.gs, full.N, full.K)
    wg, wu = host.rows(0, inter), host.rows(inter, 2 * inter)
    keep = mm.place_weights([wg, wu], rt.device)
    xb = mm.make_activations(M, K, seed=1)
    y = rt.torch.empty((M, inter), dtype=rt.torch.bfloat16, device=rt.device)
    rt.mlp_gate_up_async(rt.to_device_bf16(xb), wg, wu, y)
    rt.sync()
    assert rt.device_status() == 0
    got = rt.from_device_bf16(y)
    for (a, b) in windows(inter, 128):
        g = oracle.gemm_f4(xb, wg.payload, wg.scales, wg.gs, n_begin=a, n_end=b)
        u = oracle.gemm_f4(xb, wu.payload, wu.scales, wu.gs, n_begin=a, n_end=b)
        assert row_rel_l2(got[:, a:b], oracle.silu_mul(g, u)) <= 2 * REL_L2_TOL, (a, b)
    del keep


@pytest.mark.parametrize("M", [512, 2048])
@pytest.mark.parametrize("name", ["q", "k", "v", "o", "down", "gate_up"])
def test_prefill_chunk_shapes(rt, oracle, name, M):
    w = weight(rt, name)
    K, N = SHAPES[name]
    assert mm.select_plan(M, K, N).variant == V_UMMA
    xb = mm.make_activations(M, K, seed=1)
    y = rt.from_device_bf16(rt.gemm_f4(rt.to_device_bf16(xb), w))
    assert rt.device_status() == 0
    rows = sorted({0, 1, 127, 128, 255, 256, M // 2 + 3, M - 129, M - 1})
    check_windows(oracle, xb, w, y, rows=rows, width=256 if N > 1024 else 1024)


def test_prefill_8192_gate_up_sampled(rt, oracle):
    w = weight(rt, "gate_up")
    M, K = 8192, 5120
    xb = mm.make_activations(M, K, seed=1)
    y = rt.from_device_bf16(rt.gemm_f4(rt.to_device_bf16(xb), w))
    assert rt.device_status() == 0
    check_windows(oracle, xb, w, y, rows=[0, 255, 256, 4095, 4096, 8191])


@pytest.mark.parametrize("M", [32, 8192])
def test_lm_head(rt, oracle, M):
    w = weight(rt, "lm_head")
    K, N = SHAPES["lm_head"]
    xb = mm.make_activations(M, K, seed=1)
    y = rt.from_device_bf16(rt.gemm_f4(rt.to_device_bf16(xb), w))
    assert rt.device_status() == 0
    rows = None if M <= 32 else [0, 129, 4097, 8191]
    check_windows(oracle, xb, w, y, rows=rows)


@pytest.mark.parametrize("name,world,M", [("gate_up", 2, 32), ("gate_up", 4, 32), ("gate_up", 8, 32),
                                          ("lm_head", 2, 32), ("lm_head", 4, 32), ("lm_head", 8, 32),
                                          ("gate_up", 8, 8192), ("lm_head", 8, 2048)])
def test_tensor_parallel_shards_on_one_gpu(rt, oracle, name, world, M):
    """mm_f4_linear_tp on every rank's shard in turn, each call storing its columns into two
    full-width outputs (the kernel epilogue's store loop over destinations, leading dimension
    and column offset as on `world` GPUs).  Both outputs must hold the full result."""
    torch = rt.torch
    w = weight(rt, name)
    K, N = SHAPES[name]
    ns = N // world
    assert ns * world == N and ns % 8 == 0
    xb = mm.make_activations(M, K, seed=1)
    x = rt.to_device_bf16(xb)
    outs = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for _ in range(2)]
    ptrs = (C.c_void_p * 2)(outs[0].data_ptr(), outs[1].data_ptr())
    torch.cuda.synchronize()                  # the zero fills ran on another stream than the ops
    for r in range(world):
        pay = w.dev_payload[r * ns:(r + 1) * ns]
        sc = w.dev_scales[r * ns:(r + 1) * ns]
        L.check(rt.lib.mm_f4_linear_tp(x.data_ptr(), pay.data_ptr(), sc.data_ptr(), w.gs, ptrs, 2, N, r * ns,
                                       M, K, ns, None), "mm_f4_linear_tp")
    rt.sync()
    assert rt.device_status() == 0
    y0, y1 = rt.from_device_bf16(outs[0]), rt.from_device_bf16(outs[1])
    assert np.array_equal(y0, y1)
    rows = None if M <= 32 else [0, 255, M // 2, M - 1]
    for r in sorted({0, world // 2, world - 1}):          # windows inside a shard and across its edges
        for (a, b) in ((r * ns, r * ns + 256), ((r + 1) * ns - 256, (r + 1) * ns),
                       (max(0, r * ns - 128), max(0, r * ns - 128) + 256)):
            want = oracle.gemm_f4(xb, w.payload, w.scales, w.gs, rows=rows, n_begin=a, n_end=b)
            got = (y0 if rows is None else y0[rows])[:, a:b]
            assert row_rel_l2(got, want) <= REL_L2_TOL, (r, a, b)


def test_push_of_row_chunks_on_one_gpu(rt, oracle):
    """The copy engines' form of the exchange with both "ranks" on one GPU: rank 1 of 2 runs its
    shard chunk of rows by chunk of rows into its own full-width output (mm_f4_linear_tp with
    one destination) and pushes every chunk to the other output (mm_f4_tp_push).  After the join
    the other output holds the shard's columns and nothing else."""
    from mimfer_b200.tp import push_chunks
    torch = rt.torch
    w = weight(rt, "gate_up")
    K, N = SHAPES["gate_up"]
    M, world, r = 1280, 2, 1
    ns = N // world
    xb = mm.make_activations(M, K, seed=1)
    x = rt.to_device_bf16(xb)
    outs = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for _ in range(2)]
    ptrs = (C.c_void_p * 2)(outs[0].data_ptr(), outs[1].data_ptr())
    own = (C.c_void_p * 1)()
    torch.cuda.synchronize()
    pay, sc = w.dev_payload[r * ns:(r + 1) * ns], w.dev_scales[r * ns:(r + 1) * ns]
    for r0, rows in push_chunks(M, 512):
        own[0] = outs[0].data_ptr() + r0 * N * 2
        L.check(rt.lib.mm_f4_linear_tp(x.data_ptr() + r0 * K * 2, pay.data_ptr(), sc.data_ptr(), w.gs, own, 1,
                                       N, r * ns, rows, K, ns, None), "mm_f4_linear_tp")
        L.check(rt.lib.mm_f4_tp_push(ptrs, 2, N, r * ns, ns, r0, rows), "mm_f4_tp_push")
    L.check(rt.lib.mm_f4_tp_push_join(), "mm_f4_tp_push_join")
    rt.sync()
    assert rt.device_status() == 0
    y0, y1 = rt.from_device_bf16(outs[0]), rt.from_device_bf16(outs[1])
    assert np.array_equal(y0, y1)
    assert not y1[:, :r * ns].any()                        # the other rank's columns stay untouched
    rows = [0, 255, 511, 512, 1023, 1024, M - 1]           # both sides of every chunk edge
    for (a, b) in ((r * ns, r * ns + 256), (N - 256, N)):
        want = oracle.gemm_f4(xb, w.payload, w.scales, w.gs, rows=rows, n_begin=a, n_end=b)
        assert row_rel_l2(y1[rows][:, a:b], want) <= REL_L2_TOL, (a, b)


@pytest.mark.parametrize("world,r", [(8, 3), (4, 1)])
def test_decode_sweep_shards_as_one_group_launch(rt, oracle, world, r):
    """The bench's tensor-parallel decode sweep as rank r of `world` runs it: the ten ops (gate+up
    and down at M = 1..16), each op's r-th N-shard, added with mm_lin_engine_add_tp and launched as
    one group whose epilogue stores into two full-width outputs.  Both must hold the shard's
    columns - against the oracle on windows at the shard's edges - and nothing else."""
    torch = rt.torch
    eng = mm.LinearEngine(rt, max_ops=12)
    ops, keep = [], []
    try:
        for name in ("gate_up", "down"):
            w = weight(rt, name)
            K, N = SHAPES[name]
            ns = N // world
            assert ns * world == N and ns % 8 == 0
            host = mm.NvFp4Weight(w.payload, w.scales, w.gs, w.N, w.K)
            shard = host.rows(r * ns, (r + 1) * ns).to_device(rt.device)
            for M in (1, 2, 4, 8, 16):
                xb = mm.make_activations(M, K, seed=10 + M)
                x = rt.to_device_bf16(xb)
                outs = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for _ in range(2)]
                ptrs = (C.c_void_p * 2)(outs[0].data_ptr(), outs[1].data_ptr())
                keep.append((x, ptrs, shard))
                eng.add_tp(x, shard, outs[0], ptrs, 2, r * ns)
                ops.append((name, M, xb, outs, ns))
        torch.cuda.synchronize()
        eng.capture()
        for _ in range(2):
            eng.launch()
        rt.sync()
        assert rt.device_status() == 0 and eng.n_group_launches() >= 1
        for name, M, xb, outs, ns in ops:
            w = weight(rt, name)
            a, b = rt.from_device_bf16(outs[0]), rt.from_device_bf16(outs[1])
            assert np.array_equal(a, b), (name, M)
            assert not a[:, :r * ns].any() and not a[:, (r + 1) * ns:].any(), (name, M)
            width = min(256, ns)
            for lo in (r * ns, (r + 1) * ns - width):
                want = oracle.gemm_f4(xb, w.payload, w.scales, w.gs, n_begin=lo, n_end=lo + width)
                assert row_rel_l2(a[:, lo:lo + width], want) <= REL_L2_TOL, (name, M, lo)
    finally:
        eng.close()
