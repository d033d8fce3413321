"""Dependency-aware launch order of the op-list engine (mm_lin_engine_overlap):
independent ops run ahead of their predecessors, dependent ones wait; results
are those of the serial order.  This is the engine with group launches off; the
run-ahead form of the streaming kernel is tested with that kernel selected, the
plane cache with the block-scaled one."""
import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import _lib as L
from conftest import REL_L2_TOL, row_rel_l2

pytestmark = pytest.mark.gpu


def _dev(rt, w):
    return mm.NvFp4Weight(w.payload, w.scales, w.gs, w.N, w.K).to_device(rt.device)


def test_chain_with_dependent_and_independent_ops(stream_kernel, oracle):
    """q, k, v read the same x (independent); o reads q's output (dependent);
    two split-K ops in a row take different workspace regions; a third reuse of a
    buffer forces a wait."""
    rt = stream_kernel
    torch = rt.torch
    M, K = 4, 1024
    wq, wk, wv = (mm.make_weight(n, K, seed=s) for n, s in ((1024, 1), (256, 2), (256, 3)))
    wo = mm.make_weight(512, 1024, seed=4)
    wd = mm.make_weight(256, 4096, seed=5)                     # few tiles, long K: split-K
    dq, dk, dv, do, dd = (_dev(rt, w) for w in (wq, wk, wv, wo, wd))
    xb = mm.make_activations(M, K, seed=7)
    xdb = mm.make_activations(M, 4096, seed=8)
    x, xd = rt.to_device_bf16(xb), rt.to_device_bf16(xdb)
    bf = dict(dtype=torch.bfloat16, device=rt.device)
    yq, yk, yv = torch.zeros((M, 1024), **bf), torch.zeros((M, 256), **bf), torch.zeros((M, 256), **bf)
    yo, yd1, yd2 = torch.zeros((M, 512), **bf), torch.zeros((M, 256), **bf), torch.zeros((M, 256), **bf)

    def build(overlap):
        eng = mm.LinearEngine(rt)
        eng.overlap(overlap)
        eng.group(False)
        eng.add(x, dq, yq)          # 0 first op: waits
        eng.add(x, dk, yk)          # 1 independent
        eng.add(x, dv, yv)          # 2 independent
        eng.add(yq, do, yo)         # 3 reads op 0's output: waits
        eng.add(xd, dd, yd1)        # 4 independent, split-K region 0
        eng.add(xd, dd, yd2)        # 5 independent, split-K region 1
        eng.add(xd, dd, yd1)        # 6 writes op 4's output again: waits
        return eng

    assert mm.select_plan(M, 4096, 256, ws_bytes=16 << 20).split_k > 1
    ref_q = oracle.gemm_f4(xb, wq.payload, wq.scales, wq.gs)
    want = {
        "q": ref_q, "k": oracle.gemm_f4(xb, wk.payload, wk.scales, wk.gs),
        "v": oracle.gemm_f4(xb, wv.payload, wv.scales, wv.gs),
        "d": oracle.gemm_f4(xdb, wd.payload, wd.scales, wd.gs),
    }
    outs = {}
    for overlap in (False, True):
        eng = build(overlap)
        for captured in (False, True):
            if captured:
                eng.capture()
                assert eng.n_independent() == (4 if overlap else 0)
            for t in (yq, yk, yv, yo, yd1, yd2):
                t.zero_()
            for _ in range(3 if captured else 1):
                eng.launch()
            rt.sync()
            assert rt.device_status() == 0
            got = {n: rt.from_device_bf16(t) for n, t in
                   (("q", yq), ("k", yk), ("v", yv), ("o", yo), ("d1", yd1), ("d2", yd2))}
            for n in ("q", "k", "v"):
                assert row_rel_l2(got[n], want[n]) <= REL_L2_TOL
            assert row_rel_l2(got["d1"], want["d"]) <= REL_L2_TOL
            assert np.array_equal(got["d1"], got["d2"])
            # o consumed the q this run produced
            assert row_rel_l2(got["o"], oracle.gemm_f4(got["q"], wo.payload, wo.scales, wo.gs)) <= REL_L2_TOL
            outs[(overlap, captured)] = got
        eng.close()
    for n in outs[(False, True)]:                      # bitwise the serial result
        assert np.array_equal(outs[(False, True)][n], outs[(True, True)][n]), n


def test_many_independent_split_ops_stay_correct(stream_kernel, oracle):
    """More split-K ops in a row than workspace regions, replayed many times."""
    rt = stream_kernel
    torch = rt.torch
    M, K, N = 8, 8192, 512
    ws = [mm.make_weight(N, K, seed=20 + i) for i in range(6)]
    ds = [_dev(rt, w) for w in ws]
    xb = mm.make_activations(M, K, seed=9)
    x = rt.to_device_bf16(xb)
    ys = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for _ in ws]
    eng = mm.LinearEngine(rt)
    eng.overlap(True)
    eng.group(False)
    for d, y in zip(ds, ys):
        eng.add(x, d, y)
    eng.capture()
    assert 1 <= eng.n_independent() <= 5
    for _ in range(20):
        eng.launch()
    rt.sync()
    assert rt.device_status() == 0
    for w, y in zip(ws, ys):
        assert row_rel_l2(rt.from_device_bf16(y), oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL
    eng.close()


def test_run_ahead_ops_on_shallow_split(stream_kernel, oracle):
    """Overlap level 2: ops that run ahead take fewer K slices.  Same answer within the
    op's tolerance, the same bits on every replay, and the first op (which waits) keeps
    the bits of the serial order."""
    rt = stream_kernel
    torch = rt.torch
    M, K, N = 4, 17408, 2048                            # 8 row tiles: 17 slices alone, 8 when running ahead
    ws = [mm.make_weight(N, K, seed=30 + i) for i in range(3)]
    ds = [_dev(rt, w) for w in ws]
    xb = mm.make_activations(M, K, seed=11)
    x = rt.to_device_bf16(xb)
    ys = [torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device) for _ in ws]
    runs = {}
    for level in (1, 2):
        eng = mm.LinearEngine(rt)
        eng.overlap(level)
        eng.group(False)
        for d, y in zip(ds, ys):
            eng.add(x, d, y)
        eng.capture()
        assert eng.n_independent() == 2
        got = []
        for rep in range(2):
            for y in ys:
                y.zero_()
            eng.launch()
            rt.sync()
            assert rt.device_status() == 0
            got.append([rt.from_device_bf16(y) for y in ys])
        eng.close()
        for a, b in zip(*got):
            assert np.array_equal(a, b)                 # run to run
        for w, y in zip(ws, got[0]):
            assert row_rel_l2(y, oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL
        runs[level] = got[0]
    assert np.array_equal(runs[1][0], runs[2][0])       # the op that waits is planned as before


def test_plane_cache_with_the_block_scaled_kernel(rt, oracle):
    """Overlap mode without group launches: activations that no op of the list writes are
    turned into digit planes once, ahead of the ops; q, k and v share one set, the op that
    reads q's output slices for itself."""
    torch = rt.torch
    M, K = 4, 1024
    wq, wk, wv = (mm.make_weight(n, K, seed=s) for n, s in ((1024, 1), (256, 2), (256, 3)))
    wo = mm.make_weight(512, 1024, seed=4)
    dq, dk, dv, do = (_dev(rt, w) for w in (wq, wk, wv, wo))
    xb = mm.make_activations(M, K, seed=7)
    x = rt.to_device_bf16(xb)
    bf = dict(dtype=torch.bfloat16, device=rt.device)
    yq, yk, yv, yo = (torch.zeros((M, n), **bf) for n in (1024, 256, 256, 512))
    eng = mm.LinearEngine(rt)
    eng.overlap(2)
    eng.group(False)
    for a, w, y in ((x, dq, yq), (x, dk, yk), (x, dv, yv), (yq, do, yo)):
        eng.add(a, w, y)
    eng.capture()
    assert rt.lib.mm_lin_engine_n_sliced_ahead(eng.h) == 1
    for _ in range(3):
        eng.launch()
    rt.sync()
    assert rt.device_status() == 0
    for w, y in ((wq, yq), (wk, yk), (wv, yv)):
        assert row_rel_l2(rt.from_device_bf16(y), oracle.gemm_f4(xb, w.payload, w.scales, w.gs)) <= REL_L2_TOL
    q = rt.from_device_bf16(yq)
    assert row_rel_l2(rt.from_device_bf16(yo), oracle.gemm_f4(q, wo.payload, wo.scales, wo.gs)) <= REL_L2_TOL
    eng.close()
