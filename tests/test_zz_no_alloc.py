"""mm_f4_linear_static_ws: the decode op with its split-K scratch built into
the library, for callers that may not allocate device memory (start-up-only
allocation policies, serving loops that must stay off the allocator).

It must agree with the regular entry point, which is given a caller-owned
workspace, twice in a row (the built-in array keeps the previous call's
contents).  Collected last so that a run stopping at the first failure has
already run every other test; also passes alone in a fresh process."""
import ctypes as C

import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import _lib as L
from conftest import REL_L2_TOL, row_rel_l2

pytestmark = pytest.mark.gpu

STATIC_WS_BYTES = 16384 + (4 << 20)


def both_ways(rt, M, K, N, seed):
    torch = rt.torch
    w = mm.make_weight(N, K, seed=seed).to_device(rt.device)
    xb = mm.make_activations(M, K, seed=seed + 1)
    x = rt.to_device_bf16(xb)
    y_ref = torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device)
    rt.linear_async(x, w, y_ref)                       # existing entry point, caller's workspace
    rt.sync()
    want = rt.from_device_bf16(y_ref)
    stream = rt.stream_ptr()
    outs = []
    for _ in range(2):                                 # two calls in a row share the array
        y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=rt.device)
        torch.cuda.synchronize()
        st = rt.lib.mm_f4_linear_static_ws(x.data_ptr(), w.dev_payload.data_ptr(), w.dev_scales.data_ptr(),
                                           w.gs, y.data_ptr(), M, K, N, stream)
        assert st == L.MM_OK
        flags = C.c_uint(99)
        assert rt.lib.mm_f4_device_status_on(stream, C.byref(flags)) == L.MM_OK     # the caller's own stream
        assert flags.value == 0
        outs.append(rt.from_device_bf16(y))
    return want, outs, (xb, w)


@pytest.mark.parametrize("M,K,N", [(16, 17408, 5120), (1, 5120, 5120), (4, 5120, 34816), (32, 2048, 1000)])
def test_static_workspace_matches_regular_entry_point_and_oracle(rt, oracle, M, K, N):
    plan = mm.select_plan(M, K, N, ws_bytes=STATIC_WS_BYTES, variant=L.V_STREAM)
    want, outs, (xb, w) = both_ways(rt, M, K, N, seed=M + N)
    n_end = min(N, 2048)                                # the oracle on the first 2048 output features
    truth = oracle.gemm_f4(xb, w.payload, w.scales, w.gs, n_end=n_end)
    for got in outs:
        assert row_rel_l2(got, want) <= REL_L2_TOL
        assert row_rel_l2(got[:, :n_end], truth) <= REL_L2_TOL
    if plan.split_k > 1:                               # scratch really was exercised
        assert plan.ws_needed <= STATIC_WS_BYTES
    assert np.array_equal(outs[0], outs[1])


def test_static_workspace_rejects_what_it_cannot_hold(rt):
    torch = rt.torch
    rt.lib.mm_log_set_level(-1)
    try:
        # split-K scratch beyond the built-in 4 MiB
        M, K, N = 32, 17408, 17408
        big = mm.select_plan(M, K, N, ws_bytes=1 << 40, variant=L.V_STREAM)
        assert big.ws_needed > STATIC_WS_BYTES
        buf = torch.zeros(N * K // 2 + 256, dtype=torch.uint8, device=rt.device)
        x = torch.zeros((M, K), dtype=torch.bfloat16, device=rt.device)
        y = torch.zeros((M, N), dtype=torch.bfloat16, device=rt.device)
        st = rt.lib.mm_f4_linear_static_ws(x.data_ptr(), buf.data_ptr(), buf.data_ptr(), 1.0, y.data_ptr(),
                                           M, K, N, rt.stream_ptr())
        assert st == L.MM_ERR_CAPACITY
        # shapes the decode kernel does not take
        assert rt.lib.mm_f4_linear_static_ws(x.data_ptr(), buf.data_ptr(), buf.data_ptr(), 1.0, y.data_ptr(),
                                             64, 512, 64, rt.stream_ptr()) == L.MM_ERR_UNSUPPORTED
        assert rt.lib.mm_f4_linear_static_ws(x.data_ptr(), buf.data_ptr(), buf.data_ptr(), 1.0, y.data_ptr(),
                                             4, 48, 64, rt.stream_ptr()) == L.MM_ERR_UNSUPPORTED
        assert rt.lib.mm_f4_linear_static_ws(None, buf.data_ptr(), buf.data_ptr(), 1.0, y.data_ptr(),
                                             4, 512, 64, rt.stream_ptr()) == L.MM_ERR_STATE
        assert rt.lib.mm_f4_linear_static_ws(x.data_ptr(), buf.data_ptr(), buf.data_ptr(), 1.0, y.data_ptr(),
                                             4, 24, 64, rt.stream_ptr()) == L.MM_ERR_SHAPE
    finally:
        rt.lib.mm_log_set_level(1)
    rt.sync()
    assert rt.device_status() == 0
