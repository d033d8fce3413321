"""Launcher and engine behaviour that needs no GPU: argument checks come before
any CUDA call, the global-scale registry, descriptor validation."""
import ctypes as C

import pytest

from mimfer_b200 import _lib as L


def kcall(op=L.OP_GEMM_F4, a=1, b=1, c=1, d=1, M=1, K=256, N=8, e=1):
    desc = L.MmOpDesc()
    desc.op, desc.layer = op, -1
    desc.a, desc.b, desc.c, desc.d = a, b, c, d
    desc.n0, desc.n1, desc.n2 = M, K, N
    return L.MmKcall(C.pointer(desc), e, None), desc


def test_dispatcher_null_checks(lib):
    assert lib.mm_kx_invoke(None) == L.MM_ERR_STATE
    kc, _ = kcall(e=None)
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_STATE       # reference: kx.c:19-20
    kc = L.MmKcall(None, 1, None)
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_STATE


def test_dispatcher_routes_only_owned_opcodes(lib):
    lib.mm_log_set_level(-1)
    for op in range(19):
        owned = (L.OP_GEMM_F4, L.OP_QKV, L.OP_LMHEAD, L.OP_SILU_MUL, L.OP_ADD_RMSNORM, L.OP_NOP)
        assert lib.kx_cuda_oppref(op) == (1 if op in owned else 0)
    kc, _ = kcall(op=L.OP_NOP)
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_OK
    kc, _ = kcall(op=L.OP_GEMM_BF16)
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_UNSUPPORTED
    kc, _ = kcall(op=L.OP_QKV, d=None)
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_UNSUPPORTED  # bf16 qkv is not served
    kc, _ = kcall(op=L.OP_LMHEAD, d=None)
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_UNSUPPORTED  # nor a bf16 head
    kc, _ = kcall(op=L.OP_SILU_MUL, a=None)
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_STATE
    kc, _ = kcall(op=L.OP_ADD_RMSNORM, d=None)               # no gain tensor
    assert lib.mm_kx_invoke(C.byref(kc)) == L.MM_ERR_STATE
    lib.mm_log_set_level(1)


def test_gemm_f4_argument_errors_precede_cuda(lib):
    lib.mm_log_set_level(-1)
    kc, _ = kcall(K=24)
    assert lib.kx_op_gemm_f4(C.byref(kc)) == L.MM_ERR_SHAPE      # reference: cx.cu:365-366
    kc, _ = kcall(a=None)
    assert lib.kx_op_gemm_f4(C.byref(kc)) == L.MM_ERR_STATE
    # runtime not initialised on a CPU-only machine -> state error, never a crash
    kc, _ = kcall()
    assert lib.kx_op_gemm_f4(C.byref(kc)) in (L.MM_ERR_STATE, L.MM_ERR_CUDA)
    assert lib.mm_f4_linear(None, 1, 1, 1.0, 1, 1, 256, 8, None) == L.MM_ERR_STATE
    assert lib.mm_f4_linear(1, 1, 1, 1.0, 1, 0, 256, 8, None) == L.MM_ERR_SHAPE
    lib.mm_log_set_level(1)


def test_global_scale_registry(lib):
    lib.mm_f4_gscale_clear()
    assert lib.mm_f4_gscale_get(0x1000) == 1.0                   # unregistered = reference maths
    for i in range(1, 200):
        assert lib.mm_f4_gscale_set(0x1000 * i, 0.5 * i) == L.MM_OK
    for i in range(1, 200):
        assert lib.mm_f4_gscale_get(0x1000 * i) == 0.5 * i
    assert lib.mm_f4_gscale_set(0x1000, 3.0) == L.MM_OK and lib.mm_f4_gscale_get(0x1000) == 3.0
    lib.mm_log_set_level(-1)
    assert lib.mm_f4_gscale_set(None, 1.0) == L.MM_ERR_STATE
    assert lib.mm_f4_gscale_set(0x10, 0.0) == L.MM_ERR_RANGE
    assert lib.mm_f4_gscale_set(0x10, float("nan")) == L.MM_ERR_RANGE
    lib.mm_log_set_level(1)
    lib.mm_f4_gscale_clear()
    assert lib.mm_f4_gscale_get(0x1000) == 1.0


def test_engine_validates_descriptors(lib):
    lib.mm_log_set_level(-1)
    h = C.c_void_p()
    assert lib.mm_lin_engine_create(C.byref(h), 2) == L.MM_OK
    _, good = kcall()
    _, bad_k = kcall(K=24)
    _, bad_op = kcall(op=L.OP_GEMM_BF16)
    _, null = kcall(b=None)
    assert lib.mm_lin_engine_add(h, C.byref(bad_k)) == L.MM_ERR_SHAPE
    assert lib.mm_lin_engine_add(h, C.byref(bad_op)) == L.MM_ERR_UNSUPPORTED
    assert lib.mm_lin_engine_add(h, C.byref(null)) == L.MM_ERR_STATE
    assert lib.mm_lin_engine_add(h, C.byref(good)) == L.MM_OK
    assert lib.mm_lin_engine_add(h, C.byref(good)) == L.MM_OK
    assert lib.mm_lin_engine_add(h, C.byref(good)) == L.MM_ERR_CAPACITY
    assert lib.mm_lin_engine_n_ops(h) == 2
    lib.mm_lin_engine_destroy(h)
    lib.mm_log_set_level(1)


def test_engine_tensor_parallel_ops_validate_their_destinations(lib):
    """mm_lin_engine_add_tp: the op's own output is the first destination, the shard's
    columns fit the row pitch, at most eight aligned destinations; a refused op is not added."""
    lib.mm_log_set_level(-1)
    h = C.c_void_p()
    assert lib.mm_lin_engine_create(C.byref(h), 4) == L.MM_OK
    _, op = kcall(a=0x10000, b=0x20000, c=0x50000, d=0x30000, M=4, K=512, N=256)
    own, peer = op.c, 0x70000
    ptrs = (C.c_void_p * 2)(own, peer)
    assert lib.mm_lin_engine_add_tp(h, C.byref(op), ptrs, 2, 512, 256) == L.MM_OK
    assert lib.mm_lin_engine_add_tp(h, C.byref(op), ptrs, 2, 512, 264) == L.MM_ERR_SHAPE      # 264 + 256 > 512
    assert lib.mm_lin_engine_add_tp(h, C.byref(op), ptrs, 9, 4096, 0) == L.MM_ERR_RANGE
    assert lib.mm_lin_engine_add_tp(h, C.byref(op), ptrs, 0, 4096, 0) == L.MM_ERR_RANGE
    swapped = (C.c_void_p * 2)(peer, own)
    assert lib.mm_lin_engine_add_tp(h, C.byref(op), swapped, 2, 512, 0) == L.MM_ERR_STATE     # own copy first
    odd = (C.c_void_p * 2)(own, peer + 2)
    assert lib.mm_lin_engine_add_tp(h, C.byref(op), odd, 2, 512, 0) == L.MM_ERR_STATE
    _, silu = kcall(op=L.OP_SILU_MUL)
    assert lib.mm_lin_engine_add_tp(h, C.byref(silu), ptrs, 2, 512, 0) == L.MM_ERR_STATE
    assert lib.mm_lin_engine_n_ops(h) == 1
    lib.mm_lin_engine_destroy(h)
    lib.mm_log_set_level(1)


def test_runtime_refuses_without_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    import mimfer_b200
    with pytest.raises(RuntimeError):
        mimfer_b200.Runtime(0)
    assert lib.mm_cuda_stream_raw(0) is None and lib.mm_cuda_capturing() == 0


def test_tensor_parallel_entry_point_validates_arguments(lib):
    lib.mm_log_set_level(-1)
    ptrs = (C.c_void_p * 2)(0x1000, 0x2000)
    bad = (C.c_void_p * 2)(0x1000, 0x2008)              # peer copy not 16-byte aligned
    assert lib.mm_f4_linear_tp(1, 1, 1, 1.0, None, 2, 512, 0, 1, 256, 256, None) == L.MM_ERR_RANGE
    assert lib.mm_f4_linear_tp(1, 1, 1, 1.0, ptrs, 9, 512, 0, 1, 256, 256, None) == L.MM_ERR_RANGE
    assert lib.mm_f4_linear_tp(1, 1, 1, 1.0, bad, 2, 512, 0, 1, 256, 256, None) == L.MM_ERR_STATE
    assert lib.mm_f4_linear_tp(1, 1, 1, 1.0, ptrs, 2, 512, 384, 1, 256, 256, None) == L.MM_ERR_SHAPE
    assert lib.mm_f4_linear_tp(1, 1, 1, 1.0, ptrs, 2, 512, 0, 1, 24, 256, None) == L.MM_ERR_SHAPE
    lib.mm_log_set_level(1)


def _desc(op, a, b, c, d, n0, n1, n2):
    desc = L.MmOpDesc()
    desc.op, desc.layer = op, -1
    desc.a, desc.b, desc.c, desc.d = a, b, c, d
    desc.n0, desc.n1, desc.n2 = n0, n1, n2
    return desc


def test_engine_mlp_fusion_is_a_host_decision(lib):
    """The planner's gate GEMM, up GEMM, SILU_MUL sequence (reference: src/plan/plan.c:223-247)
    collapses to one op only when asked to and when the fused kernel can take it."""
    X, G, U, Y = 0x10000, 0x20000, 0x30000, 0x40000
    PG, SG, PU, SU = 0x100000, 0x200000, 0x300000, 0x400000       # both tensors gate-first
    M, K, inter = 4, 512, 256

    def build(fuse, up_scale=SU, k=K, up_first=False, other_x=False):
        h = C.c_void_p()
        assert lib.mm_lin_engine_create(C.byref(h), 8) == L.MM_OK
        assert lib.mm_lin_engine_fuse_mlp(h, fuse) == L.MM_OK
        gate = _desc(L.OP_GEMM_F4, X, PG, G, SG, M, k, inter)
        up = _desc(L.OP_GEMM_F4, X + (0x1000 if other_x else 0), PU, U, up_scale, M, k, inter)
        for d in ((up, gate) if up_first else (gate, up)):
            assert lib.mm_lin_engine_add(h, C.byref(d)) == L.MM_OK
        silu = _desc(L.OP_SILU_MUL, G, U, Y, None, M, inter, 0)
        assert lib.mm_lin_engine_add(h, C.byref(silu)) == L.MM_OK
        n = lib.mm_lin_engine_n_ops(h)
        lib.mm_lin_engine_destroy(h)
        return n

    assert build(0) == 3                       # off by default
    assert build(1) == 1
    assert build(1, up_first=True) == 1        # emission order does not matter
    assert build(1, up_scale=0x150000) == 3    # scale tensors in the opposite address order
    assert build(1, k=272) == 3                # K % 256 != 0: fallback kernel, no fused form
    assert build(1, other_x=True) == 3         # different activations
    # a SILU_MUL with nothing to fuse is kept as its own op; bad operands are refused
    h = C.c_void_p()
    assert lib.mm_lin_engine_create(C.byref(h), 4) == L.MM_OK
    lib.mm_lin_engine_fuse_mlp(h, 1)
    assert lib.mm_lin_engine_add(h, C.byref(_desc(L.OP_SILU_MUL, G, U, Y, None, M, inter, 0))) == L.MM_OK
    lib.mm_log_set_level(-1)
    assert lib.mm_lin_engine_add(h, C.byref(_desc(L.OP_SILU_MUL, G, None, Y, None, M, inter, 0))) == L.MM_ERR_STATE
    assert lib.mm_lin_engine_add(h, C.byref(_desc(L.OP_SILU_MUL, G, U, Y, None, 0, inter, 0))) == L.MM_ERR_SHAPE
    lib.mm_log_set_level(1)
    assert lib.mm_lin_engine_n_ops(h) == 1
    lib.mm_lin_engine_destroy(h)


def test_misaligned_operands_are_refused_before_any_launch(lib):
    """Every form of the op needs 16-byte aligned x, payload, scales and output (all
    kernels load 16-byte vectors): a sliced activation view two bytes off is
    MM_ERR_SHAPE, on the tensor-parallel entry point too, and nothing is launched."""
    lib.mm_log_set_level(-1)
    before = lib.mm_f4_launch_count(0)
    ptrs = (C.c_void_p * 2)(0x1000, 0x2000)
    assert lib.mm_f4_linear_tp(0x10002, 0x20000, 0x30000, 1.0, ptrs, 2, 512, 0, 1, 256, 256, None) == L.MM_ERR_SHAPE
    assert lib.mm_f4_linear_tp(0x10000, 0x20008, 0x30000, 1.0, ptrs, 2, 512, 0, 1, 256, 256, None) == L.MM_ERR_SHAPE
    assert lib.mm_f4_linear_tp(0x10000, 0x20000, 0x30004, 1.0, ptrs, 2, 512, 0, 1, 256, 256, None) == L.MM_ERR_SHAPE
    assert lib.mm_f4_linear(0x10002, 0x20000, 0x30000, 1.0, 0x40000, 1, 256, 256, None) == L.MM_ERR_SHAPE
    assert lib.mm_f4_launch_count(0) == before
    lib.mm_log_set_level(1)


def test_global_scale_entries_can_be_taken_back(lib):
    lib.mm_f4_gscale_clear()
    room = lib.mm_f4_gscale_room()
    assert room >= 4096                      # at least one registration per tensor the loader admits
    for i in range(1, 50):
        assert lib.mm_f4_gscale_set(0x2000 * i, 2.0 * i) == L.MM_OK
    lib.mm_f4_gscale_unset(0x2000 * 7)
    assert lib.mm_f4_gscale_get(0x2000 * 7) == 1.0
    assert lib.mm_f4_gscale_get(0x2000 * 8) == 16.0      # probing runs past the emptied slot
    assert lib.mm_f4_gscale_set(0x2000 * 7, 5.0) == L.MM_OK and lib.mm_f4_gscale_get(0x2000 * 7) == 5.0
    assert lib.mm_f4_gscale_room() == room - 49
    lib.mm_f4_gscale_clear()


def test_tensor_parallel_push_validates_arguments(lib):
    """mm_f4_tp_push: at most eight aligned copies, the slice inside the row pitch, 16-byte rows."""
    lib.mm_log_set_level(-1)
    ptrs = (C.c_void_p * 2)(0x1000, 0x2000)
    bad = (C.c_void_p * 2)(0x1000, 0x2008)
    assert lib.mm_f4_tp_push(None, 2, 512, 0, 256, 0, 4) == L.MM_ERR_RANGE
    assert lib.mm_f4_tp_push(ptrs, 9, 512, 0, 256, 0, 4) == L.MM_ERR_RANGE
    assert lib.mm_f4_tp_push(ptrs, 2, 512, 384, 256, 0, 4) == L.MM_ERR_SHAPE      # 384 + 256 > 512
    assert lib.mm_f4_tp_push(ptrs, 2, 512, 0, 0, 0, 4) == L.MM_ERR_SHAPE
    assert lib.mm_f4_tp_push(ptrs, 2, 512, 0, 256, 0, 0) == L.MM_ERR_SHAPE
    assert lib.mm_f4_tp_push(ptrs, 2, 512, 4, 256, 0, 4) == L.MM_ERR_SHAPE        # rows of the slice not 16-byte aligned
    assert lib.mm_f4_tp_push(ptrs, 2, 516, 0, 256, 0, 4) == L.MM_ERR_SHAPE
    assert lib.mm_f4_tp_push(bad, 2, 512, 0, 256, 0, 4) == L.MM_ERR_STATE
    lib.mm_log_set_level(1)


def test_tune_keys_of_the_tensor_parallel_forms(lib):
    """mm_f4_tune returns the previous value: copy streams per peer (key 11, 0 = automatic) and
    the spread of a tensor-parallel prefill launch's first wave in percent (key 12, default 100,
    capped at 400); an unknown key is refused."""
    assert lib.mm_f4_tune(11, 4) == 0
    assert lib.mm_f4_tune(11, 0) == 4
    assert lib.mm_f4_tune(12, 0) == 100
    assert lib.mm_f4_tune(12, 1000) == 0
    assert lib.mm_f4_tune(12, 100) == 400
    assert lib.mm_f4_tune(99, 1) == -1
