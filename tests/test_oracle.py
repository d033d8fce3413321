"""The CPU oracle against the reference: golden fixtures generated from the
reference's own kernel (tests/golden/make_golden.py) and, when the compiled
reference is present, a live comparison."""
import glob
import os

import numpy as np
import pytest

import mimfer_b200 as mm
from conftest import GOLDEN, bf16_bits_to_f32, fnv1a64

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)


def test_e2m1_values(oracle):
    got = np.array([oracle.lib.orc_e2m1_decode(n) for n in range(16)], np.float32)
    assert np.array_equal(got, E2M1)
    assert np.signbit(got[8])


def test_e4m3_special_codes(oracle):
    d = oracle.lib.orc_e4m3_decode
    assert d(0x7F) == 0.0 and d(0xFF) == 0.0 and not np.signbit(np.float32(d(0xFF)))
    assert d(0x7E) == 448.0 and d(0xFE) == -448.0
    assert d(0x01) == 2.0 ** -9 and d(0x08) == 2.0 ** -6 and d(0x38) == 1.0
    vals = [d(b) for b in range(0x7F)]
    assert all(a < b for a, b in zip(vals, vals[1:]))          # monotone over positive codes


def test_decode_products_match_reference_fixture(oracle):
    gold = np.load(os.path.join(GOLDEN, "decode_products.npz"))
    table = oracle.decode_table().view(np.float32)             # index s*16+n
    for name in ("low_nibble_col0", "high_nibble_col1", "second_block_col17"):
        ref = bf16_bits_to_f32(gold[name])
        assert np.array_equal(table, ref), name                # values (+-0 compare equal)
    # every product fits a bf16: the tensor-core operand form relies on it
    assert np.array_equal(table.view(np.uint32) & 0xFFFF, np.zeros(4096, np.uint32))


def test_silu_mul_fixture(oracle):
    """SILU_MUL restatement against the reference's own kernel on every bf16 gate value."""
    gold = np.load(os.path.join(GOLDEN, "silu_mul.npz"))["y"]
    gate = np.arange(65536, dtype=np.uint16)
    up = np.random.Generator(np.random.PCG64(5)).integers(0, 65536, 65536, dtype=np.uint16)
    got = oracle.silu_mul(gate, up)
    nan = np.isnan(bf16_bits_to_f32(gold))
    assert np.array_equal(nan, np.isnan(bf16_bits_to_f32(got)))
    assert np.array_equal(got[~nan], gold[~nan])
    assert nan.sum() < 2000                                    # NaN/Inf inputs only


def test_random_bytes_fixture(oracle):
    g = np.load(os.path.join(GOLDEN, "random_bytes.npz"))
    y = oracle.gemm_f4(g["x"], g["payload"], g["scales"], 1.0)
    assert np.array_equal(y, g["y"])
    y1 = oracle.gemm_f4(g["x"], g["payload"], g["scales"], 1.0, threads=1)
    assert np.array_equal(y1, g["y"])


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "seeded_*.npz"))),
                         ids=lambda p: os.path.basename(p)[:-4])
def test_seeded_fixtures(oracle, lib, path):
    g = np.load(path)
    M, K, N = (int(v) for v in os.path.basename(path)[7:-4].split("x"))
    w = mm.make_weight(N, K, seed=0, std=0.02)
    x = mm.make_activations(M, K, seed=1)
    # the generator and the packer are pinned too
    assert fnv1a64(w.payload) == int(g["payload_fnv"])
    assert fnv1a64(w.scales) == int(g["scales_fnv"])
    assert fnv1a64(x) == int(g["x_fnv"])
    assert np.float32(w.gs) == g["gs"]
    assert np.array_equal(oracle.gemm_f4(x, w.payload, w.scales, 1.0), g["y"])


def test_status_fixture(oracle):
    g = np.load(os.path.join(GOLDEN, "status.npz"))
    assert int(g["k_not_multiple_of_16"]) == 4                  # MM_ERR_SHAPE
    with pytest.raises(ValueError):
        oracle.gemm_f4(np.zeros((1, 24), np.uint16), np.zeros((2, 12), np.uint8),
                       np.zeros((2, 2), np.uint8))


def test_sampled_rows_and_columns_agree_with_full(oracle, lib):
    w = mm.make_weight(80, 512, seed=3)
    x = mm.make_activations(9, 512, seed=4)
    full = oracle.gemm_f4(x, w.payload, w.scales, w.gs)
    part = oracle.gemm_f4(x, w.payload, w.scales, w.gs, rows=[1, 7, 8], n_begin=16, n_end=51)
    assert np.array_equal(part, full[[1, 7, 8], 16:51])


def test_global_scale_is_one_multiply_before_rounding(oracle, lib):
    w = mm.make_weight(48, 256, seed=5)
    x = mm.make_activations(4, 256, seed=6)
    y1, acc = oracle.gemm_f4(x, w.payload, w.scales, 1.0, want_acc=True)
    # power-of-two scale: reference result times gs is exact
    y4 = oracle.gemm_f4(x, w.payload, w.scales, 0.25)
    assert np.array_equal(bf16_bits_to_f32(y4), bf16_bits_to_f32(y1) * np.float32(0.25))
    # general scale: bf16_rne(acc * gs)
    gs = np.float32(w.gs)
    yg = oracle.gemm_f4(x, w.payload, w.scales, float(gs))
    want = mm.linear.f32_to_bf16(acc * gs)
    assert np.array_equal(yg, want)


def test_live_reference_silu_mul(oracle, reference):
    if not reference.available:
        pytest.skip("compiled reference not present")
    g = mm.make_activations(1, 5000, seed=12, std=4.0)[0]
    u = mm.make_activations(1, 5000, seed=13)[0]
    rc, y = reference.silu_mul(g, u)
    assert rc == 0 and np.array_equal(y, oracle.silu_mul(g, u))


def test_live_reference_when_present(oracle, reference, lib):
    if not reference.available:
        pytest.skip("compiled reference not present on this machine")
    for (M, K, N, s) in [(2, 1024, 50, 11), (7, 256, 19, 12), (1, 5120, 128, 13)]:
        w = mm.make_weight(N, K, seed=s)
        x = mm.make_activations(M, K, seed=s + 100)
        rc, yr = reference.gemm_f4(x, w.payload, w.scales)
        assert rc == 0
        assert np.array_equal(oracle.gemm_f4(x, w.payload, w.scales, 1.0), yr)
        rc, ym = reference.gemm_f4(x, w.payload, w.scales, threads=3)
        assert rc == 0 and np.array_equal(ym, yr)


def _golden_norm_inputs():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    return mg


def test_add_rmsnorm_fixture(oracle, lib):
    """The restatement of OP_ADD_RMSNORM against outputs of the reference's own
    kx_op_add_rmsnorm (src/kernels/cpu/cx.c:132-150): bit for bit, the in-place sum too."""
    mg = _golden_norm_inputs()
    g = np.load(os.path.join(GOLDEN, "add_rmsnorm.npz"))
    for (M, H) in mg.ADD_RMSNORM_SHAPES:
        res, delta, gain = mg.add_rmsnorm_inputs(M, H)
        res_out, y = oracle.add_rmsnorm(res, delta, gain, mg.ADD_RMSNORM_EPS)
        assert np.array_equal(res_out, g[f"res_{M}x{H}"])
        assert np.array_equal(y, g[f"y_{M}x{H}"])


def test_live_reference_add_rmsnorm(oracle, reference, lib):
    if not reference.available:
        pytest.skip("compiled reference not present")
    res = mm.make_activations(5, 2048, seed=21, std=3.0)
    delta = mm.make_activations(5, 2048, seed=22)
    gain = mm.make_activations(1, 2048, seed=23, std=0.3)[0]
    for eps in (1.0e-6, 1.0e-5, 0.0):
        rc, r1, y1 = reference.add_rmsnorm(res, delta, gain, eps)
        r2, y2 = oracle.add_rmsnorm(res, delta, gain, eps)
        assert rc == 0 and np.array_equal(r1, r2) and np.array_equal(y1, y2)
