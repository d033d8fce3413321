"""The quantising packer and the seeded generator (host C)."""
import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200.linear import fill_normal, f32_to_bf16, bf16_to_f32


def dequant(w, oracle):
    tab = oracle.decode_table().view(np.float32).reshape(256, 16)
    nib = np.stack([w.payload & 15, w.payload >> 4], -1).reshape(w.N, w.K)
    return tab[np.repeat(w.scales, 16, axis=1), nib] * np.float32(w.gs)


def test_layout_shapes_and_determinism(lib):
    a = mm.make_weight(40, 512, seed=0)
    b = mm.make_weight(40, 512, seed=0)
    assert a.payload.shape == (40, 256) and a.scales.shape == (40, 32)
    assert np.array_equal(a.payload, b.payload) and np.array_equal(a.scales, b.scales) and a.gs == b.gs
    c = mm.make_weight(40, 512, seed=1)
    assert not np.array_equal(a.payload, c.payload)


def test_make_weight_equals_pack_of_generated(lib):
    W = fill_normal(24, 256, 0, 0.0, 0.02)
    a, b = mm.pack_weight(W), mm.make_weight(24, 256, seed=0, std=0.02)
    assert np.array_equal(a.payload, b.payload) and np.array_equal(a.scales, b.scales) and a.gs == b.gs


def test_representable_values_round_trip(lib, oracle):
    """W built from representable (nibble, scale) pairs packs back to the same values."""
    rng = np.random.Generator(np.random.PCG64(1))
    tab = oracle.decode_table().view(np.float32).reshape(256, 16)
    N, K = 16, 256
    scales = rng.integers(0x40, 0x78, (N, K // 16)).astype(np.uint8)
    nib = rng.integers(0, 16, (N, K)).astype(np.uint8)
    nib[:, ::16] = 7                                           # every block reaches |6|
    scales[0, 0] = 0x7E                                        # and the tensor reaches 6*448
    nib[0, 0] = 7
    W = tab[np.repeat(scales, 16, axis=1), nib].astype(np.float32)
    w = mm.pack_weight(W)
    assert abs(w.gs - 1.0) < 1e-6
    assert np.allclose(dequant(w, oracle), W, rtol=1e-6, atol=0)


def test_quantisation_error_and_scale_range(lib, oracle):
    W = fill_normal(64, 1024, 0, 0.0, 0.02)
    w = mm.pack_weight(W)
    assert w.gs == pytest.approx(np.abs(W).max() / (6 * 448), rel=1e-6)
    rel = np.linalg.norm(dequant(w, oracle) - W) / np.linalg.norm(W)
    assert rel < 0.12                                          # NVFP4 with amax/6 block scales
    assert w.scales.max() <= 0x7E and (w.scales & 0x80).max() == 0
    assert len(np.unique(w.scales)) > 8                        # the global scale keeps e4m3 resolution


def test_all_zero_tensor(lib):
    w = mm.pack_weight(np.zeros((4, 64), np.float32))
    assert w.gs == 1.0 and not w.payload.any() and not w.scales.any()


def test_bad_shapes(lib):
    with pytest.raises(mm.MimferError) as e:
        mm.pack_weight(np.zeros((4, 24), np.float32))
    assert e.value.status == 4


def test_bf16_conversion_is_rne(lib):
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40], np.float32)
    bits = f32_to_bf16(x)
    assert bits[0] == 0x3F80
    assert bits[1] == 0x3F80           # 1 + 2^-8: tie, rounds to even
    assert bits[2] == 0x3F82           # 1 + 3*2^-8: tie, rounds to even (up)
    assert np.array_equal(bf16_to_f32(bits)[[0, 3]], np.array([1.0, -2.5], np.float32))


def test_generator_statistics_and_row_independence(lib):
    a = fill_normal(64, 4096, 9, 0.0, 1.0)
    assert abs(a.mean()) < 0.01 and abs(a.std() - 1.0) < 0.01
    b = fill_normal(32, 4096, 9, 0.0, 1.0)
    assert np.array_equal(a[:32], b)                           # rows do not depend on the row count


def test_host_only_packer_of_the_cpu_arm_matches(lib):
    """oracle/inputs.py (numpy, used where the product library must not be loaded) packs
    the same bytes as mm_f4_pack, ties and zero blocks included, and rounds to bf16 alike."""
    from oracle import inputs
    rng = np.random.Generator(np.random.PCG64(3))
    W = rng.standard_normal((96, 512), dtype=np.float32) * np.float32(0.02)
    W[3, :32] = 0.0
    W[5, 7] = 0.3
    W[9, 16:32] = np.float32(0.02) * np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0,
                                               -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0], np.float32)
    payload, scales, gs = inputs.pack(W)
    w = mm.pack_weight(W)
    assert np.array_equal(payload, w.payload) and np.array_equal(scales, w.scales) and gs == w.gs
    x = rng.standard_normal((8, 256), dtype=np.float32) * np.float32(3.0)
    x[0, :4] = [1.00390625, 1.01171875, -1.00390625, 3.0e-40]          # ties and a subnormal
    assert np.array_equal(inputs.bf16_bits(x), mm.linear.f32_to_bf16(x))
