"""Tile / variant selection (pure host C)."""
import pytest

import mimfer_b200 as mm
from mimfer_b200 import V_ROWWARP, V_STREAM, V_UMMA, V_STREAMT

WS = 64 << 20
SMEM_MAX = 232448


def test_decode_shapes_use_stream_and_fill_the_gpu(lib):
    for M in (1, 2, 4, 8, 16):
        for (K, N) in ((5120, 34816), (17408, 5120), (5120, 5120)):
            p = mm.select_plan(M, K, N, ws_bytes=WS)
            assert p.variant == V_STREAM
            assert p.m_tiles == -(-M // 8)
            assert p.k_steps == K // 256 and p.tile_n == 256 and p.grid_x == -(-N // 256)
            assert 100 <= p.grid_x * p.grid_y <= 148
            assert p.smem_bytes <= SMEM_MAX and p.stages >= 2
            if p.split_k > 1:
                assert p.ws_needed <= WS and p.k_steps // p.split_k >= 4


def test_small_weights_get_half_height_tiles(lib):
    """k and v projections (N = 1024): 256-row tiles give 20 CTAs at the deepest split, so
    the selector halves the tile; bigger weights keep 256 rows."""
    p = mm.select_plan(16, 5120, 1024, ws_bytes=WS)
    assert p.variant == V_STREAM and p.tile_n == 128 and p.grid_x == 8 and p.split_k == 5
    for (K, N) in ((5120, 6144), (5120, 34816), (17408, 5120)):
        assert mm.select_plan(16, K, N, ws_bytes=WS).tile_n == 256


def test_no_workspace_means_no_split(lib):
    p = mm.select_plan(16, 17408, 5120, ws_bytes=0)
    assert p.variant == V_STREAM and p.split_k == 1 and p.ws_needed == 0


def test_prefill_shapes_use_umma(lib):
    for M in (512, 2048, 8192):
        for (K, N) in ((5120, 34816), (17408, 5120), (5120, 6144), (5120, 1024), (6144, 5120)):
            p = mm.select_plan(M, K, N)
            assert p.variant == V_UMMA
            assert p.tile_m in (128, 256) and p.tile_n in (128, 256)
            assert p.grid_x == -(-N // p.tile_n) and p.grid_y == -(-M // p.tile_m)
            assert p.smem_bytes <= SMEM_MAX and p.stages >= 2 and p.k_steps == K // 64
    assert (mm.select_plan(8192, 5120, 34816).tile_m, mm.select_plan(8192, 5120, 34816).tile_n) == (256, 256)


def test_odd_shapes_fall_to_rowwarp(lib):
    assert mm.select_plan(3, 48, 7).variant == V_ROWWARP                 # K % 256 != 0
    assert mm.select_plan(64, 528, 100).variant == V_ROWWARP
    assert mm.select_plan(4, 512, 64, ptr_align=8).variant == V_ROWWARP   # TMA needs 16-byte bases
    assert mm.select_plan(100, 512, 102).variant == V_ROWWARP         # UMMA stores need N % 8 == 0


def test_deterministic(lib):
    a = mm.select_plan(16, 5120, 34816, ws_bytes=WS).as_dict()
    for _ in range(3):
        assert mm.select_plan(16, 5120, 34816, ws_bytes=WS).as_dict() == a


def test_errors(lib):
    for bad in ((0, 256, 8), (1, 0, 8), (1, 256, 0), (1, 24, 8)):
        with pytest.raises(mm.MimferError) as e:
            mm.select_plan(*bad)
        assert e.value.status == 4
    with pytest.raises(mm.MimferError) as e:
        mm.select_plan(64, 512, 64, variant=V_STREAM)            # M too large for the decode kernel
    assert e.value.status == 7
    with pytest.raises(mm.MimferError) as e:
        mm.select_plan(4, 48, 64, variant=V_UMMA)
    assert e.value.status == 7


def test_streamt_plan_mirrors_stream_decomposition(lib):
    for M in (1, 9, 16, 17, 32):
        a = mm.select_plan(M, 17408, 5120, ws_bytes=WS, variant=V_STREAM)
        b = mm.select_plan(M, 17408, 5120, ws_bytes=WS, variant=V_STREAMT)
        assert b.variant == V_STREAMT and b.tile_m == (16 if M <= 16 else 32)
        assert (b.grid_x, b.k_steps, b.tile_n) == (a.grid_x, a.k_steps, a.tile_n)
        assert b.split_k >= 1 and b.smem_bytes <= SMEM_MAX and b.threads == 736
        if b.split_k > 1:
            assert b.ws_needed == 16384 + b.split_k * b.tile_m * 5120 * 4
    with pytest.raises(mm.MimferError):
        mm.select_plan(64, 512, 64, variant=V_STREAMT)


def test_gated_pair_plans(lib):
    """mm_f4_select_glu: N counts output features; a CTA tile is 128 rows of each projection."""
    p = mm.select_plan(16, 5120, 17408, ws_bytes=WS, glu=True)
    assert p.variant == V_STREAM and p.grid_x == 17408 // 128 and p.split_k == 1
    p = mm.select_plan(4, 5120, 1000, ws_bytes=WS, glu=True)          # 8 tiles: K is split
    assert p.grid_x == 8 and p.split_k > 1
    assert p.ws_needed == 16384 + p.split_k * p.tile_m * 8 * 256 * 4  # partials per padded tile row
    for M in (512, 8192):
        p = mm.select_plan(M, 5120, 17408, glu=True)
        assert p.variant == V_UMMA and p.tile_n == 256 and p.grid_x == 136
        assert p.tile_m in (128, 256) and p.grid_y == -(-M // p.tile_m)
        assert p.smem_bytes <= SMEM_MAX
    for bad in ((4, 272, 128, 256), (64, 512, 100, 256), (4, 512, 128, 8)):
        M, K, N, align = bad
        with pytest.raises(mm.MimferError) as e:
            mm.select_plan(M, K, N, ptr_align=align, glu=True)
        assert e.value.status == 7                                    # MM_ERR_UNSUPPORTED
