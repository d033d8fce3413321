"""Tile / variant selection (pure host C)."""
import pytest

import mimfer_b200 as mm
from mimfer_b200 import V_ROWWARP, V_STREAM, V_UMMA, V_MX

WS = 64 << 20
SMEM_MAX = 232448


def test_decode_shapes_use_the_block_scaled_kernel_and_fill_the_gpu(lib):
    for M in (1, 2, 4, 8, 16, 32):
        for (K, N) in ((5120, 34816), (17408, 5120), (5120, 5120)):
            p = mm.select_plan(M, K, N, ws_bytes=WS)
            assert p.variant == V_MX and p.threads == 352
            assert p.m_tiles == -(-M // 4) and p.tile_m == 6 * 4 * p.m_tiles      # six digit planes per row
            assert p.k_steps == K // 256 and 32 <= p.tile_n <= 256 and p.tile_n % 4 == 0
            assert p.grid_x == -(-N // p.tile_n) and p.grid_y == p.split_k
            assert 100 <= p.grid_x * p.grid_y <= 148 or p.grid_x > 148
            assert p.smem_bytes <= SMEM_MAX and p.stages >= 2
            assert p.ws_needed <= WS
            if p.split_k > 1:
                assert p.k_steps // p.split_k >= 4


def test_block_scaled_tiles_even_out_over_the_sms(lib):
    """gate+up (34816 rows) runs as 148 tiles of 236 rows, not 136 of 256; down (5120
    rows) as 21 tiles x 7 K slices."""
    p = mm.select_plan(1, 5120, 34816, ws_bytes=WS)
    assert (p.tile_n, p.grid_x, p.split_k) == (236, 148, 1)
    p = mm.select_plan(16, 17408, 5120, ws_bytes=WS)
    assert (p.grid_x, p.split_k) == (21, 7) and p.tile_n * 21 >= 5120


def test_stream_kernel_when_asked_or_when_the_planes_do_not_fit(lib):
    for M in (1, 2, 4, 8, 16):
        for (K, N) in ((5120, 34816), (17408, 5120), (5120, 5120)):
            p = mm.select_plan(M, K, N, ws_bytes=WS, variant=V_STREAM)
            assert p.variant == V_STREAM
            assert p.m_tiles == -(-M // 8)
            assert p.k_steps == K // 256 and p.tile_n == 256 and p.grid_x == -(-N // 256)
            assert 100 <= p.grid_x * p.grid_y <= 148
            assert p.smem_bytes <= SMEM_MAX and p.stages >= 2
            if p.split_k > 1:
                assert p.ws_needed <= WS and p.k_steps // p.split_k >= 4
    # no workspace: no room for digit planes, so the selector itself falls back
    assert mm.select_plan(16, 17408, 5120, ws_bytes=0).variant == V_STREAM
    with pytest.raises(mm.MimferError) as e:
        mm.select_plan(16, 17408, 5120, ws_bytes=0, variant=V_MX)
    assert e.value.status == 7
    with pytest.raises(mm.MimferError):
        mm.select_plan(33, 512, 256, ws_bytes=WS, variant=V_MX)        # more than 32 activation rows


def test_small_weights_get_half_height_tiles(lib):
    """k and v projections (N = 1024) on the streaming kernel: 256-row tiles give 20 CTAs at
    the deepest split, so the selector halves the tile; bigger weights keep 256 rows."""
    p = mm.select_plan(16, 5120, 1024, ws_bytes=WS, variant=V_STREAM)
    assert p.variant == V_STREAM and p.tile_n == 128 and p.grid_x == 8 and p.split_k == 5
    for (K, N) in ((5120, 6144), (5120, 34816), (17408, 5120)):
        assert mm.select_plan(16, K, N, ws_bytes=WS, variant=V_STREAM).tile_n == 256


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


def test_prefill_tail_split(lib):
    """The tiles of the last, partial wave are cut into K slices so that the tail fills the
    SMs; only with a workspace, never below two 256-wide K groups per slice, and never more
    fp32 partial tiles than the workspace region holds."""
    region = 32 << 20
    p = mm.select_plan(2048, 17408, 5120, ws_bytes=region)              # down: 160 tiles = 148 + 12
    assert (p.tile_m, p.tile_n, p.grid_x * p.grid_y) == (256, 256, 160)
    assert (p.m_tiles, p.split_k) == (12, 10)
    assert p.ws_needed == 16384 + 12 * 10 * 256 * 256 * 4 <= region
    p = mm.select_plan(2048, 5120, 6144, ws_bytes=region)               # q: 192 tiles, 44 in the tail
    assert (p.m_tiles, p.split_k) == (44, 2) and p.ws_needed <= region  # 3 slices would not fit 32 MiB
    p = mm.select_plan(2048, 5120, 6144, ws_bytes=64 << 20)
    assert (p.m_tiles, p.split_k) == (44, 3)
    p = mm.select_plan(2048, 17408, 5120)                               # no workspace: whole tiles
    assert (p.m_tiles, p.split_k, p.ws_needed) == (0, 1, 0)
    p = mm.select_plan(8192, 5120, 1024, ws_bytes=region)               # 128 tiles in one wave of 148: 1 slice
    assert (p.m_tiles, p.split_k) == (0, 1)
    p = mm.select_plan(512, 512, 5120, ws_bytes=region)                 # K = 512: two K groups, nothing to cut
    assert p.split_k == 1
    for (M, K, N) in ((512, 5120, 1024), (2048, 5120, 1024), (512, 6144, 5120), (8192, 17408, 5120)):
        p = mm.select_plan(M, K, N, ws_bytes=region)
        if p.split_k > 1:
            assert 0 < p.m_tiles == (p.grid_x * p.grid_y) % 148
            assert p.m_tiles * p.split_k <= 148 and (K // 256) // p.split_k >= 2
            assert p.ws_needed == 16384 + p.m_tiles * p.split_k * p.tile_m * p.tile_n * 4 <= region


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
    with pytest.raises(mm.MimferError) as e:
        mm.select_plan(4, 512, 64, variant=3)                    # no such variant
    assert e.value.status != 0


def test_gated_pair_plans(lib):
    """mm_f4_select_glu: N counts output features; a CTA tile is 128 rows of each projection."""
    p = mm.select_plan(16, 5120, 17408, ws_bytes=WS, glu=True)
    assert p.variant == V_MX and p.split_k == 1
    assert p.tile_n % 16 == 0 and p.grid_x == -(-17408 // (p.tile_n // 2)) and 136 <= p.grid_x <= 148
    p = mm.select_plan(4, 5120, 1000, ws_bytes=WS, glu=True)          # few tiles: K is split
    assert p.variant == V_MX and p.split_k > 1 and p.ws_needed <= WS
    p = mm.select_plan(4, 5120, 1000, ws_bytes=0, glu=True)           # no room for digit planes
    assert p.variant == V_STREAM and p.grid_x == 8
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


def test_seeded_random_shapes_keep_the_plan_invariants(lib):
    """600 seeded random legal shapes, with and without a workspace: whatever kernel the
    selector picks, its tiles cover the output, the launch fits shared memory and the
    workspace it was offered, and the split fields agree with each other."""
    import random
    rng = random.Random(7)
    seen = set()
    for _ in range(600):
        M = rng.choice([rng.randint(1, 32), rng.randint(33, 9000)])
        K = rng.choice([256 * rng.randint(1, 80), 16 * rng.randint(1, 600)])
        N = rng.choice([8 * rng.randint(1, 20000), rng.randint(1, 40000)])
        ws = rng.choice([0, 8 << 20, 64 << 20])
        p = mm.select_plan(M, K, N, ws_bytes=ws)
        seen.add(p.variant)
        assert p.split_k >= 1 and p.ws_needed <= ws, (M, K, N, ws)
        if p.variant == V_ROWWARP:
            continue
        assert p.smem_bytes <= SMEM_MAX and (p.stages >= 2 or p.stages == p.k_steps // p.split_k == 1), (M, K, N)
        assert p.grid_x * p.tile_n >= N and (p.grid_x - 1) * p.tile_n < N, (M, K, N)
        if p.variant in (V_MX, V_STREAM):
            assert M <= 32 and K % 256 == 0 and p.k_steps == K // 256
            assert p.grid_y == p.split_k and p.split_k <= p.k_steps
            if ws == 0:
                assert p.split_k == 1
        if p.variant == V_MX:
            assert p.tile_m == 24 * -(-M // 4)
        if p.variant == V_UMMA:
            assert M > 32 and N % 8 == 0 and K % 256 == 0 and p.k_steps == K // 64
            tiles = p.grid_x * p.grid_y
            assert p.grid_y * p.tile_m >= M and (p.grid_y - 1) * p.tile_m < M
            if p.split_k > 1:
                assert 0 < p.m_tiles <= tiles and p.m_tiles * p.split_k <= 148
                assert p.ws_needed == 16384 + p.m_tiles * p.split_k * p.tile_m * p.tile_n * 4
            else:
                assert p.m_tiles == 0 and p.ws_needed == 0
    assert seen == {V_ROWWARP, V_UMMA, V_MX} or seen == {V_ROWWARP, V_UMMA, V_MX, V_STREAM}
