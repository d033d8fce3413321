/*
 * Tile and variant selection for the NVFP4 linear op: pure host C, no CUDA,
 * deterministic (a shape always maps to the same plan, so captured graphs and
 * direct dispatch agree).
 *
 * The mimfer planner emits OP_GEMM_F4 without choosing a kernel
 * (src/plan/plan.c:204-220); its descriptor comment only sketches the intent,
 * "M<=8: split-K gemv, else dequant + bf16 mma gemm" (include/mimfer/plan.h:51-52).
 * This file is that choice for B200:
 *
 *   MX       M <= 32 with a workspace.  HBM-bound.  The block-scaled tensor
 *            path: payload and block scales are the MMA's operands as they lie
 *            in memory, the activations are re-expressed as e2m1 digit planes by
 *            a small kernel in front (scratch in the workspace).  Same tiling as
 *            STREAM.
 *   STREAM   M <= 32 without a workspace (or when asked for).  One CTA streams
 *            256 weight rows through a TMA pipeline and dequantises on the CUDA
 *            cores; K is split across CTAs until about one CTA per SM exists,
 *            partials meet in the workspace in a fixed order.
 *   UMMA     M > 32.  tcgen05 tiles of tile_m x tile_n; the tile shape is the
 *            one with the lowest modelled time (waves x per-tile cost).
 *   ROWWARP  anything the two above cannot take (K not a multiple of 256,
 *            unaligned pointers).  Always valid for K % 16 == 0.
 */
#include "../core/core.h"
#include "../kernels/launch.h"
#include <string.h>

static uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
static mm_status check_shape(const mm_f4_shape *s, mm_f4_plan *out);

static int fast_path_ok(const mm_f4_shape *s)
{
    /* TMA: 16-byte aligned bases, row pitches K/2 and K/16 multiples of 16 B */
    return s->K % 256 == 0 && s->ptr_align >= 16 && s->ptr_align % 16 == 0;
}

static void plan_rowwarp(const mm_f4_shape *s, mm_f4_plan *p)
{
    memset(p, 0, sizeof *p);
    p->variant = MM_F4_V_ROWWARP;
    p->split_k = 1;
    p->threads = 256;                       /* 8 warps = 8 weight rows per CTA */
    p->grid_x = ceil_div(s->N, 8);
    p->grid_y = ceil_div(s->M, 4);          /* 4 activation rows per pass      */
    p->grid_z = 1;
    if (p->grid_y > 65535) p->grid_y = 65535;
}

/* STREAM plan with `rows` weight rows per CTA (a multiple of 16, at most
 * MMB_ST_ROWS) and K cut into `split` slices; split = 0 picks the split that
 * gives about one CTA per SM. */
static mm_status plan_stream_with(const mm_f4_shape *s, uint32_t rows, uint32_t split, mm_f4_plan *p)
{
    if (!fast_path_ok(s) || s->M > 32)
        return MM_ERR_UNSUPPORTED;
    if (rows == 0 || rows % 16u != 0 || rows > MMB_ST_ROWS)
        return MM_ERR_RANGE;
    memset(p, 0, sizeof *p);
    p->variant = MM_F4_V_STREAM;
    p->m_tiles = (s->M + 7u) / 8u;                /* 8-row activation tiles: 1..4 */
    p->tile_n = rows;
    p->tile_m = p->m_tiles * 8;
    p->k_steps = s->K / MMB_ST_KSTEP;
    p->grid_x = ceil_div(s->N, rows);
    p->threads = MMB_ST_THREADS;

    /* split K until roughly one CTA per SM, keeping >= 4 steps per slice */
    uint32_t sms = s->sm_count ? s->sm_count : 148;
    uint32_t sk = split ? split : sms / p->grid_x;
    if (sk < 1) sk = 1;
    uint32_t max_by_steps = p->k_steps / 4 ? p->k_steps / 4 : 1;
    if (sk > max_by_steps) sk = max_by_steps;
    if (sk > 32) sk = 32;
    if (p->grid_x > MMB_WS_MAX_TILES) sk = 1;
    while (sk > 1) {
        size_t need = MMB_WS_COUNTER_B + (size_t)sk * p->tile_m * s->N * 4u;
        if (need <= s->ws_bytes) { p->ws_needed = need; break; }
        sk--;
    }
    p->split_k = sk;
    p->grid_y = sk;
    p->grid_z = 1;

    uint32_t stage = MMB_ST_STAGE_B(p->m_tiles);
    uint32_t st = (MMB_SMEM_MAX - MMB_ST_FIXED_B) / stage;
    if (st > 6) st = 6;
    uint32_t per = ceil_div(p->k_steps, sk);
    if (st > per) st = per;
    if (st < 1) st = 1;
    p->stages = st;
    p->smem_bytes = st * stage + MMB_ST_FIXED_B;
    return MM_OK;
}

static mm_status plan_stream(const mm_f4_shape *s, mm_f4_plan *p)
{
    /* A weight with few rows (k and v projections: N = 1024) cannot fill the SMs
     * with 256-row tiles even at the deepest K split; half-height tiles double
     * the CTAs that stream it (measured on B200, N = 1024, K = 5120: 3.1 us
     * against 3.7 us at M = 1, 3.8 against 4.6 at M = 16; 64-row tiles lose again). */
    uint32_t sms = s->sm_count ? s->sm_count : 148;
    uint32_t k_steps = s->K / MMB_ST_KSTEP;
    uint32_t max_split = k_steps / 4 ? k_steps / 4 : 1;
    uint32_t rows = ceil_div(s->N, MMB_ST_ROWS) * max_split * 4u < sms ? MMB_ST_ROWS / 2 : MMB_ST_ROWS;
    return plan_stream_with(s, rows, 0, p);
}

/* MX plan.  `rows` weight rows per CTA (0 = sized here) and K cut into `split`
 * slices (0 = about one CTA per SM).  The kernel takes any tile height up to 256
 * rows (two MMA halves of up to 128), so the height is what makes row tiles x K
 * slices come out at the number of SMs: gate+up runs as 148 tiles of 236 rows
 * instead of 136 of 256, down as 21 x 7 instead of 20 x 7.  Workspace of the op:
 * arrival counters, the activation scratch (row factors, digit planes, their
 * block scales), split-K partials.  `glu`: gated pair, s->N = output features =
 * rows of each projection; a tile is tile_n / 2 rows of each. */
static mm_status plan_mx_with(const mm_f4_shape *s, uint32_t rows, uint32_t split, int glu, mm_f4_plan *p)
{
    if (!fast_path_ok(s) || s->M > 32)
        return MM_ERR_UNSUPPORTED;
    const uint32_t unit = glu ? 128u : 256u;       /* largest tile, in rows of one tensor */
    const uint32_t gran = glu ? 8u : 4u;
    if (rows && (rows % (glu ? 16u : 4u) != 0 || rows > 256u))
        return MM_ERR_RANGE;
    memset(p, 0, sizeof *p);
    p->variant = MM_F4_V_MX;
    p->m_tiles = (s->M + 3u) / 4u;                 /* groups of four activation rows */
    p->tile_m = p->m_tiles * 4u * MMB_MX_PLANES;   /* B rows: six digit planes per activation row */
    p->k_steps = s->K / MMB_ST_KSTEP;
    p->threads = MMB_MX_THREADS;
    const size_t xs = MMB_WS_COUNTER_B + MMB_MX_XS_B(p->tile_m, s->K);
    if (xs > s->ws_bytes)
        return MM_ERR_UNSUPPORTED;                 /* no room for the digit planes: the CUDA-core kernel runs */

    uint32_t sms = s->sm_count ? s->sm_count : 148;
    uint32_t per = rows ? (glu ? rows / 2u : rows) : unit;        /* rows of one tensor per tile */
    uint32_t tiles = ceil_div(s->N, per);
    uint32_t sk = split ? split : sms / tiles;
    if (sk < 1) sk = 1;
    uint32_t max_by_steps = p->k_steps / 4 ? p->k_steps / 4 : 1;
    if (sk > max_by_steps) sk = max_by_steps;
    if (sk > 32) sk = 32;
    if (tiles > MMB_WS_MAX_TILES) sk = 1;
    if (!rows) {
        /* lower tiles until tiles x slices reaches the SM count (never below 32 rows) */
        uint32_t want = sms / sk;
        if (tiles > sms)                            /* several waves: make the last one full too */
            want = ceil_div(tiles, sms) * sms;
        if (want > tiles && want <= MMB_WS_MAX_TILES) {
            per = ceil_div(ceil_div(s->N, want), gran) * gran;
            if (per < 32u) per = 32u;
            if (per > unit) per = unit;
            tiles = ceil_div(s->N, per);
        }
    }
    p->tile_n = glu ? 2u * per : per;
    p->grid_x = tiles;
    p->ws_needed = xs;
    while (sk > 1) {
        size_t need = xs + (size_t)sk * p->m_tiles * 4u * ((size_t)tiles * 256u) * 4u;
        if (need <= s->ws_bytes) { p->ws_needed = need; break; }
        sk--;
    }
    p->split_k = sk;
    p->grid_y = sk;
    p->grid_z = 1;
    uint32_t stage = MMB_MX_STAGE_B(p->tile_n, p->tile_m, glu);
    uint32_t st = (MMB_SMEM_MAX - MMB_MX_FIXED_B) / stage;
    if (st > 6) st = 6;
    uint32_t steps = ceil_div(p->k_steps, sk);
    if (st > steps) st = steps;
    if (st < 1) st = 1;
    p->stages = st;
    p->smem_bytes = st * stage + MMB_MX_FIXED_B;
    return MM_OK;
}

static mm_status plan_mx(const mm_f4_shape *s, mm_f4_plan *p)
{
    return plan_mx_with(s, 0, 0, 0, p);
}

/* MX plan of an op inside a group launch.  The CTAs take the work units of all
 * the group's ops in turn, so an op need not fill the SMs by itself: what counts
 * is that a unit is large enough to amortise its hand-over (accumulator switch,
 * epilogue, split-K exchange) and small enough for the tail of the group to stay
 * balanced.  Tiles of the full height, evened out over the rows; K is cut only
 * where a unit would exceed about 768 KiB of weights (split_k = 0), or as the
 * caller says. */
mm_status mmb_plan_mx_group(const mm_f4_shape *s, int glu, uint32_t split_k, mm_f4_plan *p)
{
    mm_status st = check_shape(s, p);
    if (st != MM_OK)
        return st;
    const uint32_t unit = glu ? 128u : 256u, gran = glu ? 8u : 4u;
    uint32_t tiles = ceil_div(s->N, unit);
    uint32_t per = ceil_div(ceil_div(s->N, tiles), gran) * gran;
    if (per > unit) per = unit;
    const uint32_t rows = glu ? 2u * per : per;
    const uint32_t k_steps = s->K / MMB_ST_KSTEP;
    uint32_t max_steps = (768u << 10) / (rows * 144u);
    if (max_steps < 4u) max_steps = 4u;
    uint32_t split = k_steps ? ceil_div(k_steps, max_steps) : 1u;
    if (split_k)                                    /* the caller's own K split */
        split = split_k;
    if (split > 32u) split = 32u;
    if (split < 1u) split = 1u;
    st = plan_mx_with(s, rows, split, glu, p);
    return st;
}

mm_status mmb_plan_mx_with(const mm_f4_shape *s, uint32_t rows, uint32_t split, mm_f4_plan *p)
{
    mm_status st = check_shape(s, p);
    return st != MM_OK ? st : plan_mx_with(s, rows, split, 0, p);
}

mm_status mmb_plan_stream_with(const mm_f4_shape *s, uint32_t rows, uint32_t split, mm_f4_plan *p)
{
    mm_status st = check_shape(s, p);
    return st != MM_OK ? st : plan_stream_with(s, rows ? rows : MMB_ST_ROWS, split, p);
}

/* modelled cost of one CTA tile, in MMA time of a 256 x 256 tile = 65536.  A K block's
 * time does not shrink with the tile below about 0.85 of a 256 x 256 tile's: measured
 * on B200, 64-wide K blocks take 0.55 us on 256 x 256 tiles and 0.45-0.5 us on 128 x 128
 * ones (k at M = 2048: 128 tiles, 80 K blocks, 44 us), whether four or eight warps
 * prepare a block's weights. */
static double umma_tile_cost(uint32_t bm, uint32_t bn)
{
    const double mma = (double)bm * bn, chain = 0.85 * 65536.0;
    return mma > chain ? mma : chain;
}

/* Tail split of the prefill kernel: the `rem` tiles of the last, partial wave are
 * cut into K slices (one CTA each) so that the tail fills the SMs once more:
 * slices = SMs / rem, at least two 256-wide K groups per slice, and as many
 * fp32 partial tiles as the workspace region holds.  Returns the slices (1 = no
 * split) and the workspace bytes. */
static uint32_t umma_tail(const mm_f4_shape *s, uint32_t bm, uint32_t bn, uint32_t tiles, size_t *ws_needed)
{
    const uint32_t sms = s->sm_count ? s->sm_count : 148;
    const uint32_t rem = tiles % sms, groups = s->K / 256u;
    const size_t tile_b = (size_t)bm * bn * 4u;
    *ws_needed = 0;
    if (rem == 0 || s->ws_bytes <= MMB_WS_COUNTER_B)
        return 1;
    uint32_t slices = sms / rem;
    const size_t room = (s->ws_bytes - MMB_WS_COUNTER_B) / tile_b;
    if ((size_t)rem * slices > room)
        slices = (uint32_t)(room / rem);
    if (slices > groups / 2u)
        slices = groups / 2u;
    if (slices < 2u)
        return 1;
    *ws_needed = MMB_WS_COUNTER_B + (size_t)rem * slices * tile_b;
    return slices;
}

/* waves of tiles a launch takes, the last wave counted as its K slices' share of a
 * tile plus what a split costs beside its K blocks (the slices' fill, the partial
 * sums out and back in, the tail kernel: about 12 us against 0.55 us per 64-wide
 * K block of a 256 x 256 tile) */
static double umma_waves(const mm_f4_shape *s, uint32_t bm, uint32_t bn, uint32_t tiles)
{
    const uint32_t sms = s->sm_count ? s->sm_count : 148;
    size_t ws = 0;
    const uint32_t slices = umma_tail(s, bm, bn, tiles, &ws);
    double w = (double)(tiles / sms);
    if (tiles % sms)
        w += slices > 1 ? 1.0 / slices + 12.0 / ((double)(s->K / MMB_UM_KBLOCK) * 0.55 *
                                                  umma_tile_cost(bm, bn) / 65536.0)
                        : 1.0;
    return w;
}

static void umma_set_tail(const mm_f4_shape *s, mm_f4_plan *p)
{
    const uint32_t sms = s->sm_count ? s->sm_count : 148;
    const uint32_t tiles = p->grid_x * p->grid_y;
    size_t ws = 0;
    const uint32_t slices = umma_tail(s, p->tile_m, p->tile_n, tiles, &ws);
    p->split_k = slices;
    p->m_tiles = slices > 1 ? tiles % sms : 0;
    p->ws_needed = ws;
}

static mm_status plan_umma(const mm_f4_shape *s, mm_f4_plan *p)
{
    /* smallest first: on equal modelled time the smaller tile wins (less padding traffic) */
    static const uint32_t cand[3][2] = { {128, 128}, {128, 256}, {256, 256} };
    if (!fast_path_ok(s) || s->N % 8 != 0)
        return MM_ERR_UNSUPPORTED;
    double best = 0.0;
    int best_i = -1;
    for (int i = 0; i < 3; i++) {
        uint32_t bm = cand[i][0], bn = cand[i][1];
        uint32_t tiles = ceil_div(s->M, bm) * ceil_div(s->N, bn);
        double t = umma_waves(s, bm, bn, tiles) * umma_tile_cost(bm, bn);
        if (best_i < 0 || t < best * 0.999) { best = t; best_i = i; }
    }
    memset(p, 0, sizeof *p);
    p->variant = MM_F4_V_UMMA;
    p->tile_m = cand[best_i][0];
    p->tile_n = cand[best_i][1];
    p->split_k = 1;
    p->k_steps = s->K / MMB_UM_KBLOCK;
    p->grid_x = ceil_div(s->N, p->tile_n);
    p->grid_y = ceil_div(s->M, p->tile_m);
    p->grid_z = 1;
    p->threads = MMB_UM_THREADS;
    uint32_t st = 6;
    while (st > 2 && MMB_UM_SMEM_B(p->tile_m, p->tile_n, st) > MMB_SMEM_MAX) st--;
    p->stages = st;
    p->smem_bytes = MMB_UM_SMEM_B(p->tile_m, p->tile_n, st);
    if (p->smem_bytes > MMB_SMEM_MAX)
        return MM_ERR_UNSUPPORTED;
    umma_set_tail(s, p);
    return MM_OK;
}

static mm_status check_shape(const mm_f4_shape *s, mm_f4_plan *out)
{
    if (!s || !out)
        return MM_ERR_STATE;
    if (s->M == 0 || s->N == 0 || s->K == 0 || s->K % 16 != 0)
        return MM_ERR_SHAPE;
    return MM_OK;
}

mm_status mm_f4_select_variant(const mm_f4_shape *s, int variant, mm_f4_plan *out)
{
    mm_status st = check_shape(s, out);
    if (st != MM_OK)
        return st;
    switch (variant) {
    case MM_F4_V_ROWWARP: plan_rowwarp(s, out); return MM_OK;
    case MM_F4_V_STREAM:  return plan_stream(s, out);
    case MM_F4_V_UMMA:    return plan_umma(s, out);
    case MM_F4_V_MX:      return plan_mx(s, out);
    default:              return MM_ERR_RANGE;
    }
}

/* Gated pair (gate and up projections + silu(gate) * up in one kernel): s->N is
 * the number of output features, so the kernels stream 2 * N weight rows and a
 * CTA's 256-row tile is 128 rows of each projection.  Only the TMA kernels have
 * the fused form; anything else is MM_ERR_UNSUPPORTED and runs as three ops. */
mm_status mm_f4_select_glu(const mm_f4_shape *s, mm_f4_plan *out)
{
    return mmb_select_glu(s, 1, out);
}

mm_status mmb_select_glu(const mm_f4_shape *s, int allow_mx, mm_f4_plan *out)
{
    mm_status st = check_shape(s, out);
    if (st != MM_OK)
        return st;
    if (!fast_path_ok(s))
        return MM_ERR_UNSUPPORTED;
    mm_f4_shape rows = *s;
    rows.N = ceil_div(s->N, MMB_ST_ROWS / 2) * MMB_ST_ROWS;      /* weight rows incl. tile padding */
    if (s->M <= 32) {
        /* the tile padding only counts rows: the planes' size follows K and M */
        if (allow_mx && plan_mx_with(s, 0, 0, 1, out) == MM_OK)
            return MM_OK;
        return plan_stream_with(&rows, MMB_ST_ROWS, 0, out);       /* partials are laid out per 256-row tile */
    }
    if (s->N % 8 != 0)
        return MM_ERR_UNSUPPORTED;
    uint32_t gx = rows.N / 256u;
    double w256 = umma_waves(s, 256, 256, ceil_div(s->M, 256) * gx), w128 = umma_waves(s, 128, 256, ceil_div(s->M, 128) * gx);
    uint32_t bm = w256 * umma_tile_cost(256, 256) <= w128 * umma_tile_cost(128, 256) * 0.999 ? 256u : 128u;
    memset(out, 0, sizeof *out);
    out->variant = MM_F4_V_UMMA;
    out->tile_m = bm;
    out->tile_n = 256;
    out->split_k = 1;
    out->k_steps = s->K / MMB_UM_KBLOCK;
    out->grid_x = gx;
    out->grid_y = ceil_div(s->M, bm);
    out->grid_z = 1;
    out->threads = MMB_UM_THREADS;
    uint32_t stg = 6;
    while (stg > 2 && MMB_UM_SMEM_B(bm, 256u, stg) > MMB_SMEM_MAX) stg--;
    out->stages = stg;
    out->smem_bytes = MMB_UM_SMEM_B(bm, 256u, stg);
    if (out->smem_bytes > MMB_SMEM_MAX)
        return MM_ERR_UNSUPPORTED;
    umma_set_tail(s, out);
    return MM_OK;
}

mm_status mm_f4_select(const mm_f4_shape *s, mm_f4_plan *out)
{
    mm_status st = check_shape(s, out);
    if (st != MM_OK)
        return st;
    /* decode: the block-scaled tensor kernel when the digit planes of the
     * activations fit the workspace, else the CUDA-core streaming kernel */
    if (s->M <= 32 && (plan_mx(s, out) == MM_OK || plan_stream(s, out) == MM_OK))
        return MM_OK;
    if (s->M > 32 && plan_umma(s, out) == MM_OK)
        return MM_OK;
    plan_rowwarp(s, out);
    return MM_OK;
}
