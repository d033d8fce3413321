/*
 * MX: the decode kernel of the NVFP4 linear op on the block-scaled tensor path
 * (M <= 32, HBM-bound).
 *
 * NVFP4 is the operand format of tcgen05.mma kind::mxf4nvf4: packed e2m1
 * payload, one e4m3 scale per 16 values.  A TMA box of payload (rows x 128 B,
 * 128-byte swizzle) is the A operand as it lies in memory, and the matching box
 * of block scales is its scale-factor tensor once copied into tensor memory.  So
 * no CUDA core touches a weight: the SM streams boxes and issues MMAs.
 *
 * The other operand has to be e2m1 with power-of-two block scales too, and the
 * reference keeps activations in bf16 (src/kernels/cpu/cx.c:211).  A small
 * kernel in front (f4_xslice_kernel) rewrites every bf16 activation as a sum
 * of six signed e2m1 digits on block scales 2^(s_p) * unit, s_p = 1, 3, 6, 9,
 * 12, 15: digit planes p = 0..5 of every activation row become rows of the B
 * operand (NB = 6 x padded M rows), the fp32 accumulator columns of the planes of
 * one activation row are added in the epilogue.  The digit set of e2m1
 * {0, .5, 1, 1.5, 2, 3, 4, 6} with signs covers every integer up to 149 796
 * units with six digits (greedy, nearest digit first), i.e. 17 bits below the
 * largest value of a 16-wide block: a bf16 value is reproduced exactly when it
 * lies within 2^9 of its block's maximum, smaller ones are rounded at 2^-17 of
 * that maximum (and never coarser than 2^-19 of the row maximum), which is below
 * the rounding error of the reference's own fp32 accumulation.  Weights and
 * block scales are exact, products are exact, sums are fp32.
 *
 * Scale bytes the tensor core reads differently from the reference decoder
 * (include/mimfer/tensor.h:98-118) are rewritten on the way into tensor memory:
 * 0x7f and 0xff (zero in the reference, NaN as ue4m3) become 0, and a byte with the sign
 * bit set (the tensor core ignores it) has the bit cleared and the sign bits of
 * the 16 payload nibbles of its block flipped in shared memory instead.
 *
 * Warp roles (11 warps): 0 = TMA producer; 1 and 10 = MMA issue for the first
 * and the second 128-row half (one thread each; warp 1 owns tensor memory);
 * 2..9 = scale-factor copies into tensor memory: one warp per lane quadrant (the
 * data is replicated over the four) and per parity of the K step, so a warp
 * has two steps' time for its copy; warps 2..5 then run the epilogue.
 *
 * It replaces the one-thread-per-output kernel of the reference
 * (src/kernels/cuda/cx.cu:345-356) for the decode regime.
 */
#include "fp4.cuh"
#include "ptx.cuh"
#include "mx.cuh"

namespace mmb {

#ifdef MMB_MX_TRACE
/* build-time option for timing studies: a timeline of kernel entries and exits
 * (global timer, first and last CTA of every launch) */
__device__ unsigned long long g_tl[4 * 4096];
__device__ unsigned g_tl_n;
__device__ __forceinline__ void tl_mark(unsigned kind)
{
    const unsigned i = atomicAdd(&g_tl_n, 1u);
    if (i < 4096u) {
        g_tl[4 * i] = kind;
        g_tl[4 * i + 1] = blockIdx.x + 1000u * blockIdx.y;
        g_tl[4 * i + 2] = globaltimer_ns();
        g_tl[4 * i + 3] = gridDim.x * gridDim.y;
    }
}
#define TL_MARK(kind) do { if (threadIdx.x == 0 && ((blockIdx.x == 0 && blockIdx.y == 0) || (blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1))) tl_mark(kind); } while (0)
/* CTA 0 records the SM clock at the hand-offs
 * of its first 32 K steps */
__device__ long long g_mx_trace[12 * 32];
#define MX_TRACE(ev, it) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (it) < 32u) g_mx_trace[(ev) * 32 + (it)] = clock64(); } while (0)
#else
#define MX_TRACE(ev, it) do { } while (0)
#define TL_MARK(kind) do { } while (0)
#endif

/* ==========================================================================
 * Activation slicing
 * ========================================================================== */
struct XsliceParams {
    const uint16_t *x;          /* bf16 [M][K]                                    */
    uint8_t        *planes;     /* [NB][K/2] e2m1 nibbles, row = 6 * m + plane     */
    uint8_t        *sfb;        /* [NB][K/16] ue4m3 powers of two                  */
    float          *row_scale;  /* [Mpad][2]: two factors whose product is 2^-G(m) */
    uint32_t        M, K, m_pad;
    uint32_t        pdl;
};

/* Thread = four consecutive activations (a quarter of a 16-wide block); a CTA
 * covers 1024 values of one activation row; grid = (ceil(K / 1024), padded M). */
__global__ void __launch_bounds__(256)
f4_xslice_kernel(const XsliceParams p)
{
    TL_MARK(1);
    grid_dep_launch();                       /* the linear kernel may start fetching weights */
    if (p.pdl != MMB_PDL_OFF)
        grid_dep_wait();                     /* x is the previous kernel's output */
    xslice_cta(p.x, p.planes, p.sfb, p.row_scale, p.M, p.K, blockIdx.y, blockIdx.x);
    TL_MARK(2);
}

/* ==========================================================================
 * The linear kernel
 * ========================================================================== */

struct MxParams {
    uint16_t       *y[MMB_MAX_PEERS];
    uint32_t        n_dst, ldy, col0;
    float          *partial;
    unsigned       *counters;
    unsigned       *status;
    const float    *row_scale;
    float           gs, gs_up;
    uint32_t        gate_plane;
    uint32_t        M, K, N;
    uint32_t        k_steps, split_k, stages;
    uint32_t        pdl;
    uint32_t        rows;        /* weight rows per CTA, a multiple of 4 up to 256 (GLU: 2 x rows of each projection) */
    uint32_t        nb;          /* B rows: 6 x M padded to a multiple of four                          */
};

__device__ __forceinline__ void mx_store_all(const MxParams &p, uint32_t m, uint32_t n, uint16_t v)
{
    const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n;
    p.y[0][off] = v;
#pragma unroll 1
    for (uint32_t d = 1; d < p.n_dst; d++)
        p.y[d][off] = v;
}

/* 128 registers per thread: the slicing kernels of the ops behind (256 threads,
 * 32 registers) must fit on the SM beside this kernel's one CTA, or they wait for
 * it to leave and then hold up the next linear kernel's CTA on that SM. */
template <bool GLU>
__global__ void __maxnreg__(128)
f4_mx_kernel(const __grid_constant__ TmaDesc tm_payload, const __grid_constant__ TmaDesc tm_scale,
             const __grid_constant__ TmaDesc tm_planes, const __grid_constant__ TmaDesc tm_sfb,
             const MxParams p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    /* The tile is two MMA halves of up to 128 weight rows.  Plain op: rows 0..127 and
     * 128..rows-1 of the box; gated pair: rows/2 rows of each projection, one after
     * the other.  Rows of a half beyond its count hold whatever the stage held before:
     * their accumulator lanes are never read, their scale factors are forced to zero. */
    const uint32_t rows = p.rows, nb = p.nb;
    const uint32_t halves = GLU ? 2u : (rows > 128u ? 2u : 1u);
    const uint32_t h1 = GLU ? rows >> 1 : 128u;                 /* first row of the second half */
    const uint32_t cnt0 = GLU ? rows >> 1 : (rows < 128u ? rows : 128u), cnt1 = rows - cnt0;
    const uint32_t pay_b = rows * 128u, pl_b = nb * 128u, sc_b = rows * 16u, sfb_b = nb * 16u;
    const uint32_t stage_b = MMB_MX_STAGE_B(rows, nb, GLU);
    const uint32_t o_pl = MMB_MX_PAY_B(rows, GLU), o_sc = o_pl + pl_b, o_sfb = o_sc + MMB_MX_SC_B(rows);
    const uint32_t bars = base + p.stages * stage_b;
    const uint32_t bar_full = bars;                              /* [stages] TMA landed             */
    const uint32_t bar_empty = bar_full + 8u * p.stages;         /* [stages] MMAs of the stage done */
    const uint32_t bar_sf_full = bar_empty + 8u * p.stages;      /* [2] scale factors in tensor memory */
    const uint32_t bar_accum = bar_sf_full + 16u;
    const uint32_t tmem_slot = bar_accum + 8u;
    const uint32_t last_flag = tmem_slot + 4u;
    const uint32_t rs_smem = last_flag + 4u;                     /* [32][2] row factors 2^-G */

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid == 0) MX_TRACE(11, 0);
    TL_MARK(3);
    const uint32_t row0 = blockIdx.x * (GLU ? rows >> 1 : rows); /* first weight row (of each projection) */
    const uint32_t ks_begin = static_cast<uint32_t>(static_cast<uint64_t>(p.k_steps) * blockIdx.y / p.split_k);
    const uint32_t ks_end = static_cast<uint32_t>(static_cast<uint64_t>(p.k_steps) * (blockIdx.y + 1) / p.split_k);
    const uint32_t nsteps = ks_end - ks_begin;
    const uint32_t first = nsteps < p.stages ? nsteps : p.stages;
    const uint32_t stage_tx = pay_b + pl_b + sc_b + sfb_b;

    if (tid == 0) {
        tma_prefetch_desc(&tm_payload);
        tma_prefetch_desc(&tm_scale);
        tma_prefetch_desc(&tm_planes);
        tma_prefetch_desc(&tm_sfb);
        for (uint32_t s = 0; s < p.stages; s++) {
            mbar_init(bar_full + 8u * s, 1u);
            mbar_init(bar_empty + 8u * s, halves);       /* one commit per issuing thread */
        }
        for (uint32_t t = 0; t < 2u; t++)
            mbar_init(bar_sf_full + 8u * t, 4u);
        mbar_init(bar_accum, halves);
        mbar_fence_init();
        /* the weight boxes of the first ring go out before anything else */
        for (uint32_t it = 0; it < first; it++) {
            const uint32_t st = base + it * stage_b, ks = ks_begin + it;
            mbar_expect_tx(bar_full + 8u * it, stage_tx);
            if constexpr (GLU) {
                tma_load_3d(st, &tm_payload, static_cast<int>(ks * 128u), static_cast<int>(row0), 0, bar_full + 8u * it);
                tma_load_3d(st + o_sc, &tm_scale, static_cast<int>(ks * 16u), static_cast<int>(row0), 0, bar_full + 8u * it);
            } else {
                tma_load_2d(st, &tm_payload, static_cast<int>(ks * 128u), static_cast<int>(row0), bar_full + 8u * it);
                tma_load_2d(st + o_sc, &tm_scale, static_cast<int>(ks * 16u), static_cast<int>(row0), bar_full + 8u * it);
            }
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512u);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds32(tmem_slot);
    if (p.pdl == MMB_PDL_TRIGGER_FIRST)
        grid_dep_launch();

    if (warp == 0) {
        /* ------------------------------ TMA producer ------------------------ */
        if (lane == 0) {
            if (p.pdl == MMB_PDL_INDEPENDENT) {
                grid_dep_launch();
            } else {
                grid_dep_wait();                 /* the digit planes come from the kernel in front */
                if (p.pdl == MMB_PDL_WAIT_FIRST)
                    grid_dep_launch();
            }
            for (uint32_t it = 0; it < first; it++) {
                const uint32_t st = base + it * stage_b, ks = ks_begin + it;
                tma_load_2d(st + o_pl, &tm_planes, static_cast<int>(ks * 128u), 0, bar_full + 8u * it);
                tma_load_2d(st + o_sfb, &tm_sfb, static_cast<int>(ks * 16u), 0, bar_full + 8u * it);
                MX_TRACE(0, it);
            }
            uint32_t s = 0, round = 1;
            for (uint32_t it = first; it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u, round += (s == 0u)) {
                const uint32_t st = base + s * stage_b, ks = ks_begin + it, bar = bar_full + 8u * s;
                mbar_wait(bar_empty + 8u * s, (round - 1u) & 1u, p.status);
                mbar_expect_tx(bar, stage_tx);
                if constexpr (GLU) {
                    tma_load_3d(st, &tm_payload, static_cast<int>(ks * 128u), static_cast<int>(row0), 0, bar);
                    tma_load_3d(st + o_sc, &tm_scale, static_cast<int>(ks * 16u), static_cast<int>(row0), 0, bar);
                } else {
                    tma_load_2d(st, &tm_payload, static_cast<int>(ks * 128u), static_cast<int>(row0), bar);
                    tma_load_2d(st + o_sc, &tm_scale, static_cast<int>(ks * 16u), static_cast<int>(row0), bar);
                }
                tma_load_2d(st + o_pl, &tm_planes, static_cast<int>(ks * 128u), 0, bar);
                tma_load_2d(st + o_sfb, &tm_sfb, static_cast<int>(ks * 16u), 0, bar);
                MX_TRACE(0, it);
            }
            if (p.pdl == MMB_PDL_INDEPENDENT)
                grid_dep_wait();                 /* this kernel completes after its predecessor */
        }
    } else if (warp == 1 || warp == 10) {
        /* ------------------------------ MMA issue ---------------------------- *
         * One thread per 128-row half: eight MMAs per K step cost one thread more
         * issue time than the step's weights take to arrive. */
        const uint32_t h = warp == 1 ? 0u : 1u;
        if (lane == 0 && h < halves) {
            const uint32_t idesc = umma_idesc_mxf4(nb);
            uint32_t s = 0, round = 0;
            for (uint32_t it = 0; it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u, round += (s == 0u)) {
                const uint32_t t = it & 1u, st = base + s * stage_b;
                mbar_wait(bar_full + 8u * s, round & 1u, p.status);
                if (h == 0) MX_TRACE(1, it);
                mbar_wait(bar_sf_full + 8u * t, (it >> 1) & 1u, p.status);
                tc_fence_after();
                if (h == 0) MX_TRACE(2, it);
                const uint32_t sf = tmem + MMB_MX_SF_COL + t * MMB_MX_SF_SLOT;
                const uint64_t ad = umma_desc_sw128(st + h * h1 * 128u), bd = umma_desc_sw128(st + o_pl);
#pragma unroll
                for (uint32_t j = 0; j < 4u; j++)       /* 32 bytes along K per slice: + 2 in the address field */
                    umma_mxf4(tmem + h * nb, ad + 2u * j, bd + 2u * j, idesc, (it | j) ? 1u : 0u,
                              sf + h * 16u + 4u * j, sf + MMB_MX_SFB_OFF + 8u * j);
                umma_commit(bar_empty + 8u * s);       /* frees the stage and, two steps on, the scale slot */
                if (h == 0) MX_TRACE(3, it);
            }
            umma_commit(bar_accum);
        }
    } else {
        /* ------------------------------ scale factors ------------------------ *
         * Lane l of a slot's column c holds the four scale bytes (K = 64) of row
         * 32 c + l; every lane quadrant holds a copy, so the four warps write the
         * same values, each into its own quadrant. */
        const uint32_t quad = warp & 3u;
        const uint32_t mine_t = (warp - 2u) >> 2;      /* this warp fills slot 0 (even steps) or 1 (odd steps) */
        const uint32_t tq = tmem + ((quad * 32u) << 16);
        const uint32_t ncol = (nb + 31u) >> 5;
        uint32_t s = 0, round = 0;
        uint32_t s1 = 0, round1 = 0, s2 = 0, round2 = 0;      /* stage and use count of the steps one and two back */
        for (uint32_t it = 0; it < nsteps; it++, s2 = s1, round2 = round1, s1 = s, round1 = round,
                                           s = (s + 1u == p.stages) ? 0u : s + 1u, round += (s == 0u)) {
            const uint32_t t = it & 1u, st = base + s * stage_b;
            if (t != mine_t)
                continue;
            mbar_wait_warp(bar_full + 8u * s, round & 1u, p.status);
            if (warp == 2u && lane == 0) MX_TRACE(4, it);
            if (it == 0u && warp == 2u) {
                /* the planes of step 0 have landed, so the kernel that made them is done:
                 * its row factors go to shared memory for the epilogue */
                sts32(rs_smem + 4u * lane, __float_as_uint(lane < 2u * p.M ? __ldcg(p.row_scale + lane) : 0.0f));
                sts32(rs_smem + 4u * (lane + 32u),
                      __float_as_uint(lane + 32u < 2u * p.M ? __ldcg(p.row_scale + lane + 32u) : 0.0f));
            }
            if (it >= 2u)                        /* the slot is free once the MMAs of step it - 2 are done */
                mbar_wait_warp(bar_empty + 8u * s2, round2 & 1u, p.status);
            tc_fence_after();
            if (warp == 2u && lane == 0) MX_TRACE(5, it);
            const uint32_t sf = tq + MMB_MX_SF_COL + t * MMB_MX_SF_SLOT;
            bool patched = false;
            uint32_t v[64];                      /* the slot: A scales of both halves, then B scales */
            uint4 qa[8];
#pragma unroll
            for (uint32_t i = 0; i < 8u; i++) {
                const uint32_t in_half = 32u * (i & 3u) + lane;
                qa[i] = make_uint4(0u, 0u, 0u, 0u);
                if (in_half < ((i >> 2) ? cnt1 : cnt0))
                    qa[i] = lds128(st + o_sc + ((i >> 2) * h1 + in_half) * 16u);
            }
            if (warp == 2u && lane == 0) MX_TRACE(8, it);
            /* Branch-free on the common path (a lone warp pays dearly for every
             * branch): 0x7f and 0xff, zero in the reference, are cleared; sign bits
             * are cleared and collected. */
            uint32_t negs = 0u;
#pragma unroll
            for (uint32_t i = 0; i < 8u; i++) {
                const uint32_t w[4] = { qa[i].x, qa[i].y, qa[i].z, qa[i].w };
#pragma unroll
                for (uint32_t j = 0; j < 4u; j++) {
                    const uint32_t nan = (((w[j] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) >> 7;
                    const uint32_t clean = w[j] & ~(nan * 0xffu);
                    negs |= clean & 0x80808080u;
                    v[(i >> 2) * 16u + 4u * j + (i & 3u)] = clean & 0x7f7f7f7fu;
                }
            }
            if (__any_sync(0xffffffffu, negs != 0u)) {
                /* negative block scales (no packer writes them, the reference decodes
                 * them): flip the signs of the block's 16 weights in shared memory
                 * instead; one warp does it, every warp has cleared the sign bits */
                if (quad == 2u && negs) {
#pragma unroll
                    for (uint32_t i = 0; i < 8u; i++) {
                        const uint32_t r = (i >> 2) * h1 + 32u * (i & 3u) + lane;     /* row of the payload box */
                        const uint32_t w[4] = { qa[i].x, qa[i].y, qa[i].z, qa[i].w };
#pragma unroll
                        for (uint32_t j = 0; j < 4u; j++) {
                            const uint32_t nan = (((w[j] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) >> 7;
                            const uint32_t neg = w[j] & ~(nan * 0xffu) & 0x80808080u;
                            for (uint32_t b = 0; neg && b < 4u; b++)
                                if (neg & (0x80u << (8u * b))) {
                                    const uint32_t o = (4u * j + b) * 8u;
                                    const uint32_t a = st + r * 128u + ((((o >> 4) ^ (r & 7u)) << 4) | (o & 15u));
                                    sts32(a, lds32(a) ^ 0x88888888u);
                                    sts32(a + 4u, lds32(a + 4u) ^ 0x88888888u);
                                }
                        }
                    }
                }
                patched = true;
            }
            if (warp == 2u && lane == 0) MX_TRACE(9, it);
#pragma unroll
            for (uint32_t c = 0; c < 8u; c++) {
                const uint32_t r = 32u * c + lane;
                uint4 q = make_uint4(0u, 0u, 0u, 0u);
                if (c < ncol && r < nb)
                    q = lds128(st + o_sfb + r * 16u);
                v[MMB_MX_SFB_OFF + c] = q.x;
                v[MMB_MX_SFB_OFF + 8u + c] = q.y;
                v[MMB_MX_SFB_OFF + 16u + c] = q.z;
                v[MMB_MX_SFB_OFF + 24u + c] = q.w;
            }
            if (warp == 2u && lane == 0) MX_TRACE(10, it);
            tmem_st_x64(sf, v);
            if (warp == 2u && lane == 0) MX_TRACE(6, it);
            tmem_st_wait();
            if (warp == 2u && lane == 0) MX_TRACE(7, it);
            if (patched)
                fence_proxy_async_smem();        /* the tensor core reads the rewritten payload */
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(bar_sf_full + 8u * t);
        }

        /* ------------------------------ epilogue ----------------------------- *
         * Thread = weight row (lane of tensor memory); four activation rows (24
         * plane columns) at a time.  One warp per quadrant. */
        if (mine_t != 0u)
            goto done;
        mbar_wait_warp(bar_accum, 0u, p.status);
        tc_fence_after();
        if (warp == 2u && lane == 0) MX_TRACE(11, 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");       /* row factors written by warp 2 */
        const uint32_t lr = quad * 32u + lane;   /* row within a half */
        const uint32_t groups = nb / 24u;
        const bool direct = p.split_k == 1u;
        const uint32_t pitch = GLU ? gridDim.x * 256u : p.N;   /* partials: one column per weight row of the tiles */
        float *mine = p.partial + static_cast<size_t>(blockIdx.y) * (groups * 4u) * pitch;
        for (uint32_t g = 0; g < groups; g++) {
            uint32_t c0[24], c1[24];
            tmem_ld_x8(tq + g * 24u, *reinterpret_cast<uint32_t (*)[8]>(&c0[0]));
            tmem_ld_x8(tq + g * 24u + 8u, *reinterpret_cast<uint32_t (*)[8]>(&c0[8]));
            tmem_ld_x8(tq + g * 24u + 16u, *reinterpret_cast<uint32_t (*)[8]>(&c0[16]));
            if (halves == 2u) {
                tmem_ld_x8(tq + nb + g * 24u, *reinterpret_cast<uint32_t (*)[8]>(&c1[0]));
                tmem_ld_x8(tq + nb + g * 24u + 8u, *reinterpret_cast<uint32_t (*)[8]>(&c1[8]));
                tmem_ld_x8(tq + nb + g * 24u + 16u, *reinterpret_cast<uint32_t (*)[8]>(&c1[16]));
            }
            tmem_ld_wait();
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const uint32_t m = g * 4u + r;
                if (m >= p.M)
                    break;
                const float f1 = __uint_as_float(lds32(rs_smem + 8u * m)), f2 = __uint_as_float(lds32(rs_smem + 8u * m + 4u));
                const float a0 = mx_row_sum(c0, r) * f1 * f2;
                const float a1 = halves == 2u ? mx_row_sum(c1, r) * f1 * f2 : 0.0f;
                if constexpr (GLU) {
                    /* half 0 = plane 0 of the pair, half 1 = plane 1; one output per thread */
                    const uint32_t n = row0 + lr;
                    const bool ok = lr < cnt0 && n < p.N;
                    if (direct) {
                        if (ok)
                            mx_store_all(p, m, n, glu_out_bf16(p.gate_plane ? a1 : a0, p.gate_plane ? a0 : a1,
                                                               p.gs, p.gs_up));
                    } else if (ok) {
                        __stcg(mine + static_cast<size_t>(m) * pitch + blockIdx.x * 256u + lr, a0);
                        __stcg(mine + static_cast<size_t>(m) * pitch + blockIdx.x * 256u + 128u + lr, a1);
                    }
                } else {
#pragma unroll
                    for (uint32_t h = 0; h < 2u; h++) {
                        if (h >= halves)
                            break;
                        const uint32_t n = row0 + h * 128u + lr;
                        const float a = h ? a1 : a0;
                        if (lr >= (h ? cnt1 : cnt0) || n >= p.N)
                            continue;
                        if (direct) {
                            __nv_bfloat16 hv = __float2bfloat16_rn(a * p.gs);
                            mx_store_all(p, m, n, *reinterpret_cast<uint16_t *>(&hv));
                        } else {
                            __stcg(mine + static_cast<size_t>(m) * pitch + n, a);
                        }
                    }
                }
            }
        }
        if (!direct) {
            /* split-K: the CTA of a row tile that arrives last adds the slices in
             * ascending order (results do not depend on scheduling) */
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tid == 64u) {
                __threadfence();
                const unsigned ticket = atomicAdd(p.counters + blockIdx.x, 1u);
                __threadfence();
                sts32(last_flag, (ticket == p.split_k - 1u) ? 1u : 0u);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (lds32(last_flag)) {
                const size_t slice = static_cast<size_t>(groups * 4u) * pitch;
                /* column of this thread's two outputs in a partial row, and whether they exist */
                const uint32_t col0 = GLU ? blockIdx.x * 256u + lr : row0 + lr, col1 = col0 + 128u;
                const bool ok0 = lr < cnt0 && row0 + lr < p.N;
                const bool ok1 = GLU ? ok0 : (lr < cnt1 && row0 + 128u + lr < p.N);
                /* four activation rows x eight slices x two halves of loads in flight, added
                 * slice by slice in ascending order */
                for (uint32_t m0 = 0; m0 < p.M; m0 += 4u) {
                    float s0[4] = { 0.0f, 0.0f, 0.0f, 0.0f }, s1[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
                    for (uint32_t sl0 = 0; sl0 < p.split_k; sl0 += 8u) {
                        float v0[4][8], v1[4][8];
#pragma unroll
                        for (uint32_t r = 0; r < 4u; r++)
#pragma unroll
                            for (uint32_t u = 0; u < 8u; u++) {
                                const bool live = m0 + r < p.M && sl0 + u < p.split_k;
                                const float *src = p.partial + (sl0 + u) * slice + static_cast<size_t>(m0 + r) * pitch;
                                v0[r][u] = live && ok0 ? __ldcg(src + col0) : 0.0f;
                                v1[r][u] = live && ok1 ? __ldcg(src + col1) : 0.0f;
                            }
#pragma unroll
                        for (uint32_t r = 0; r < 4u; r++)
#pragma unroll
                            for (uint32_t u = 0; u < 8u; u++) {
                                s0[r] += v0[r][u];
                                s1[r] += v1[r][u];
                            }
                    }
#pragma unroll
                    for (uint32_t r = 0; r < 4u; r++) {
                        const uint32_t m = m0 + r;
                        if (m >= p.M)
                            break;
                        if constexpr (GLU) {
                            if (ok0)
                                mx_store_all(p, m, row0 + lr, glu_out_bf16(p.gate_plane ? s1[r] : s0[r],
                                                                           p.gate_plane ? s0[r] : s1[r], p.gs, p.gs_up));
                        } else {
                            if (ok0) {
                                __nv_bfloat16 hv = __float2bfloat16_rn(s0[r] * p.gs);
                                mx_store_all(p, m, row0 + lr, *reinterpret_cast<uint16_t *>(&hv));
                            }
                            if (ok1) {
                                __nv_bfloat16 hv = __float2bfloat16_rn(s1[r] * p.gs);
                                mx_store_all(p, m, row0 + 128u + lr, *reinterpret_cast<uint16_t *>(&hv));
                            }
                        }
                    }
                }
                if (tid == 64u)
                    p.counters[blockIdx.x] = 0u;
            }
        }
    }

done:
    if (warp == 2u && lane == 0) MX_TRACE(11, 2);
    tc_fence_before();
    __syncthreads();
    if (tid == 0) MX_TRACE(11, 3);
    TL_MARK(4);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512u);
    }
}

static void fill_desc(TmaDesc &d, const unsigned char *src) { memcpy(d.bytes, src, 128); }

template <bool GLU>
static int launch_mx(const mmb_args *a, unsigned *status, cudaStream_t st)
{
    MxParams p;
    if (a->n_dst) {
        for (uint32_t d = 0; d < a->n_dst; d++) p.y[d] = static_cast<uint16_t *>(a->y_dst[d]);
        p.n_dst = a->n_dst; p.ldy = a->ldy; p.col0 = a->col0;
    } else {
        p.y[0] = static_cast<uint16_t *>(a->y);
        p.n_dst = 1; p.ldy = a->N; p.col0 = 0;
    }
    unsigned char *ws = static_cast<unsigned char *>(a->ws);
    p.counters = reinterpret_cast<unsigned *>(ws);
    p.partial = reinterpret_cast<float *>(ws + a->mx_partial_off);
    p.row_scale = reinterpret_cast<const float *>(static_cast<const unsigned char *>(a->mx_x_ws) + MMB_MX_ROWSCALE_OFF);
    p.status = status;
    p.gs = a->gs; p.gs_up = a->gs_up;
    p.gate_plane = a->gate_plane ? 1u : 0u;
    p.M = a->M; p.K = a->K; p.N = a->N;
    p.k_steps = a->plan.k_steps; p.split_k = a->plan.split_k; p.stages = a->plan.stages;
    p.pdl = static_cast<uint32_t>(a->pdl);
    p.rows = a->plan.tile_n;
    p.nb = a->plan.tile_m;
    TmaDesc tp, ts, tx, tf;
    fill_desc(tp, a->tm_payload);
    fill_desc(ts, a->tm_scale);
    fill_desc(tx, a->tm_x);
    fill_desc(tf, a->tm_sfb);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a->plan.grid_x, a->plan.grid_y);
    cfg.blockDim = dim3(MMB_MX_THREADS);
    cfg.dynamicSmemBytes = a->plan.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = a->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, f4_mx_kernel<GLU>, tp, ts, tx, tf, p));
}

} // namespace mmb

#ifdef MMB_MX_TRACE
extern "C" int mmb_mx_timeline_read(unsigned long long *out, unsigned *n, int reset)
{
    cudaError_t e = cudaMemcpyFromSymbol(n, mmb::g_tl_n, sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out, mmb::g_tl, sizeof(unsigned long long) * 4 * 4096);
    if (e == cudaSuccess && reset) { unsigned z = 0; e = cudaMemcpyToSymbol(mmb::g_tl_n, &z, sizeof z); }
    return static_cast<int>(e);
}
extern "C" int mmb_mx_trace_read(long long *out)
{
    return static_cast<int>(cudaMemcpyFromSymbol(out, mmb::g_mx_trace, sizeof(long long) * 12 * 32));
}
#endif

extern "C" int mmb_mx_init(void)
{
    cudaError_t e = cudaFuncSetAttribute(mmb::f4_mx_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         MMB_SMEM_MAX);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(mmb::f4_mx_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMB_SMEM_MAX);
    return static_cast<int>(e);
}

/* Digit planes of the activations into the op's scratch (a->mx_x_ws). */
extern "C" int mmb_launch_xslice_rows(const void *x, void *scratch, uint32_t M, uint32_t K, uint32_t nb, int pdl,
                                      void *stream);

extern "C" int mmb_launch_xslice(const mmb_args *a, void *stream)
{
    /* rows up to 32768 long: one pass over the activations, a cluster per row */
    const int rc = mmb_launch_xslice_rows(a->x, a->mx_x_ws, a->M, a->K, a->plan.tile_m, a->pdl, stream);
    if (rc >= 0)
        return rc;
    mmb::XsliceParams p;
    unsigned char *xs = static_cast<unsigned char *>(a->mx_x_ws);
    const uint32_t m_pad = a->plan.tile_m / MMB_MX_PLANES;
    p.x = static_cast<const uint16_t *>(a->x);
    p.row_scale = reinterpret_cast<float *>(xs + MMB_MX_ROWSCALE_OFF);
    p.planes = xs + MMB_MX_PLANES_OFF;
    p.sfb = xs + MMB_MX_PLANES_OFF + MMB_MX_PLANES_B(a->plan.tile_m, a->K);
    p.M = a->M; p.K = a->K; p.m_pad = m_pad;
    p.pdl = static_cast<uint32_t>(a->pdl);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a->K / 4u + 255u) / 256u, m_pad);
    cfg.blockDim = dim3(256);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = a->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, mmb::f4_xslice_kernel, p));
}

extern "C" int mmb_launch_mx(const mmb_args *a, void *stream)
{
    unsigned *status = nullptr;
    int e = mmb_status_word(&status);
    if (e) return e;
    if (!a->ws || !a->mx_x_ws)
        return static_cast<int>(cudaErrorInvalidValue);
    if (a->plan.tile_n == 0 || a->plan.tile_n > 256u || a->plan.tile_n % (a->glu ? 16u : 4u) != 0 ||
        a->plan.tile_m == 0 || a->plan.tile_m % 24u != 0 || a->plan.tile_m > MMB_MX_MAX_NB)
        return static_cast<int>(cudaErrorInvalidValue);
    if (a->glu && a->n_dst)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return a->glu ? mmb::launch_mx<true>(a, status, st) : mmb::launch_mx<false>(a, status, st);
}
