/*
 * UMMA: the prefill kernel of the NVFP4 linear op (M > 32, tensor-bound).
 *
 * y[M][N] tile of BM x BN per CTA, accumulated in tensor memory by
 * tcgen05.mma kind::f16 (bf16 x bf16 -> fp32).  Activations stay bf16 in the
 * reference (src/kernels/cpu/cx.c:211), so the weights are dequantised to bf16
 * in shared memory; e2m1 x e4m3 fits a bf16 exactly, so every product the
 * tensor core forms is the reference's product.
 *
 * Warp roles (10 warps):
 *   warp 0      TMA producer: activation tile (BM x 64 bf16, 128-byte swizzle),
 *               packed payload (BN rows x 32 B per 64-wide K block) and block
 *               scales (BN rows x 16 B per 256-wide K group).
 *   warp 1      owns tensor memory; one lane issues the MMAs and commits.
 *   warps 2-9   dequantise (two groups of four warps, alternate K blocks): 16-byte
 *               shared load of 32 nibbles, unpack + scale
 *               in registers (fp4.cuh), 16-byte stores into the K-major
 *               swizzled B tile, fence.proxy.async, mbarrier hand-off to warp 1.
 *               After the K loop the same warps drain tensor memory:
 *               tcgen05.ld, times global scale, bf16, 16-byte global stores.
 *
 * Operand roles: A = activations (BM/128 tiles of 128 rows), B = weights
 * (BN rows), so accumulator lane = activation row and column = output
 * feature, which makes the epilogue's rows contiguous in y.
 *
 * Tail split.  Tiles are numbered activation tile fastest and one CTA takes one
 * tile, so a launch runs in waves of one CTA per SM.  The tiles of the last,
 * partial wave (plan.m_tiles of them) are cut into plan.split_k K slices each, a
 * CTA per slice, so that the tail fills the SMs too: a slice leaves its fp32
 * sums in the workspace and a second, small kernel (f4_umma_tail_kernel, the whole
 * GPU on a few tens of MB) adds the slices of every split tile in ascending order
 * and writes the outputs.  One CTA cannot do that addition at the end of the main
 * kernel: an SM takes in about 60 GB/s, i.e. 4 us per 256 KB slice.
 *
 * It replaces the one-thread-per-output kernel of the reference
 * (src/kernels/cuda/cx.cu:345-356) for the prefill regime; the design the
 * reference only sketches is "dequant + bf16 mma gemm"
 * (include/mimfer/plan.h:51-52).
 */
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

struct UmmaParams {
    uint16_t *y[MMB_MAX_PEERS];  /* destinations: own output, then peers' (tensor parallel) */
    uint32_t  n_dst, ldy, col0;   /* row pitch and column offset inside each destination */
    unsigned *status;
    float     gs;
    uint32_t  M, K, N;
    uint32_t  k_blocks;      /* K / 64 */
    uint32_t  stages;
    uint32_t  pdl;           /* MMB_PDL_* (INDEPENDENT is served as WAIT_FIRST)  */
    float     gs_up;         /* gated pair: scale of the up projection          */
    uint32_t  gate_plane;    /* gated pair: which half of the weight tile is the gate */
    uint32_t  m_tiles;       /* activation-row tiles (tile id = n_tile * m_tiles + m_tile) */
    uint32_t  full_tiles;    /* tiles that run whole; the ones after them are split      */
    uint32_t  splits;        /* K slices of every tile after full_tiles (>= 1)           */
    float    *partial;       /* [split tile][slice][half][32-column chunk][4-column group][128 rows][4] fp32 sums */
    uint32_t  stagger_ns, stagger_ctas;   /* tensor parallel: CTA i < stagger_ctas starts i / stagger_ctas of stagger_ns late */
};


/* One weight box.  Gated pair: a 3-D box brings BN/2 rows of each projection,
 * plane 0 first, so accumulator columns [0, BN/2) belong to plane 0. */
template <bool GLU>
__device__ __forceinline__ void load_w(uint32_t dst, const TmaDesc *map, uint32_t x, uint32_t row,
                                       uint32_t bar)
{
    if constexpr (GLU)
        tma_load_3d(dst, map, static_cast<int>(x), static_cast<int>(row), 0, bar);
    else
        tma_load_2d(dst, map, static_cast<int>(x), static_cast<int>(row), bar);
}

template <int BM, int BN, bool GLU>
__global__ void __launch_bounds__(MMB_UM_THREADS, 1)
f4_umma_kernel(const __grid_constant__ TmaDesc tm_x, const __grid_constant__ TmaDesc tm_payload,
               const __grid_constant__ TmaDesc tm_scale, const UmmaParams p)
{
    constexpr uint32_t A_B = MMB_UM_A_B(BM), B_B = MMB_UM_B_B(BN);
    constexpr uint32_t PAY_B = MMB_UM_PAY_B(BN), SC_B = MMB_UM_SC_B(BN);
    constexpr uint32_t HALVES = BM / 128;
    constexpr uint32_t PAY_SLOTS = MMB_UM_PAY_SLOTS(BN);
    constexpr uint32_t TMEM_COLS = HALVES * BN;              /* 128, 256 or 512 */
    constexpr uint32_t ITEMS = BN * 2 / (MMB_UM_DEQ_WARPS * 32);
    constexpr uint32_t IDESC = umma_idesc_bf16(128, BN);

    extern __shared__ unsigned char smem_raw[];
    const uint32_t ST = p.stages;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sm_a = base;
    const uint32_t sm_b = sm_a + ST * A_B;
    const uint32_t sm_pay = sm_b + ST * B_B;
    const uint32_t sm_sc = sm_pay + PAY_SLOTS * PAY_B;
    const uint32_t lut = sm_sc + MMB_UM_SC_SLOTS * SC_B;
    const uint32_t bars = lut + 1024u;
    /* barrier map (8 bytes each) */
    const uint32_t full_a = bars;                       /* [ST] TMA -> MMA              */
    const uint32_t full_b = full_a + 8u * ST;           /* [ST] dequant -> MMA          */
    const uint32_t empty_ab = full_b + 8u * ST;         /* [ST] MMA done -> TMA, dequant */
    const uint32_t full_pay = empty_ab + 8u * ST;       /* [PAY_SLOTS]                  */
    const uint32_t empty_pay = full_pay + 8u * PAY_SLOTS;
    const uint32_t full_sc = empty_pay + 8u * PAY_SLOTS;
    const uint32_t empty_sc = full_sc + 8u * MMB_UM_SC_SLOTS;
    const uint32_t accum_full = empty_sc + 8u * MMB_UM_SC_SLOTS;
    const uint32_t tmem_slot = accum_full + 8u;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    /* Tensor parallel: the epilogues store every tile to all ranks, and NVLink takes a
     * wave's tiles more slowly than the SMs make them.  CTAs that start together reach
     * their first epilogues together and share the link evenly; the first wave therefore
     * starts spread over the time the link needs for one wave's tiles, and later CTAs
     * inherit the spread.  Measured on four ranks: gate+up (3.7 waves) 0.86 -> 0.76 ms,
     * the LM head (32 waves, whose CTAs drift apart by themselves) 3.24 -> 3.20 ms. */
    if (p.stagger_ns && blockIdx.x < p.stagger_ctas) {
        if (tid == 0) {
            const uint64_t t0 = globaltimer_ns();
            const uint64_t late = static_cast<uint64_t>(p.stagger_ns) * blockIdx.x / p.stagger_ctas;
            while (globaltimer_ns() - t0 < late)
                __nanosleep(500);
        }
        __syncthreads();
    }
    /* activation-row tile fastest: the CTAs running together share a few weight
     * tiles (and all of x) through L2 instead of each streaming the whole weight */
    static_assert(!GLU || BN == 256, "the gated pair runs on 256-row weight tiles");
    /* n0: first weight row of the tile (of each projection, and the first output
     * column, for a gated pair) */
    uint32_t tile = blockIdx.x, slice = 0, n_slices = 1;
    if (tile >= p.full_tiles) {
        const uint32_t e = tile - p.full_tiles;
        tile = p.full_tiles + e / p.splits;
        slice = e % p.splits;
        n_slices = p.splits;
    }
    const uint32_t m0 = (tile % p.m_tiles) * BM, n0 = (tile / p.m_tiles) * (GLU ? BN / 2 : BN);
    /* this CTA's K blocks [kb0, kb0 + KB): slices are cut at 256-wide K groups (one scale box) */
    const uint32_t groups = p.k_blocks / 4u;
    const uint32_t kb0 = n_slices > 1 ? 4u * (groups * slice / n_slices) : 0u;
    const uint32_t KB = (n_slices > 1 ? 4u * (groups * (slice + 1u) / n_slices) : p.k_blocks) - kb0;
    const uint32_t pre_pay = KB < PAY_SLOTS ? KB : PAY_SLOTS;   /* payload boxes issued in the prologue */

    if (tid < 256u)
        sts32(lut + tid * 4u, scale_lut_entry(tid));
    if (tid == 0) {
        for (uint32_t s = 0; s < ST; s++) {
            mbar_init(full_a + 8u * s, 1u);
            mbar_init(full_b + 8u * s, MMB_UM_DEQ_WARPS / 2u);    /* a K block is prepared by four of the eight warps */
            mbar_init(empty_ab + 8u * s, 1u);
        }
        for (uint32_t s = 0; s < PAY_SLOTS; s++) {
            mbar_init(full_pay + 8u * s, 1u);
            mbar_init(empty_pay + 8u * s, MMB_UM_DEQ_WARPS / 2u);
        }
        for (uint32_t s = 0; s < MMB_UM_SC_SLOTS; s++) {
            mbar_init(full_sc + 8u * s, 1u);
            mbar_init(empty_sc + 8u * s, MMB_UM_DEQ_WARPS);
        }
        mbar_init(accum_full, 1u);
        mbar_fence_init();
        /* this thread is also the TMA producer: the first weight boxes go out now,
         * ahead of the table build, the TMEM allocation and the grid-dependency wait */
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_payload);
        tma_prefetch_desc(&tm_scale);
        for (uint32_t kb = 0; kb < pre_pay; kb++) {
            mbar_expect_tx(full_pay + 8u * kb, PAY_B);
            load_w<GLU>(sm_pay + kb * PAY_B, &tm_payload, (kb0 + kb) * 32u, n0, full_pay + 8u * kb);
        }
        mbar_expect_tx(full_sc, SC_B);
        load_w<GLU>(sm_sc, &tm_scale, (kb0 >> 2) * 16u, n0, full_sc);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    if (p.pdl == MMB_PDL_TRIGGER_FIRST)
        grid_dep_launch();

    if (warp == 0) {
        /* ------------------------------ TMA producer ---------------------- *
         * Weights do not depend on the previous kernel in the stream, the
         * activations may: the first payload and scale boxes went out in the
         * prologue, the first activation box follows the grid-dependency wait. */
        if (lane == 0) {
            grid_dep_wait();
            if (p.pdl >= MMB_PDL_WAIT_FIRST)
                grid_dep_launch();
            uint32_t s = 0, round = 0;                 /* A/B stage index and its use count */
            for (uint32_t kb = 0; kb < KB; kb++, s = (s + 1u == ST) ? 0u : s + 1u, round += (s == 0u)) {
                const uint32_t ps = kb % PAY_SLOTS;
                if ((kb & 3u) == 0 && kb > 0) {
                    const uint32_t grp = kb >> 2, ss = grp % MMB_UM_SC_SLOTS;
                    if (grp >= MMB_UM_SC_SLOTS)
                        mbar_wait(empty_sc + 8u * ss, ((grp / MMB_UM_SC_SLOTS) - 1u) & 1u, p.status);
                    mbar_expect_tx(full_sc + 8u * ss, SC_B);
                    load_w<GLU>(sm_sc + ss * SC_B, &tm_scale, ((kb0 >> 2) + grp) * 16u, n0, full_sc + 8u * ss);
                }
                if (kb >= pre_pay) {
                    mbar_wait(empty_pay + 8u * ps, ((kb / PAY_SLOTS) - 1u) & 1u, p.status);
                    mbar_expect_tx(full_pay + 8u * ps, PAY_B);
                    load_w<GLU>(sm_pay + ps * PAY_B, &tm_payload, (kb0 + kb) * 32u, n0, full_pay + 8u * ps);
                }
                if (round > 0)
                    mbar_wait(empty_ab + 8u * s, (round - 1u) & 1u, p.status);
                mbar_expect_tx(full_a + 8u * s, A_B);
                tma_load_2d(sm_a + s * A_B, &tm_x, static_cast<int>((kb0 + kb) * MMB_UM_KBLOCK),
                            static_cast<int>(m0), full_a + 8u * s);
            }
        }
    } else if (warp == 1) {
        /* ------------------------------ MMA issue -------------------------- */
        if (lane == 0) {
            uint32_t s = 0, round = 0;
            for (uint32_t kb = 0; kb < KB; kb++, s = (s + 1u == ST) ? 0u : s + 1u, round += (s == 0u)) {
                const uint32_t par = round & 1u;
                mbar_wait(full_a + 8u * s, par, p.status);
                mbar_wait(full_b + 8u * s, par, p.status);
                tc_fence_after();
#pragma unroll
                for (uint32_t k = 0; k < MMB_UM_KBLOCK / 16u; k++) {
                    const uint64_t bd = umma_desc_sw128(sm_b + s * B_B + k * 32u);
#pragma unroll
                    for (uint32_t h = 0; h < HALVES; h++) {
                        const uint64_t ad = umma_desc_sw128(sm_a + s * A_B + h * 16384u + k * 32u);
                        umma_bf16(tmem_base + h * BN, ad, bd, IDESC, (kb | k) ? 1u : 0u);
                    }
                }
                umma_commit(empty_ab + 8u * s);
            }
            umma_commit(accum_full);
        }
    } else {
        /* ------------------------------ dequantise -------------------------- */
        /* Two groups of four warps take alternate K blocks, so that the chain of one block
         * (shared loads, unpack, stores, proxy fence, hand-over) overlaps the other group's.
         * Measured against all eight warps on every block: 3 to 5 % on the 256 x 256 shapes
         * (down at M = 8192 1 312 -> 1 375 TFLOP/s), nothing on the short ones. */
        const uint32_t td = tid - 64u;                       /* 0..255 */
        const uint32_t grp2 = td >> 7, tg = td & 127u;       /* group, thread of the group */
        uint32_t s = 0, round = 0;
        for (uint32_t kb = 0; kb < KB; kb++, s = (s + 1u == ST) ? 0u : s + 1u, round += (s == 0u)) {
            if ((kb & 1u) != grp2)
                continue;
            const uint32_t ps = kb % PAY_SLOTS;
            const uint32_t grp = kb >> 2, ss = grp % MMB_UM_SC_SLOTS, j = kb & 3u;
            mbar_wait_warp(full_sc + 8u * ss, (grp / MMB_UM_SC_SLOTS) & 1u, p.status);
            mbar_wait_warp(full_pay + 8u * ps, (kb / PAY_SLOTS) & 1u, p.status);
            if (round > 0)
                mbar_wait_warp(empty_ab + 8u * s, (round - 1u) & 1u, p.status);
            const uint32_t pay = sm_pay + ps * PAY_B, scl = sm_sc + ss * SC_B;
            const uint32_t bt = sm_b + s * B_B;
#pragma unroll
            for (uint32_t item = 0; item < 2u * ITEMS; item++) {
                const uint32_t idx = tg + item * 128u;
                const uint32_t n = idx >> 1, half = idx & 1u;
                const uint4 raw = lds128(pay + n * 32u + half * 16u);
                const uint32_t sc2 = lds16(scl + n * 16u + j * 4u + half * 2u);
                const uint32_t c0 = lds32(lut + (sc2 & 255u) * 4u);
                const uint32_t c1 = lds32(lut + (sc2 >> 8) * 4u);
                const uint32_t rowb = bt + n * 128u, sw = n & 7u, ch = half * 4u;
                sts128(rowb + (((ch + 0u) ^ sw) << 4), unpack8_natural(raw.x, c0));
                sts128(rowb + (((ch + 1u) ^ sw) << 4), unpack8_natural(raw.y, c0));
                sts128(rowb + (((ch + 2u) ^ sw) << 4), unpack8_natural(raw.z, c1));
                sts128(rowb + (((ch + 3u) ^ sw) << 4), unpack8_natural(raw.w, c1));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full_b + 8u * s);
                mbar_arrive(empty_pay + 8u * ps);
                if (j >= 2u)                     /* this group's last K block of the scale group */
                    mbar_arrive(empty_sc + 8u * ss);
            }
        }

        /* ------------------------------ epilogue --------------------------- *
         * Each warp drains pieces of 32 rows x 128 columns: tensor memory ->
         * registers -> bf16 -> its own staging tile in shared memory (the
         * operand stages are free once every MMA has completed), then rows go
         * out as full 256-byte runs, two rows per warp store, once per
         * destination.  Whole 128-byte lines matter for the peer copies: the
         * stores cross NVLink as they are issued. */
        mbar_wait_warp(accum_full, 0u, p.status);
        tc_fence_after();
        const float out_scale = p.gs * 256.0f;      /* undo the 2^-8 of the operand form */
        const uint32_t quad = warp & 3u;            /* TMEM lanes this warp may read   */
        const uint32_t pair = (warp - 2u) >> 2;     /* two warps share a quadrant       */
        constexpr uint32_t TILE_F = BM * BN;        /* fp32 sums of one K slice         */
        const bool emit = n_slices == 1;
        if (!emit) {
            /* K slice of a split tile: leave the sums in the workspace (this warp's
             * quadrant of both halves, its half of the columns); the tail kernel adds
             * the slices and writes the output */
            const uint32_t st_idx = tile - p.full_tiles;
            float *mine = p.partial + (static_cast<size_t>(st_idx) * n_slices + slice) * TILE_F;
            /* layout of a slice: [half][32-column chunk][group of 4 columns][128 rows] float4, i.e.
             * the order tensor memory is read in: a warp's store is 512 contiguous bytes */
            for (uint32_t h = 0; h < HALVES; h++) {
                for (uint32_t c32 = pair * (BN / 64u); c32 < (pair + 1u) * (BN / 64u); c32++) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quad * 32u) << 16) + h * BN + c32 * 32u, r);
                    tmem_ld_wait();
                    float4 *dst = reinterpret_cast<float4 *>(mine) +
                                  static_cast<size_t>(h * (BN / 32u) + c32) * 8u * 128u + quad * 32u + lane;
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        __stcg(dst + j * 128, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                }
            }
        }
        if (!emit) {
            /* nothing to write: another CTA finishes this tile */
        } else if constexpr (GLU) {
            /* Gated pair: pieces of 32 rows x 64 outputs.  Gate and up sums of an
             * output sit 128 columns apart in the same lane; silu(gate) * up on
             * their bf16 roundings, staged, then 128-byte row runs go out, four
             * rows per warp store. */
            constexpr uint32_t GPITCH = 144u;       /* 128 B of data + 16 B */
            const float s_gate = p.gs * 256.0f, s_up = p.gs_up * 256.0f;
            const uint32_t gstg = sm_a + (warp - 2u) * (32u * GPITCH);
            const uint32_t gcol = p.gate_plane ? BN / 2 : 0u, ucol = p.gate_plane ? 0u : BN / 2;
            const bool gvec = (p.N % 8u) == 0;
            for (uint32_t c = pair; c < HALVES * 2u; c += 2u) {
                const uint32_t h = c >> 1, cc = c & 1u;
#pragma unroll
                for (uint32_t q = 0; q < 2; q++) {
                    uint32_t a[32], b[32];
                    const uint32_t col = tmem_base + ((quad * 32u) << 16) + h * BN + cc * 64u + q * 32u;
                    tmem_ld_32x32(col + gcol, a);
                    tmem_ld_32x32(col + ucol, b);
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            w[e] = glu_out_bf16x2(__uint_as_float(a[8 * v + 2 * e]),
                                                  __uint_as_float(a[8 * v + 2 * e + 1]),
                                                  __uint_as_float(b[8 * v + 2 * e]),
                                                  __uint_as_float(b[8 * v + 2 * e + 1]), s_gate, s_up);
                        sts128(gstg + lane * GPITCH + q * 64u + v * 16u, make_uint4(w[0], w[1], w[2], w[3]));
                    }
                }
                __syncwarp();
                const uint32_t sub = lane >> 3, col8 = lane & 7u;     /* 4 rows x 8 chunks per store */
                const uint32_t n = n0 + cc * 64u + col8 * 8u;
#pragma unroll 4
                for (uint32_t rr = 0; rr < 32u; rr += 4u) {
                    const uint32_t row = rr + sub;
                    const uint32_t m = m0 + h * 128u + quad * 32u + row;
                    if (m < p.M && n < p.N) {
                        const uint4 o = lds128(gstg + row * GPITCH + col8 * 16u);
                        const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n;
                        if (gvec) {
                            for (uint32_t d = 0; d < p.n_dst; d++)
                                *reinterpret_cast<uint4 *>(p.y[d] + off) = o;
                        } else {
                            const uint32_t w4[4] = { o.x, o.y, o.z, o.w };
                            for (uint32_t e = 0; e < 8u && n + e < p.N; e++)
                                for (uint32_t d = 0; d < p.n_dst; d++)
                                    p.y[d][off + e] = static_cast<uint16_t>(w4[e >> 1] >> (16u * (e & 1u)));
                        }
                    }
                }
                __syncwarp();
            }
        } else {
            /* One piece per warp: 32 rows of one 128-row half, and as many columns as make
             * the two warps of a quadrant equal (all BN columns when the tile has two halves).
             * A row of a piece leaves as one run of up to 512 bytes: measured on four GPUs, all
             * storing to all, NVLink carried tiles written in 256-byte runs at 568 GB/s per GPU
             * and in 512-byte runs at 617. */
            constexpr uint32_t CG = HALVES == 2 ? 1u : 2u;         /* column groups of a tile */
            constexpr uint32_t W = BN / CG;                        /* columns of a piece: 256, 128 or 64 */
            constexpr uint32_t PITCH = W * 2u + 16u;               /* + 16 B: conflict-free both ways */
            static_assert(MMB_UM_DEQ_WARPS * 32u * PITCH <= 2u * (A_B + B_B) + PAY_SLOTS * PAY_B,
                          "the staging tiles lie in the operand stages (at least two) and the payload slots");
            const uint32_t stg = sm_a + (warp - 2u) * (32u * PITCH);
            const bool vec_ok = (p.N % 8u) == 0;
            /* Tensor parallel: every lane hands its finished row to the bulk-copy engine, once
             * per destination (plain stores to the peers and the engine ended at the same time:
             * the link is the limit, not the way the SM feeds it). */
            const bool bulk = p.n_dst > 1u && vec_ok && ((p.ldy | p.col0) & 7u) == 0u;
            const uint32_t h = pair / CG, cc = pair % CG;
            const uint32_t n_base = n0 + cc * W;
#pragma unroll
            for (uint32_t q = 0; q < W / 32u; q++) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((quad * 32u) << 16) + h * BN + cc * W + q * 32u, r);
                tmem_ld_wait();
#pragma unroll
                for (int v = 0; v < 4; v++) {
                    uint4 o;
                    o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]) * out_scale,
                                      __uint_as_float(r[8 * v + 1]) * out_scale);
                    o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]) * out_scale,
                                      __uint_as_float(r[8 * v + 3]) * out_scale);
                    o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]) * out_scale,
                                      __uint_as_float(r[8 * v + 5]) * out_scale);
                    o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]) * out_scale,
                                      __uint_as_float(r[8 * v + 7]) * out_scale);
                    sts128(stg + lane * PITCH + q * 64u + v * 16u, o);
                }
            }
            if (bulk) {
                fence_proxy_async_smem();                    /* the row this lane wrote, for the copy engine */
                const uint32_t m = m0 + h * 128u + quad * 32u + lane;
                const uint32_t cols = n_base < p.N ? (p.N - n_base < W ? p.N - n_base : W) : 0u;
                if (m < p.M && cols) {
                    const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n_base;
                    for (uint32_t d = 0; d < p.n_dst; d++)
                        bulk_store(p.y[d] + off, stg + lane * PITCH, cols * 2u);
                }
                bulk_commit();
            } else {
                __syncwarp();
                constexpr uint32_t PER_ROW = W / 8u;             /* 16-byte chunks of a row: 32, 16 or 8 lanes */
                const uint32_t sub = lane / PER_ROW, chunk = lane % PER_ROW;
                const uint32_t n = n_base + chunk * 8u;
#pragma unroll 4
                for (uint32_t rr = 0; rr < 32u; rr += 32u / PER_ROW) {
                    const uint32_t row = rr + sub;
                    const uint32_t m = m0 + h * 128u + quad * 32u + row;
                    if (m < p.M && n < p.N) {
                        const uint4 o = lds128(stg + row * PITCH + chunk * 16u);
                        const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n;
                        if (vec_ok) {
                            for (uint32_t d = 0; d < p.n_dst; d++)
                                *reinterpret_cast<uint4 *>(p.y[d] + off) = o;
                        } else {
                            const uint32_t w4[4] = { o.x, o.y, o.z, o.w };
                            for (uint32_t e = 0; e < 8u && n + e < p.N; e++)
                                for (uint32_t d = 0; d < p.n_dst; d++)
                                    p.y[d][off + e] = static_cast<uint16_t>(w4[e >> 1] >> (16u * (e & 1u)));
                        }
                    }
                }
            }
            if (bulk)
                bulk_wait_all();                             /* before the CTA gives up its shared memory */
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

/* ---- the split tiles' outputs ----------------------------------------------------
 * One CTA per (split tile, 128-row half, 32 output columns).  A thread owns 16 columns of
 * one row: it adds the K slices' sums in ascending order (four 16-byte loads per slice,
 * lanes along the rows, which is how the slices were stored), applies the epilogue of the
 * main kernel and puts its 32 bytes into a shared tile; the tile then goes out as 64-byte
 * row runs to every destination. */
struct UmmaTailParams {
    uint16_t    *y[MMB_MAX_PEERS];
    uint32_t     n_dst, ldy, col0;
    const float *partial;
    float        gs, gs_up;
    uint32_t     gate_plane, glu;
    uint32_t     M, N;
    uint32_t     bm, bn;            /* tile */
    uint32_t     m_tiles, full_tiles, splits, pdl;
};

__global__ void __launch_bounds__(256) f4_umma_tail_kernel(const UmmaTailParams p)
{
    __shared__ __align__(16) uint16_t tile_s[128][40];         /* 32 columns + 8 of padding per row */
    grid_dep_launch();
    if (p.pdl != MMB_PDL_OFF)
        grid_dep_wait();                         /* the main kernel's partial sums */
    const uint32_t chunks = p.bn / 32u;                        /* 32-column chunks of the accumulators */
    const uint32_t out_chunks = p.glu ? chunks / 2u : chunks;
    const uint32_t h = blockIdx.x / out_chunks, oc = blockIdx.x % out_chunks;
    const uint32_t st_idx = blockIdx.y, tile = p.full_tiles + st_idx;
    const uint32_t row = threadIdx.x & 127u, jh = threadIdx.x >> 7;      /* row of the half; columns 16 * jh .. + 15 */
    const size_t slice_f4 = static_cast<size_t>(p.bm) * p.bn / 4u;
    const float4 *base = reinterpret_cast<const float4 *>(p.partial) + static_cast<size_t>(st_idx) * p.splits * slice_f4;
    /* chunk of the first operand (the only one, or the gate's) and of the up projection */
    const uint32_t gate_off = p.glu && p.gate_plane ? chunks / 2u : 0u, up_off = p.glu && !p.gate_plane ? chunks / 2u : 0u;
    const size_t ia = (static_cast<size_t>(h * chunks + gate_off + oc) * 8u + jh * 4u) * 128u + row;
    const size_t ib = (static_cast<size_t>(h * chunks + up_off + oc) * 8u + jh * 4u) * 128u + row;
    float a[16], b[16];
#pragma unroll
    for (int i = 0; i < 16; i++) a[i] = b[i] = 0.0f;
    for (uint32_t s0 = 0; s0 < p.splits; s0 += 2u) {
        float4 va[2][4], vb[2][4];
#pragma unroll
        for (uint32_t j = 0; j < 2u; j++) {
            const float4 *sl = base + static_cast<size_t>(s0 + j < p.splits ? s0 + j : s0) * slice_f4;
#pragma unroll
            for (uint32_t q = 0; q < 4u; q++) {
                va[j][q] = __ldcg(sl + ia + q * 128u);
                vb[j][q] = p.glu ? __ldcg(sl + ib + q * 128u) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < 2u; j++) {
            if (s0 + j >= p.splits)
                break;
#pragma unroll
            for (uint32_t q = 0; q < 4u; q++) {
                a[4 * q] += va[j][q].x; a[4 * q + 1] += va[j][q].y; a[4 * q + 2] += va[j][q].z; a[4 * q + 3] += va[j][q].w;
                b[4 * q] += vb[j][q].x; b[4 * q + 1] += vb[j][q].y; b[4 * q + 2] += vb[j][q].z; b[4 * q + 3] += vb[j][q].w;
            }
        }
    }
    uint32_t o[8];
    if (p.glu) {
        const float sg = p.gs * 256.0f, su = p.gs_up * 256.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = glu_out_bf16x2(a[2 * i], a[2 * i + 1], b[2 * i], b[2 * i + 1], sg, su);
    } else {
        const float sc = p.gs * 256.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = pack_bf16x2(a[2 * i] * sc, a[2 * i + 1] * sc);
    }
    *reinterpret_cast<uint4 *>(&tile_s[row][jh * 16u]) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4 *>(&tile_s[row][jh * 16u + 8u]) = make_uint4(o[4], o[5], o[6], o[7]);
    __syncthreads();
    /* 128 rows x 64 bytes: four threads per row, two rows of the tile per thread */
    const uint32_t m0 = (tile % p.m_tiles) * p.bm + h * 128u;
    const uint32_t n0 = (tile / p.m_tiles) * (out_chunks * 32u) + oc * 32u;
#pragma unroll
    for (uint32_t k = 0; k < 2u; k++) {
        const uint32_t idx = threadIdx.x + k * 256u, r = idx >> 2, piece = idx & 3u;
        const uint32_t m = m0 + r, n = n0 + piece * 8u;
        if (m >= p.M || n >= p.N)
            continue;
        const uint4 v = *reinterpret_cast<const uint4 *>(&tile_s[r][piece * 8u]);
        const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n;
        for (uint32_t d = 0; d < p.n_dst; d++)
            *reinterpret_cast<uint4 *>(p.y[d] + off) = v;
    }
}

template <int BM, int BN, bool GLU>
static int launch_tile(const mmb_args *a, unsigned *status, cudaStream_t st)
{
    UmmaParams p = {};
    if (a->n_dst) {
        for (uint32_t d = 0; d < a->n_dst; d++) p.y[d] = static_cast<uint16_t *>(a->y_dst[d]);
        p.n_dst = a->n_dst; p.ldy = a->ldy; p.col0 = a->col0;
    } else {
        p.y[0] = static_cast<uint16_t *>(a->y);
        p.n_dst = 1; p.ldy = a->N; p.col0 = 0;
    }
    p.status = status;
    p.gs = a->gs;
    p.M = a->M; p.K = a->K; p.N = a->N;
    p.k_blocks = a->plan.k_steps;
    p.stages = a->plan.stages;
    p.gs_up = a->gs_up;
    p.gate_plane = a->gate_plane ? 1u : 0u;
    p.pdl = static_cast<uint32_t>(a->pdl);
    p.stagger_ns = a->stagger_ns;
    p.stagger_ctas = a->stagger_ctas;
    const uint32_t tiles = a->plan.grid_x * a->plan.grid_y;
    const bool split = a->plan.split_k > 1 && a->plan.m_tiles > 0 && a->plan.m_tiles <= tiles && a->ws;
    p.m_tiles = a->plan.grid_y;
    p.splits = split ? a->plan.split_k : 1u;
    p.full_tiles = split ? tiles - a->plan.m_tiles : tiles;
    p.partial = a->ws ? reinterpret_cast<float *>(static_cast<unsigned char *>(a->ws) + MMB_WS_COUNTER_B) : nullptr;
    TmaDesc tx, tp, ts;
    memcpy(tx.bytes, a->tm_x, 128);
    memcpy(tp.bytes, a->tm_payload, 128);
    memcpy(ts.bytes, a->tm_scale, 128);
    cudaLaunchConfig_t cfg = {};
    /* tile id = weight tile * activation tiles + activation tile; split tiles last */
    cfg.gridDim = dim3(p.full_tiles + (tiles - p.full_tiles) * p.splits);
    cfg.blockDim = dim3(MMB_UM_THREADS);
    cfg.dynamicSmemBytes = a->plan.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = a->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, f4_umma_kernel<BM, BN, GLU>, tx, tp, ts, p);
    if (err != cudaSuccess || !split)
        return static_cast<int>(err);
    UmmaTailParams t;
    for (uint32_t d = 0; d < MMB_MAX_PEERS; d++) t.y[d] = p.y[d];
    t.n_dst = p.n_dst; t.ldy = p.ldy; t.col0 = p.col0;
    t.partial = p.partial;
    t.gs = p.gs; t.gs_up = p.gs_up; t.gate_plane = p.gate_plane; t.glu = GLU ? 1u : 0u;
    t.M = p.M; t.N = p.N; t.bm = BM; t.bn = BN;
    t.m_tiles = p.m_tiles; t.full_tiles = p.full_tiles; t.splits = p.splits;
    t.pdl = p.pdl;
    cudaLaunchConfig_t tc = {};
    tc.gridDim = dim3((BM / 128u) * ((GLU ? BN / 2 : BN) / 32u), tiles - p.full_tiles);
    tc.blockDim = dim3(256);
    tc.stream = st;
    tc.attrs = attr;
    tc.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&tc, f4_umma_tail_kernel, t));
}

template <int BM, int BN, bool GLU>
static int set_smem()
{
    return static_cast<int>(cudaFuncSetAttribute(f4_umma_kernel<BM, BN, GLU>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 MMB_SMEM_MAX));
}

} // namespace mmb

extern "C" int mmb_umma_init(void)
{
    int e;
    if ((e = mmb::set_smem<256, 256, false>())) return e;
    if ((e = mmb::set_smem<128, 256, false>())) return e;
    if ((e = mmb::set_smem<128, 128, false>())) return e;
    if ((e = mmb::set_smem<256, 256, true>())) return e;
    return mmb::set_smem<128, 256, true>();
}

extern "C" int mmb_launch_umma(const mmb_args *a, void *stream)
{
    unsigned *status = nullptr;
    int e = mmb_status_word(&status);
    if (e) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t bm = a->plan.tile_m, bn = a->plan.tile_n;
    if (a->glu) {
        if (bm == 256 && bn == 256) return mmb::launch_tile<256, 256, true>(a, status, st);
        if (bm == 128 && bn == 256) return mmb::launch_tile<128, 256, true>(a, status, st);
        return static_cast<int>(cudaErrorInvalidValue);
    }
    if (bm == 256 && bn == 256) return mmb::launch_tile<256, 256, false>(a, status, st);
    if (bm == 128 && bn == 256) return mmb::launch_tile<128, 256, false>(a, status, st);
    if (bm == 128 && bn == 128) return mmb::launch_tile<128, 128, false>(a, status, st);
    return static_cast<int>(cudaErrorInvalidValue);
}
