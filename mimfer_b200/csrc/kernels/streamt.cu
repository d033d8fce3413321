/*
 * STREAM-T: decode kernel of the NVFP4 linear op on the tcgen05 tensor core
 * (M <= 32, HBM-bound).  Same job and same decomposition as stream.cu (one CTA
 * = 256 weight rows x a range of 256-wide K steps, TMA ring, split-K through
 * the workspace) but the multiply-accumulate moves from warp MMAs with
 * register accumulators to tcgen05.mma with the *weights* as the A operand in
 * tensor memory:
 *
 *   thread <-> weight row.  A dequant thread reads 32 bytes of its row's
 *   payload (64 nibbles) and 4 scale bytes from shared memory, unpacks in
 *   registers (fp4.cuh) and writes the 64 fp16/bf16 values straight into tensor
 *   memory with tcgen05.st (row = TMEM lane, two values per 32-bit column).
 *   No dequantised weight ever touches shared memory, so shared-memory traffic
 *   stays at the packed bytes.
 *   A single thread issues tcgen05.mma.kind::f16 with A = [128 rows x 16] from
 *   tensor memory, B = the activations ([16 or 32 rows] x 16, K-major, 128-byte
 *   swizzle, straight from TMA), D = [128 rows x 16/32] fp32 in tensor memory.
 *   Nothing per weight is left on the CUDA cores except the unpack itself.
 *
 * Operand format per K step as in stream.cu: fp16 when every activation of the
 * step converts to fp16 exactly (transform warps convert the TMA-delivered
 * bf16 slice in place), bf16 otherwise; both are exact, both add into the same
 * accumulators.
 *
 * Tensor memory map (512 columns allocated): two accumulators for each of the
 * two 128-row tiles at columns [0, 128) (consecutive MMAs alternate between them,
 * so none waits for the previous one's accumulate); three A slots of 128 columns
 * each (2 tiles x 64 columns = 128 K values per row) at [128, 512).  A slot holds
 * half a K step.
 *
 * It replaces the one-thread-per-output kernel of the reference
 * (src/kernels/cuda/cx.cu:345-356) for the decode regime.
 */
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

struct StreamTParams {
    uint16_t *y[MMB_MAX_PEERS];    /* destinations: own output, then peers' (tensor parallel) */
    uint32_t  n_dst, ldy, col0;
    float    *partial;             /* workspace + MMB_WS_COUNTER_B, or NULL */
    unsigned *counters;            /* workspace base, or NULL               */
    unsigned *status;
    float     gs;
    uint32_t  M, K, N;
    uint32_t  k_steps, split_k, stages;
};

constexpr uint32_t ST_NACC = 2u;           /* independent accumulators per tile: consecutive MMAs
                                              never chain on one accumulator; summed in order at the end */
constexpr uint32_t ST_D_COL = 0u;          /* accumulator a of tile t at (t * ST_NACC + a) * NPAD, <= 128 columns */
constexpr uint32_t ST_A_COL = 128u;        /* A slot s, tile t at ST_A_COL + s * 128 + t * 64 */
constexpr uint32_t ST_A_SLOTS = 3u;        /* each holds half a K step for both tiles */
constexpr uint32_t ST_TMEM_COLS = 512u;

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
/* D[tmem] (+)= A[tmem] * B[smem]^T, one CTA, both operands fp16 or both bf16. */
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
/* kind::f16 descriptor: fp32 accumulate, K-major B, both operands fp16 (0) or bf16 (1). */
__host__ __device__ constexpr uint32_t umma_idesc_16(uint32_t m, uint32_t n, uint32_t fmt)
{
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

/* 0xffffffff when both bf16 halves of u convert to fp16 exactly. */
__device__ __forceinline__ uint32_t t_fp16_exact_mask(uint32_t u)
{
    const __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&u));
    const __nv_bfloat162 hi = __float2bfloat162_rn(65536.0f);
    const __nv_bfloat162 lo = __float2bfloat162_rn(7.62939453125e-06f);       /* 2^-17 */
    const __nv_bfloat162 zero = __float2bfloat162_rn(0.0f);
    return __hlt2_mask(a, hi) & (__hge2_mask(a, lo) | __heq2_mask(a, zero));
}
__device__ __forceinline__ uint32_t t_bf16x2_to_f16x2(uint32_t u)
{
    const __half2 h = __floats2half2_rn(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    return *reinterpret_cast<const uint32_t *>(&h);
}

/* 64 weights of one row (two 16-byte payload chunks, four scale entries) -> 32
 * packed operand registers in column order. */
template <bool HALF>
__device__ __forceinline__ void dequant64(const uint4 &p0, const uint4 &p1, const uint32_t (&c)[4],
                                          uint32_t (&out)[32])
{
    const uint32_t w[8] = { p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w };
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint4 q;
        if (HALF) {
            q = unpack8_natural_f16(w[i], c[i >> 1]);
        } else {
            q = unpack8_natural(w[i], c[i >> 1]);       /* value * scale * 2^-8 ... */
            q.x = mul_bf16x2(q.x, 0x43804380u);         /* ... times 256: exact      */
            q.y = mul_bf16x2(q.y, 0x43804380u);
            q.z = mul_bf16x2(q.z, 0x43804380u);
            q.w = mul_bf16x2(q.w, 0x43804380u);
        }
        out[4 * i + 0] = q.x; out[4 * i + 1] = q.y; out[4 * i + 2] = q.z; out[4 * i + 3] = q.w;
    }
}

template <int NPAD>                      /* activation rows padded to 16 or 32 */
__global__ void __launch_bounds__(MMB_STT_THREADS, 1)
f4_streamt_kernel(const __grid_constant__ TmaDesc tm_payload,
                  const __grid_constant__ TmaDesc tm_scale, const __grid_constant__ TmaDesc tm_x,
                  const StreamTParams p)
{
    constexpr uint32_t X_B = NPAD * 512u;                  /* four [NPAD x 128 B] sub-tiles */
    constexpr uint32_t STAGE_B = MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B + X_B;
    constexpr uint32_t XFORM_THREADS = MMB_STT_XFORM_WARPS * 32u;
    constexpr uint32_t X_ITEMS = NPAD * 32u / XFORM_THREADS;   /* 16-byte chunks per transform thread */
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t lut_bf = base + p.stages * STAGE_B;
    const uint32_t lut_hf = lut_bf + 1024u;
    const uint32_t bar_raw = lut_hf + 1024u;               /* [stages] TMA landed                 */
    const uint32_t bar_x = bar_raw + 8u * p.stages;        /* [stages] activations converted       */
    const uint32_t bar_empty = bar_x + 8u * p.stages;      /* [stages] MMAs of the stage complete  */
    const uint32_t a_full = bar_empty + 8u * p.stages;     /* [slots] A slot written               */
    const uint32_t a_empty = a_full + 8u * ST_A_SLOTS;     /* [slots] A slot consumed              */
    const uint32_t accum_full = a_empty + 8u * ST_A_SLOTS;
    const uint32_t fmt_flag = accum_full + 8u;             /* [stages] 1 = fp16 step               */
    const uint32_t tmem_slot = fmt_flag + 4u * p.stages;
    const uint32_t last_flag = tmem_slot + 4u;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t row0 = blockIdx.x * MMB_ST_ROWS;
    const uint32_t ks_begin = static_cast<uint32_t>(
        static_cast<uint64_t>(p.k_steps) * blockIdx.y / p.split_k);
    const uint32_t ks_end = static_cast<uint32_t>(
        static_cast<uint64_t>(p.k_steps) * (blockIdx.y + 1) / p.split_k);
    const uint32_t nsteps = ks_end - ks_begin;

    const uint32_t stage_bytes = MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B + X_B;
    const uint32_t first = nsteps < p.stages ? nsteps : p.stages;   /* steps of the first ring */
    if (tid < 256u) {
        sts32(lut_bf + tid * 4u, scale_lut_entry(tid));
        sts32(lut_hf + tid * 4u, scale_lut_entry_f16(tid));
    }
    if (tid == MMB_STT_DEQ_WARPS * 32u) {
        /* the issuing thread sets the barriers up itself and starts the weight
         * stream at once */
        tma_prefetch_desc(&tm_payload);
        tma_prefetch_desc(&tm_scale);
        tma_prefetch_desc(&tm_x);
        for (uint32_t s = 0; s < p.stages; s++) {
            mbar_init(bar_raw + 8u * s, 1u);
            mbar_init(bar_x + 8u * s, XFORM_THREADS);
            mbar_init(bar_empty + 8u * s, 2u);                 /* one commit per issuing thread */
        }
        for (uint32_t s = 0; s < ST_A_SLOTS; s++) {
            mbar_init(a_full + 8u * s, MMB_STT_DEQ_WARPS);
            mbar_init(a_empty + 8u * s, 2u);
        }
        mbar_init(accum_full, 2u);
        mbar_fence_init();
        for (uint32_t it = 0; it < first; it++) {
            const uint32_t stage = base + it * STAGE_B, ks = ks_begin + it;
            mbar_expect_tx(bar_raw + 8u * it, stage_bytes);
            tma_load_2d(stage, &tm_payload, static_cast<int>(ks * 128u),
                        static_cast<int>(row0), bar_raw + 8u * it);
            tma_load_2d(stage + MMB_ST_PAYLOAD_B, &tm_scale, static_cast<int>(ks * 16u),
                        static_cast<int>(row0), bar_raw + 8u * it);
        }
    }
    if (warp == MMB_STT_DEQ_WARPS + 1u) {                  /* the MMA warp owns tensor memory */
        tmem_alloc(tmem_slot, ST_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    grid_dep_launch();

    if (warp == MMB_STT_DEQ_WARPS) {
        /* ------------------------------ TMA issue ---------------------------- *
         * Weights first (they do not depend on the previous kernel), then the
         * grid-dependency wait, then the activations. */
        if (lane == 0) {
            grid_dep_wait();
            for (uint32_t it = 0; it < first; it++)
#pragma unroll
                for (uint32_t sub = 0; sub < 4u; sub++)
                    tma_load_2d(base + it * STAGE_B + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B + sub * (NPAD * 128u),
                                &tm_x, static_cast<int>((ks_begin + it) * MMB_ST_KSTEP + sub * 64u), 0,
                                bar_raw + 8u * it);
            uint32_t s = 0, round = 1;
            for (uint32_t it = first; it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u,
                                                   round += (s == 0u)) {
                const uint32_t stage = base + s * STAGE_B, ks = ks_begin + it;
                mbar_wait(bar_empty + 8u * s, (round - 1u) & 1u, p.status);
                fence_proxy_async_smem();
                mbar_expect_tx(bar_raw + 8u * s, stage_bytes);
                tma_load_2d(stage, &tm_payload, static_cast<int>(ks * 128u),
                            static_cast<int>(row0), bar_raw + 8u * s);
                tma_load_2d(stage + MMB_ST_PAYLOAD_B, &tm_scale, static_cast<int>(ks * 16u),
                            static_cast<int>(row0), bar_raw + 8u * s);
#pragma unroll
                for (uint32_t sub = 0; sub < 4u; sub++)
                    tma_load_2d(stage + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B + sub * (NPAD * 128u), &tm_x,
                                static_cast<int>(ks * MMB_ST_KSTEP + sub * 64u), 0, bar_raw + 8u * s);
            }
        }
    } else if (warp == MMB_STT_DEQ_WARPS + 1u || warp == MMB_STT_DEQ_WARPS + 2u) {
        /* ------------------------------ MMA issue ----------------------------- *
         * Two issuing threads, one per 128-row tile: a single thread's serial
         * instruction stream would otherwise pace the whole CTA. */
        if (lane == 0) {
            const uint32_t t = warp - (MMB_STT_DEQ_WARPS + 1u);
            const uint32_t d_base = tmem_base + ST_D_COL + t * ST_NACC * NPAD;
            const uint32_t a_base = tmem_base + ST_A_COL + t * 64u;
            uint32_t s = 0, round = 0, half_idx = 0, slot = 0, use = 0;   /* A slot and its use count */
            for (uint32_t it = 0; it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u,
                                               round += (s == 0u)) {
                const uint32_t xs = base + s * STAGE_B + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B;
                mbar_wait(bar_x + 8u * s, round & 1u, p.status);
                const uint32_t idesc = umma_idesc_16(128u, NPAD, lds32(fmt_flag + 4u * s) ? 0u : 1u);
                const uint64_t bd0 = umma_desc_sw128(xs);
#pragma unroll
                for (uint32_t kh = 0; kh < 2u; kh++, half_idx++,
                              slot = (slot + 1u == ST_A_SLOTS) ? 0u : slot + 1u, use += (slot == 0u)) {
                    mbar_wait(a_full + 8u * slot, use & 1u, p.status);
                    tc_fence_after();
                    const uint32_t a_slot = a_base + slot * 128u;
                    const uint32_t fresh = half_idx == 0 ? 0u : 1u;   /* very first use of the accumulators */
#pragma unroll
                    for (uint32_t j = 0; j < 8u; j++) {
                        const uint32_t k16 = kh * 8u + j;             /* 16-wide K block of the step */
                        /* descriptor start address is in 16-byte units */
                        const uint64_t bd = bd0 + (((k16 >> 2) * (NPAD * 128u) + (k16 & 3u) * 32u) >> 4);
                        umma_ts(d_base + (j & (ST_NACC - 1u)) * NPAD, a_slot + j * 8u, bd, idesc,
                                j < ST_NACC ? fresh : 1u);
                    }
                    umma_commit(a_empty + 8u * slot);
                }
                umma_commit(bar_empty + 8u * s);
            }
            umma_commit(accum_full);
        }
    } else if (warp > MMB_STT_DEQ_WARPS + 2u) {
        /* ------------------------------ activation transform ------------------ *
         * In place, element for element: the swizzled K-major layout TMA wrote
         * is what the tensor core reads; only the number format changes. */
        const uint32_t xt = tid - (MMB_STT_DEQ_WARPS + 3u) * 32u;
        uint32_t s = 0, round = 0;
        for (uint32_t it = 0; it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u,
                                           round += (s == 0u)) {
            const uint32_t xs = base + s * STAGE_B + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B;
            mbar_wait_warp(bar_raw + 8u * s, round & 1u, p.status);
            uint4 v[X_ITEMS];
            uint32_t ok = 0xffffffffu;
#pragma unroll
            for (uint32_t i = 0; i < X_ITEMS; i++) {
                v[i] = lds128(xs + (i * XFORM_THREADS + xt) * 16u);
                ok &= t_fp16_exact_mask(v[i].x) & t_fp16_exact_mask(v[i].y) &
                      t_fp16_exact_mask(v[i].z) & t_fp16_exact_mask(v[i].w);
            }
            uint32_t half_ok;
            asm volatile(
                "{\n\t.reg .pred q, r;\n\t"
                "setp.eq.u32 q, %1, 0xffffffff;\n\t"
                "bar.red.and.pred r, 2, %2, q;\n\t"
                "selp.u32 %0, 1, 0, r;\n\t}"
                : "=r"(half_ok) : "r"(ok), "r"(XFORM_THREADS) : "memory");
            if (half_ok) {
#pragma unroll
                for (uint32_t i = 0; i < X_ITEMS; i++) {
                    uint4 o;
                    o.x = t_bf16x2_to_f16x2(v[i].x);
                    o.y = t_bf16x2_to_f16x2(v[i].y);
                    o.z = t_bf16x2_to_f16x2(v[i].z);
                    o.w = t_bf16x2_to_f16x2(v[i].w);
                    sts128(xs + (i * XFORM_THREADS + xt) * 16u, o);
                }
                fence_proxy_async_smem();              /* the tensor core reads through the async proxy */
            }
            if (xt == 0)
                sts32(fmt_flag + 4u * s, half_ok);
            mbar_arrive(bar_x + 8u * s);
        }
    } else {
        /* ------------------------------ dequantise into tensor memory --------- */
        const uint32_t quad = warp & 3u, tile = (warp >> 2) & 1u, kq = warp >> 3;
        const uint32_t row = tile * 128u + quad * 32u + lane;            /* row within the CTA */
        const uint32_t lane_addr = (quad * 32u) << 16;
        uint32_t s = 0, round = 0, slot = 0, use = 0;
        for (uint32_t it = 0; it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u,
                                           round += (s == 0u)) {
            const uint32_t stage = base + s * STAGE_B;
            mbar_wait_warp(bar_raw + 8u * s, round & 1u, p.status);   /* weights and scales landed */
            mbar_wait_warp(bar_x + 8u * s, round & 1u, p.status);     /* operand format of the step known */
            const bool half_step = lds32(fmt_flag + 4u * s) != 0u;
            const uint32_t lut = half_step ? lut_hf : lut_bf;
            const uint4 sc16 = lds128(stage + MMB_ST_PAYLOAD_B + row * 16u);
#pragma unroll
            for (uint32_t kh = 0; kh < 2u; kh++,
                          slot = (slot + 1u == ST_A_SLOTS) ? 0u : slot + 1u, use += (slot == 0u)) {
                /* 64 weights: K offset kh*128 + kq*64 of the step = payload chunks 4kh+2kq, +1 */
                const uint32_t c0 = 4u * kh + 2u * kq;
                const uint4 p0 = lds128(stage + row * 128u + (((c0 + 0u) ^ (row & 7u)) << 4));
                const uint4 p1 = lds128(stage + row * 128u + (((c0 + 1u) ^ (row & 7u)) << 4));
                const uint32_t sc4 = kh == 0 ? (kq ? sc16.y : sc16.x) : (kq ? sc16.w : sc16.z);
                uint32_t c[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    c[j] = lds32(lut + ((sc4 >> (8 * j)) & 255u) * 4u);
                uint32_t out[32];
                if (half_step) dequant64<true>(p0, p1, c, out);
                else           dequant64<false>(p0, p1, c, out);
                if (use > 0u)
                    mbar_wait_warp(a_empty + 8u * slot, (use - 1u) & 1u, p.status);
                tc_fence_after();
                tmem_st_32x32(tmem_base + lane_addr + ST_A_COL + slot * 128u + tile * 64u + kq * 32u, out);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(a_full + 8u * slot);
            }
        }

        /* ------------------------------ epilogue ------------------------------ */
        mbar_wait_warp(accum_full, 0u, p.status);
        tc_fence_after();
        if (kq == 0) {                                   /* one warp per (tile, lane quadrant) */
            uint32_t acc[NPAD];
#pragma unroll
            for (uint32_t a = 0; a < ST_NACC; a++) {         /* accumulators added in a fixed order */
                uint32_t part[NPAD];
                const uint32_t taddr = tmem_base + lane_addr + ST_D_COL + (tile * ST_NACC + a) * NPAD;
                if (NPAD == 16) tmem_ld_32x16(taddr, *reinterpret_cast<uint32_t (*)[16]>(part));
                else            tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t (*)[32]>(part));
                tmem_ld_wait();
#pragma unroll
                for (uint32_t m = 0; m < NPAD; m++)
                    acc[m] = a == 0 ? part[m]
                                    : __float_as_uint(__uint_as_float(acc[m]) + __uint_as_float(part[m]));
            }
            const uint32_t n = row0 + row;
            if (p.split_k == 1) {
                if (n < p.N) {
#pragma unroll
                    for (uint32_t m = 0; m < NPAD; m++)
                        if (m < p.M) {
                            __nv_bfloat16 hv = __float2bfloat16_rn(__uint_as_float(acc[m]) * p.gs);
                            const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n;
                            for (uint32_t d = 0; d < p.n_dst; d++)
                                p.y[d][off] = *reinterpret_cast<uint16_t *>(&hv);
                        }
                }
            } else if (n < p.N) {
                float *mine = p.partial + static_cast<size_t>(blockIdx.y) * NPAD * p.N;
#pragma unroll
                for (uint32_t m = 0; m < NPAD; m++)
                    if (m < p.M)
                        __stcg(mine + static_cast<size_t>(m) * p.N + n, __uint_as_float(acc[m]));
            }
        }
        if (p.split_k > 1) {
            /* publish this slice; the CTA that arrives last adds the slices in order */
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(MMB_STT_DEQ_WARPS * 32) : "memory");
            if (tid == 0) {
                const unsigned ticket = atomicAdd(p.counters + blockIdx.x, 1u);
                sts32(last_flag, (ticket == p.split_k - 1u) ? 1u : 0u);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(MMB_STT_DEQ_WARPS * 32) : "memory");
            if (lds32(last_flag)) {
                __threadfence();
                /* 512 threads cover 256 rows x 2 halves of the activation rows */
                const uint32_t n = row0 + (tid & 255u), mh = tid >> 8;
                constexpr uint32_t MH = NPAD / 2;
                if (n < p.N) {
                    float sum[MH];
#pragma unroll
                    for (uint32_t i = 0; i < MH; i++) sum[i] = 0.0f;
                    for (uint32_t sl = 0; sl < p.split_k; sl++) {
                        float v[MH];
#pragma unroll
                        for (uint32_t i = 0; i < MH; i++) {
                            const uint32_t m = mh * MH + i;
                            v[i] = m < p.M ? __ldcg(p.partial + (static_cast<size_t>(sl) * NPAD + m) * p.N + n)
                                           : 0.0f;
                        }
#pragma unroll
                        for (uint32_t i = 0; i < MH; i++) sum[i] += v[i];
                    }
#pragma unroll
                    for (uint32_t i = 0; i < MH; i++) {
                        const uint32_t m = mh * MH + i;
                        if (m < p.M) {
                            __nv_bfloat16 hv = __float2bfloat16_rn(sum[i] * p.gs);
                            const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n;
                            for (uint32_t d = 0; d < p.n_dst; d++)
                                p.y[d][off] = *reinterpret_cast<uint16_t *>(&hv);
                        }
                    }
                }
                if (tid == 0)
                    p.counters[blockIdx.x] = 0u;             /* ready for the next launch */
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == MMB_STT_DEQ_WARPS + 1u) {
        tc_fence_after();
        tmem_dealloc(tmem_base, ST_TMEM_COLS);
    }
}

template <int NPAD>
static int launch_npad(const mmb_args *a, unsigned *status, cudaStream_t st)
{
    StreamTParams p;
    if (a->n_dst) {
        for (uint32_t d = 0; d < a->n_dst; d++) p.y[d] = static_cast<uint16_t *>(a->y_dst[d]);
        p.n_dst = a->n_dst; p.ldy = a->ldy; p.col0 = a->col0;
    } else {
        p.y[0] = static_cast<uint16_t *>(a->y);
        p.n_dst = 1; p.ldy = a->N; p.col0 = 0;
    }
    p.counters = static_cast<unsigned *>(a->ws);
    p.partial = a->ws ? reinterpret_cast<float *>(static_cast<unsigned char *>(a->ws) + MMB_WS_COUNTER_B)
                      : nullptr;
    p.status = status;
    p.gs = a->gs;
    p.M = a->M; p.K = a->K; p.N = a->N;
    p.k_steps = a->plan.k_steps;
    p.split_k = a->plan.split_k;
    p.stages = a->plan.stages;
    TmaDesc tp, ts, tx;
    memcpy(tp.bytes, a->tm_payload, 128);
    memcpy(ts.bytes, a->tm_scale, 128);
    memcpy(tx.bytes, a->tm_x, 128);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a->plan.grid_x, a->plan.grid_y);
    cfg.blockDim = dim3(MMB_STT_THREADS);
    cfg.dynamicSmemBytes = a->plan.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    /* this kernel only has the trigger-first form; any other mode runs as a plain launch */
    attr[0].val.programmaticStreamSerializationAllowed = a->pdl == MMB_PDL_TRIGGER_FIRST ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, f4_streamt_kernel<NPAD>, tp, ts, tx, p));
}

} // namespace mmb

extern "C" int mmb_streamt_init(void)
{
    cudaError_t e = cudaFuncSetAttribute(mmb::f4_streamt_kernel<16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, MMB_SMEM_MAX);
    if (e != cudaSuccess) return static_cast<int>(e);
    return static_cast<int>(cudaFuncSetAttribute(mmb::f4_streamt_kernel<32>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 MMB_SMEM_MAX));
}

extern "C" int mmb_launch_streamt(const mmb_args *a, void *stream)
{
    unsigned *status = nullptr;
    int e = mmb_status_word(&status);
    if (e) return e;
    if (a->plan.split_k > 1 && !a->ws)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (a->plan.tile_m) {
    case 16: return mmb::launch_npad<16>(a, status, st);
    case 32: return mmb::launch_npad<32>(a, status, st);
    default: return static_cast<int>(cudaErrorInvalidValue);
    }
}
