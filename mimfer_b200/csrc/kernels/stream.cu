/*
 * STREAM: the CUDA-core decode kernel of the NVFP4 linear op (M <= 32); the
 * selector prefers the block-scaled tensor kernel (mx.cu) and falls back to this
 * one when the activations' digit planes do not fit the workspace.
 *
 * One CTA owns the plan's number of weight rows (256; 128 for weights with few
 * rows; any multiple of 16 runs) and a contiguous range of 256-wide K steps.
 * One thread keeps a ring of stages full by TMA: per step a box of packed
 * payload (256 rows x 128 B, 128-byte swizzle), one of block scales (256 rows
 * x 16 B) and the matching slice of the activations (up to 32 rows x 512 B).
 * Four transform warps pick the operand format of the step from the
 * activations and rewrite that slice in place.  Sixteen consumer warps each take 16
 * rows: 16-byte shared loads of payload, nibble unpack and scale in registers
 * (fp4.cuh), warp MMAs with the weights as the 16-row operand and the
 * activation rows as the 8-wide operand, fp32 accumulators in registers.
 * With split-K the partial sums meet in the workspace and the CTA that
 * arrives last adds them in slice order, so the result does not depend on
 * scheduling (no atomics on data; the reference demands order-faithful
 * reductions, include/mimfer/kernels.h:14-15).
 *
 * Two operand formats per K step, chosen by the transform warps from the
 * activations of that step:
 *
 *  fp16   when every activation of the slice is zero or has 2^-17 <= |x| < 2^16,
 *         i.e. converts to fp16 without loss.  Weights go through
 *         cvt.rn.f16x2.e2m1x2 and one packed fp16 multiply by the scale (itself
 *         converted with cvt.rn.f16x2.e4m3x2, no table): about one instruction
 *         per weight.  Activations are stored in column order.
 *  bf16   otherwise (tiny, huge or non-finite activations).  Weights take the
 *         bf16 subnormal construction of fp4.cuh, about two instructions per
 *         weight, with the pairing (n0,n4)(n1,n5)(n2,n6)(n3,n7); the transform warps
 *         store each group of eight activations as (x0,x4,x1,x5,x2,x6,x3,x7) to
 *         match (the MMA sums over K, so any order works if both operands agree).
 *
 * Either way the dequantised weight and the activation are exact in the
 * operand format, so every product is the reference's product and both paths
 * add into the same fp32 accumulators.
 *
 * Lane (g, t) of a consumer warp (g = lane/4, t = lane%4) owns the 64 weights
 * [64t, 64t+64) of each of its rows per step, as eight 32-bit words.
 *
 * It replaces the one-thread-per-output kernel of the reference
 * (src/kernels/cuda/cx.cu:345-356) for the decode regime.
 */
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

struct StreamParams {
    const uint16_t *x;
    uint16_t       *y[MMB_MAX_PEERS];   /* destinations: own output, then peers' (tensor parallel) */
    uint32_t        n_dst, ldy, col0;    /* row pitch and column offset inside each destination */
    float          *partial;     /* workspace + MMB_WS_COUNTER_B, or NULL */
    unsigned       *counters;    /* workspace base, or NULL               */
    unsigned       *status;
    float           gs;
    uint32_t        M, K, N;
    uint32_t        k_steps, split_k, stages;
    uint32_t        pdl;         /* MMB_PDL_* */
    float           gs_up;       /* gated pair: scale of the up projection        */
    uint32_t        gate_plane;  /* gated pair: which half of the CTA's rows is the gate */
    uint32_t        rows;        /* weight rows per CTA: a multiple of 16, at most MMB_ST_ROWS */
    uint32_t        dbg;         /* MMB_DBG_*: measurement modes, 0 in production  */
};

/* One output element to every destination (one, or all tensor-parallel peers). */
__device__ __forceinline__ void store_all(const StreamParams &p, uint32_t m, uint32_t n, uint16_t v)
{
    const size_t off = static_cast<size_t>(m) * p.ldy + p.col0 + n;
    p.y[0][off] = v;
#pragma unroll 1                       /* kept rolled: this runs once per output, code size matters more */
    for (uint32_t d = 1; d < p.n_dst; d++)
        p.y[d][off] = v;
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* 0xffffffff when both bf16 halves of u convert to fp16 exactly. */
__device__ __forceinline__ uint32_t fp16_exact_mask(uint32_t u)
{
    const __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&u));
    const __nv_bfloat162 hi = __float2bfloat162_rn(65536.0f);
    const __nv_bfloat162 lo = __float2bfloat162_rn(7.62939453125e-06f);       /* 2^-17 */
    const __nv_bfloat162 zero = __float2bfloat162_rn(0.0f);
    return __hlt2_mask(a, hi) & (__hge2_mask(a, lo) | __heq2_mask(a, zero));
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t u)
{
    const __half2 h = __floats2half2_rn(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    return *reinterpret_cast<const uint32_t *>(&h);
}

/* Activation slot of a stage: TMA delivers MPAD rows of 512 bytes (256 values)
 * in column order; the transform warps rewrite it as rows of 576 bytes, with
 * 16 bytes of padding after every eighth 16-byte chunk.  That is conflict-free
 * both for the transform warps (a warp covers one row, chunk = lane) and for
 * the consumers (lane (g, t) reads chunk 8t + word of row g), and gives the
 * consumers compile-time offsets. */
__device__ __forceinline__ uint32_t x_slot_offset(uint32_t m, uint32_t c)
{
    return m * 576u + (c >> 3) * 144u + (c & 7u) * 16u;
}

/* One K step of one consumer warp in one operand format (HALF: fp16, else bf16). */
template <int MT, int RT, int SLOTS, bool HALF>
__device__ __forceinline__ void consume_step(float (&accs)[SLOTS][RT][MT][4], uint32_t stage,
                                             uint32_t lut, uint32_t warp, uint32_t g, uint32_t t)
{
    /* per-lane bases; everything below is base + compile-time offset */
    const uint32_t pay = stage + (warp * (16u * RT) + g) * 128u;
    const uint32_t scl = stage + MMB_ST_PAYLOAD_B + (warp * (16u * RT) + g) * 16u + t * 4u;
    const uint32_t xs = stage + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B + g * 576u + t * 144u;

    /* the four scale entries of each of this lane's rows, looked up once */
    uint32_t cs[RT][2][4];
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int rr = 0; rr < 2; rr++) {
            const uint32_t sc4 = lds32(scl + (rt * 16u + rr * 8u) * 16u);
            if (HALF) {
                scales4_f16(sc4, cs[rt][rr]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    cs[rt][rr][j] = lds32(lut + ((sc4 >> (8 * j)) & 255u) * 4u);
            }
        }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint4 pw[RT][2];
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int rr = 0; rr < 2; rr++)
                pw[rt][rr] = lds128(pay + (rt * 16u + rr * 8u) * 128u + (((2u * t + h) ^ g) << 4));
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
            const uint32_t word = 4u * h + wi;
            uint4 xb[MT];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
                xb[mt] = lds128(xs + mt * (8u * 576u) + word * 16u);
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                const uint32_t c0 = cs[rt][0][2 * h + (wi >> 1)];
                const uint32_t c8 = cs[rt][1][2 * h + (wi >> 1)];
                const uint32_t w0 = wi == 0 ? pw[rt][0].x : wi == 1 ? pw[rt][0].y
                                  : wi == 2 ? pw[rt][0].z : pw[rt][0].w;
                const uint32_t w8 = wi == 0 ? pw[rt][1].x : wi == 1 ? pw[rt][1].y
                                  : wi == 2 ? pw[rt][1].z : pw[rt][1].w;
                if (HALF) {
                    const uint4 a0 = unpack8_natural_f16(w0, c0);
                    const uint4 a8 = unpack8_natural_f16(w8, c8);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        mma_f16_16816(accs[(2 * wi) % SLOTS][rt][mt], a0.x, a8.x, a0.y, a8.y,
                                      xb[mt].x, xb[mt].y);
                        mma_f16_16816(accs[(2 * wi + 1) % SLOTS][rt][mt], a0.z, a8.z, a0.w, a8.w,
                                      xb[mt].z, xb[mt].w);
                    }
                } else {
                    uint32_t q0[4], q8[4];
                    unpack8_paired(w0, c0, q0);
                    unpack8_paired(w8, c8, q8);
#pragma unroll
                    for (int j = 0; j < 4; j++) {              /* back from the 2^-8 of the bf16 form */
                        q0[j] = mul_bf16x2(q0[j], 0x43804380u);
                        q8[j] = mul_bf16x2(q8[j], 0x43804380u);
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        mma_bf16_16816(accs[(2 * wi) % SLOTS][rt][mt], q0[0], q8[0], q0[1], q8[1],
                                       xb[mt].x, xb[mt].y);
                        mma_bf16_16816(accs[(2 * wi + 1) % SLOTS][rt][mt], q0[2], q8[2], q0[3], q8[3],
                                       xb[mt].z, xb[mt].w);
                    }
                }
            }
        }
    }
}

/* The weight boxes of one K step.  Gated pair: one 3-D box brings 128 rows of
 * each projection, plane 0 first, so the CTA's 256 rows are [plane 0 | plane 1]. */
template <bool GLU>
__device__ __forceinline__ void load_weights(uint32_t stage, const TmaDesc *tm_payload,
                                             const TmaDesc *tm_scale, uint32_t ks, uint32_t row0,
                                             uint32_t bar)
{
    if constexpr (GLU) {
        tma_load_3d(stage, tm_payload, static_cast<int>(ks * 128u), static_cast<int>(row0), 0, bar);
        tma_load_3d(stage + MMB_ST_PAYLOAD_B, tm_scale, static_cast<int>(ks * 16u),
                    static_cast<int>(row0), 0, bar);
    } else {
        tma_load_2d(stage, tm_payload, static_cast<int>(ks * 128u), static_cast<int>(row0), bar);
        tma_load_2d(stage + MMB_ST_PAYLOAD_B, tm_scale, static_cast<int>(ks * 16u),
                    static_cast<int>(row0), bar);
    }
}

/* Gated pair, last step: the warps holding plane 1 hand their sums to the warps
 * holding plane 0 through shared memory (the ring is idle by then), which apply
 * the scales, silu(gate) * up and store.  v: final fp32 sums of this thread. */
template <int MT, int RT>
__device__ __forceinline__ void glu_store(const StreamParams &p, const float (&v)[RT][MT][4],
                                          uint32_t xch, uint32_t j0, uint32_t warp, uint32_t g,
                                          uint32_t t)
{
    constexpr uint32_t MPAD = MT * 8, HALF_ROWS = MMB_ST_ROWS / 2;
    const bool upper = warp * (16u * RT) >= HALF_ROWS;
    asm volatile("bar.sync 1, %0;" ::"n"(MMB_ST_CONSUMERS * 32) : "memory");   /* every warp left the ring */
    if (upper) {
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t lr = warp * (16u * RT) + rt * 16u + (i >> 1) * 8u + g - HALF_ROWS;
                    const uint32_t m = mt * 8u + 2u * t + (i & 1);
                    sts32(xch + (lr * MPAD + m) * 4u, __float_as_uint(v[rt][mt][i]));
                }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(MMB_ST_CONSUMERS * 32) : "memory");
    if (upper)
        return;
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t lr = warp * (16u * RT) + rt * 16u + (i >> 1) * 8u + g;
                const uint32_t m = mt * 8u + 2u * t + (i & 1);
                const float other = __uint_as_float(lds32(xch + (lr * MPAD + m) * 4u));
                const float gate = p.gate_plane ? other : v[rt][mt][i];
                const float up = p.gate_plane ? v[rt][mt][i] : other;
                if (j0 + lr < p.N && m < p.M)
                    store_all(p, m, j0 + lr, glu_out_bf16(gate, up, p.gs, p.gs_up));
            }
}

template <int MT, bool GLU>
__global__ void __launch_bounds__(MMB_ST_THREADS, 1)
f4_stream_kernel(const __grid_constant__ TmaDesc tm_payload,
                 const __grid_constant__ TmaDesc tm_scale, const __grid_constant__ TmaDesc tm_x,
                 const StreamParams p)
{
    constexpr uint32_t MPAD = MT * 8;
    constexpr int RT = MMB_ST_ROWS / (16 * MMB_ST_CONSUMERS);   /* 16-row tiles per consumer warp */
    constexpr uint32_t STAGE_B = MMB_ST_STAGE_B(MT);
    constexpr uint32_t XFORM_THREADS = MMB_ST_XFORM_WARPS * 32u;
    constexpr uint32_t ITEMS = MPAD * 32u / XFORM_THREADS;    /* 16-byte chunks per transform thread */
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t lut_bf = base + p.stages * STAGE_B;       /* scale * 2^118, bf16x2 (bf16 steps) */
    const uint32_t bar_raw = lut_bf + 2048u;                 /* [stages] TMA landed      */
    const uint32_t bar_full = bar_raw + 8u * p.stages;       /* [stages] activations ready */
    const uint32_t bar_empty = bar_full + 8u * p.stages;     /* [stages] consumers done  */
    const uint32_t fmt_flag = bar_empty + 8u * p.stages;     /* [stages] 1 = fp16 step  */
    const uint32_t last_flag = fmt_flag + 4u * p.stages;     /* split-K: "this CTA reduces" */

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    /* rows of this CTA and the consumer warps that have some (16 rows each); a
     * gated pair always takes the full tile, half of it from each projection */
    const uint32_t rows = GLU ? MMB_ST_ROWS : p.rows;
    const uint32_t nc = rows >> 4;
    /* first weight row of the CTA (of each projection for a gated pair) */
    const uint32_t row0 = blockIdx.x * (GLU ? MMB_ST_ROWS / 2 : rows);
    const uint32_t ks_begin = static_cast<uint32_t>(
        static_cast<uint64_t>(p.k_steps) * blockIdx.y / p.split_k);
    const uint32_t ks_end = static_cast<uint32_t>(
        static_cast<uint64_t>(p.k_steps) * (blockIdx.y + 1) / p.split_k);
    const uint32_t nsteps = ks_end - ks_begin;

    const uint32_t stage_bytes = rows * 144u + MMB_ST_X_RAW_B(MT);   /* payload + scales + activations */
    const bool loads = !(p.dbg & MMB_DBG_NO_LOADS);
    const uint32_t first = nsteps < p.stages ? nsteps : p.stages;   /* steps of the first ring */
    if (tid == MMB_ST_CONSUMERS * 32u) {
        /* the issuing thread sets the barriers up itself and starts the weight
         * stream at once, while the other warps are still building the tables */
        tma_prefetch_desc(&tm_payload);
        tma_prefetch_desc(&tm_scale);
        tma_prefetch_desc(&tm_x);
        for (uint32_t s = 0; s < p.stages; s++) {
            mbar_init(bar_raw + 8u * s, 1u);
            mbar_init(bar_full + 8u * s, XFORM_THREADS);
            mbar_init(bar_empty + 8u * s, nc);
        }
        mbar_fence_init();
        for (uint32_t it = 0; loads && it < first; it++) {
            const uint32_t stage = base + it * STAGE_B, ks = ks_begin + it;
            mbar_expect_tx(bar_raw + 8u * it, stage_bytes);
            load_weights<GLU>(stage, &tm_payload, &tm_scale, ks, row0, bar_raw + 8u * it);
        }
    }
    if (tid < 256u)
        sts32(lut_bf + tid * 4u, scale_lut_entry(tid));     /* the fp16 steps convert their scales directly */
    __syncthreads();
    if (p.pdl == MMB_PDL_TRIGGER_FIRST)
        grid_dep_launch();

    if (warp == MMB_ST_CONSUMERS) {
        /* ------------------------------ TMA issue ------------------------- *
         * The weights do not depend on the previous kernel in the stream, the
         * activations may: the first ring of weight boxes went out in the
         * prologue, before the grid-dependency wait, the activation boxes
         * follow it.  An op known to be independent of everything in flight
         * skips that wait and makes up for it before the CTA exits (launch.h). */
        if (lane == 0) {
            if (p.pdl == MMB_PDL_INDEPENDENT) {
                grid_dep_launch();
            } else {
                grid_dep_wait();
                if (p.pdl == MMB_PDL_WAIT_FIRST)
                    grid_dep_launch();
            }
            for (uint32_t it = 0; loads && it < first; it++)
                tma_load_2d(base + it * STAGE_B + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B, &tm_x,
                            static_cast<int>((ks_begin + it) * MMB_ST_KSTEP), 0, bar_raw + 8u * it);
            uint32_t s = 0, round = 1;                 /* stage index and its use count */
            for (uint32_t it = first; loads && it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u,
                                                   round += (s == 0u)) {
                const uint32_t stage = base + s * STAGE_B, ks = ks_begin + it;
                mbar_wait(bar_empty + 8u * s, (round - 1u) & 1u, p.status);
                fence_proxy_async_smem();          /* generic writes of the slot precede the refill */
                mbar_expect_tx(bar_raw + 8u * s, stage_bytes);
                load_weights<GLU>(stage, &tm_payload, &tm_scale, ks, row0, bar_raw + 8u * s);
                tma_load_2d(stage + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B, &tm_x,
                            static_cast<int>(ks * MMB_ST_KSTEP), 0, bar_raw + 8u * s);
            }
            if (p.pdl == MMB_PDL_INDEPENDENT)
                grid_dep_wait();                   /* this kernel completes after its predecessor */
        }
        return;
    }
    if (warp > MMB_ST_CONSUMERS) {
        /* ------------------------------ activation transform --------------- *
         * TMA delivers the slice as bf16 rows in column order; these warps pick
         * the operand format of the step and rewrite the slot in place. */
        const uint32_t xt = tid - (MMB_ST_CONSUMERS + 1u) * 32u;
        uint32_t s = 0, round = 0;
        for (uint32_t it = 0; loads && it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u,
                                           round += (s == 0u)) {
            const uint32_t xs = base + s * STAGE_B + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B;
            mbar_wait_warp(bar_raw + 8u * s, round & 1u, p.status);
            uint4 v[ITEMS];
            uint32_t ok = 0xffffffffu;
#pragma unroll
            for (uint32_t i = 0; i < ITEMS; i++) {
                const uint32_t id = i * XFORM_THREADS + xt;        /* row = id / 32, chunk = lane */
                v[i] = lds128(xs + id * 16u);
                ok &= fp16_exact_mask(v[i].x) & fp16_exact_mask(v[i].y) &
                      fp16_exact_mask(v[i].z) & fp16_exact_mask(v[i].w);
            }
            /* one decision per step; the barrier also orders every read of the
             * slot before the first in-place write */
            uint32_t half_ok;
            asm volatile(
                "{\n\t.reg .pred q, r;\n\t"
                "setp.eq.u32 q, %1, 0xffffffff;\n\t"
                "bar.red.and.pred r, 2, %2, q;\n\t"
                "selp.u32 %0, 1, 0, r;\n\t}"
                : "=r"(half_ok) : "r"(ok), "r"(XFORM_THREADS) : "memory");
#pragma unroll
            for (uint32_t i = 0; i < ITEMS; i++) {
                const uint32_t id = i * XFORM_THREADS + xt;
                const uint32_t m = id >> 5, c = id & 31u;
                uint4 o;
                if (half_ok) {
                    o.x = bf16x2_to_f16x2(v[i].x);
                    o.y = bf16x2_to_f16x2(v[i].y);
                    o.z = bf16x2_to_f16x2(v[i].z);
                    o.w = bf16x2_to_f16x2(v[i].w);
                } else {
                    o.x = prmt(v[i].x, v[i].z, 0x5410u);       /* x0 x4 */
                    o.y = prmt(v[i].x, v[i].z, 0x7632u);       /* x1 x5 */
                    o.z = prmt(v[i].y, v[i].w, 0x5410u);       /* x2 x6 */
                    o.w = prmt(v[i].y, v[i].w, 0x7632u);       /* x3 x7 */
                }
                sts128(xs + x_slot_offset(m, c), o);
            }
            if (xt == 0)
                sts32(fmt_flag + 4u * s, half_ok);
            mbar_arrive(bar_full + 8u * s);
        }
        return;
    }

    /* --------------------------------- consumers ------------------------- */
    if (warp >= nc)
        return;                                        /* no rows for this warp */
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t nct = nc * 32u;                     /* threads at the consumers' named barrier */
    /* SLOTS independent accumulator sets per (row tile, activation tile): the
     * warp MMA has a long dependent-issue latency, so consecutive MMAs must not
     * chain on one accumulator.  Eight chains per warp whatever MT is. */
    constexpr int SLOTS = 4 / MT;
    float accs[SLOTS][RT][MT][4];
#pragma unroll
    for (int sl = 0; sl < SLOTS; sl++)
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) accs[sl][rt][mt][i] = 0.0f;

    uint32_t s = 0, round = 0;
    for (uint32_t it = 0; it < nsteps; it++, s = (s + 1u == p.stages) ? 0u : s + 1u,
                                       round += (s == 0u)) {
        const uint32_t stage = base + s * STAGE_B;
        if (loads)
            mbar_wait_warp(bar_full + 8u * s, round & 1u, p.status);
        if (!(p.dbg & MMB_DBG_NO_MATH)) {
            if (!loads || lds32(fmt_flag + 4u * s) != 0u)
                consume_step<MT, RT, SLOTS, true>(accs, stage, lut_bf, warp, g, t);
            else
                consume_step<MT, RT, SLOTS, false>(accs, stage, lut_bf, warp, g, t);
        }
        __syncwarp();
        if (loads && lane == 0)
            mbar_arrive(bar_empty + 8u * s);
    }

    /* --------------------------------- epilogue -------------------------- */
    const float out_scale = p.gs;
    float acc[RT][MT][4];                             /* slots added in a fixed order */
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float v = accs[0][rt][mt][i];
#pragma unroll
                for (int sl = 1; sl < SLOTS; sl++) v += accs[sl][rt][mt][i];
                acc[rt][mt][i] = v;
            }
    if (p.split_k == 1 || (p.dbg & MMB_DBG_NO_EXCHANGE)) {
        if constexpr (GLU) {
            glu_store<MT, RT>(p, acc, base, row0, warp, g, t);
        } else {
#pragma unroll
            for (int rt = 0; rt < RT; rt++)
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t n = row0 + warp * (16u * RT) + rt * 16u + (i >> 1) * 8u + g;
                        const uint32_t m = mt * 8u + 2u * t + (i & 1);
                        if (n < p.N && m < p.M) {
                            __nv_bfloat16 hv = __float2bfloat16_rn(acc[rt][mt][i] * out_scale);
                            store_all(p, m, n, *reinterpret_cast<uint16_t *>(&hv));
                        }
                    }
        }
        return;
    }

    /* split-K: publish this slice, the last CTA of the row block reduces.  The
     * partials hold one column per weight row of the CTA tiles (pitch = padded
     * row count for a gated pair, whose tiles interleave the two projections). */
#define MMB_PCOL(lr) (GLU ? blockIdx.x * MMB_ST_ROWS + (lr) : row0 + (lr))
#define MMB_PPITCH (GLU ? gridDim.x * MMB_ST_ROWS : p.N)
#define MMB_ROW_OK(lr) (GLU ? (row0 + ((lr) & (MMB_ST_ROWS / 2 - 1u)) < p.N) : (row0 + (lr) < p.N))
    float *mine = p.partial + static_cast<size_t>(blockIdx.y) * MPAD * MMB_PPITCH;
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t lr = warp * (16u * RT) + rt * 16u + (i >> 1) * 8u + g;
                const uint32_t m = mt * 8u + 2u * t + (i & 1), pc = MMB_PCOL(lr);
                if (MMB_ROW_OK(lr) && m < p.M)
                    __stcg(mine + static_cast<size_t>(m) * MMB_PPITCH + pc, acc[rt][mt][i]);
            }
    /* Every thread's partials are ordered before the ticket by the CTA barrier
     * and one device-scope fence of the thread that takes the ticket; on the
     * other side the same thread fences after the ticket and the barrier hands
     * the visibility on to the CTA (the pattern of a grid-wide barrier). */
    asm volatile("bar.sync 1, %0;" ::"r"(nct) : "memory");
    if (tid == 0) {
        __threadfence();
        const unsigned ticket = atomicAdd(p.counters + blockIdx.x, 1u);
        __threadfence();
        sts32(last_flag, (ticket == p.split_k - 1u) ? 1u : 0u);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nct) : "memory");
    if (!lds32(last_flag))
        return;
    /* Slices are added in ascending order for every output, so the sum does not
     * depend on which CTA arrived last; the loads of several slices (all
     * outputs of this thread) are issued together. */
    float sum[RT][MT][4];
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) sum[rt][mt][i] = 0.0f;
    constexpr int BATCH = 8 / MT;                 /* slices whose loads are in flight together */
    for (uint32_t sl = 0; sl < p.split_k; sl += BATCH) {
        float v[BATCH][RT][MT][4];
#pragma unroll
        for (int u = 0; u < BATCH; u++)
#pragma unroll
            for (int rt = 0; rt < RT; rt++)
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t lr = warp * (16u * RT) + rt * 16u + (i >> 1) * 8u + g;
                        const uint32_t m = mt * 8u + 2u * t + (i & 1), pc = MMB_PCOL(lr);
                        v[u][rt][mt][i] = 0.0f;
                        if (MMB_ROW_OK(lr) && m < p.M && sl + u < p.split_k)
                            v[u][rt][mt][i] = __ldcg(p.partial +
                                (static_cast<size_t>(sl + u) * MPAD + m) * MMB_PPITCH + pc);
                    }
#pragma unroll
        for (int u = 0; u < BATCH; u++)
#pragma unroll
            for (int rt = 0; rt < RT; rt++)
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) sum[rt][mt][i] += v[u][rt][mt][i];
    }
    if constexpr (GLU) {
        glu_store<MT, RT>(p, sum, base, row0, warp, g, t);
    } else {
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t n = row0 + warp * (16u * RT) + rt * 16u + (i >> 1) * 8u + g;
                    const uint32_t m = mt * 8u + 2u * t + (i & 1);
                    if (n < p.N && m < p.M) {
                        __nv_bfloat16 hv = __float2bfloat16_rn(sum[rt][mt][i] * out_scale);
                        store_all(p, m, n, *reinterpret_cast<uint16_t *>(&hv));
                    }
                }
    }
    if (tid == 0)
        p.counters[blockIdx.x] = 0u;                /* ready for the next launch */
#undef MMB_ROW_OK
#undef MMB_PCOL
#undef MMB_PPITCH
}

template <int MT, bool GLU>
static int launch_mt(const mmb_args *a, unsigned *status, cudaStream_t st)
{
    StreamParams p;
    p.x = static_cast<const uint16_t *>(a->x);
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
    p.gs_up = a->gs_up;
    p.gate_plane = a->gate_plane ? 1u : 0u;
    p.rows = a->plan.tile_n;
    p.dbg = a->dbg;
    p.pdl = static_cast<uint32_t>(a->pdl);
    TmaDesc tp, ts, tx;
    memcpy(tp.bytes, a->tm_payload, 128);
    memcpy(ts.bytes, a->tm_scale, 128);
    memcpy(tx.bytes, a->tm_x, 128);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a->plan.grid_x, a->plan.grid_y);
    cfg.blockDim = dim3(MMB_ST_THREADS);
    cfg.dynamicSmemBytes = a->plan.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = a->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, f4_stream_kernel<MT, GLU>, tp, ts, tx, p));
}

} // namespace mmb

extern "C" int mmb_stream_init(void)
{
    const void *kernels[8] = {
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<1, false>),
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<2, false>),
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<3, false>),
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<4, false>),
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<1, true>),
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<2, true>),
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<3, true>),
        reinterpret_cast<const void *>(mmb::f4_stream_kernel<4, true>),
    };
    for (const void *k : kernels) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, MMB_SMEM_MAX);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    return 0;
}

extern "C" int mmb_launch_stream(const mmb_args *a, void *stream)
{
    unsigned *status = nullptr;
    int e = mmb_status_word(&status);
    if (e) return e;
    if (a->plan.split_k > 1 && !a->ws)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->glu && a->n_dst)
        return static_cast<int>(cudaErrorInvalidValue);    /* the gated pair has no peer-store form */
    if (a->plan.tile_n == 0 || a->plan.tile_n % 16u != 0 || a->plan.tile_n > MMB_ST_ROWS ||
        (a->glu && a->plan.tile_n != MMB_ST_ROWS))
        return static_cast<int>(cudaErrorInvalidValue);
    switch (a->plan.m_tiles) {
    case 1: return a->glu ? mmb::launch_mt<1, true>(a, status, st) : mmb::launch_mt<1, false>(a, status, st);
    case 2: return a->glu ? mmb::launch_mt<2, true>(a, status, st) : mmb::launch_mt<2, false>(a, status, st);
    case 3: return a->glu ? mmb::launch_mt<3, true>(a, status, st) : mmb::launch_mt<3, false>(a, status, st);
    case 4: return a->glu ? mmb::launch_mt<4, true>(a, status, st) : mmb::launch_mt<4, false>(a, status, st);
    default: return static_cast<int>(cudaErrorInvalidValue);
    }
}

/* ==========================================================================
 * Decode op with built-in split-K scratch: mm_f4_linear_static_ws
 *
 * Same kernel as above, for callers that have no device block to donate as
 * split-K workspace and must not allocate one: an integrator that lives under
 * mimfer's start-up-only allocation policy (every byte of device memory is
 * carved into arenas by a handful of cudaMalloc calls at load and none may
 * follow), or a token loop that must never take the allocator's lock.  The
 * partial sums and arrival counters live in the file-scope device array below,
 * which every GPU that loads this library holds until the process exits.
 * ========================================================================== */
#include <cuda.h>
#include "../core/core.h"

#define MMB_STATIC_WS_BYTES (MMB_WS_COUNTER_B + (4u << 20))   /* 16 KiB counters + 4 MiB partials */
#define MMB_STATIC_MAX_DEVICES 16

static __device__ __align__(256) unsigned char g_static_ws[MMB_STATIC_WS_BYTES];

namespace {

typedef CUresult (*static_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                     const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                     const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct StaticWsDevice {
    bool  ready;
    void *ws;          /* device address of g_static_ws on this device */
    int   sm_count;
};
StaticWsDevice   g_static_dev[MMB_STATIC_MAX_DEVICES];
static_encode_fn g_static_encode;

/* Once per device, with that device current: the host-side name g_static_ws is
 * only a handle, the kernel needs the address cudaGetSymbolAddress returns. */
mm_status static_ws_setup(int dev)
{
    StaticWsDevice &d = g_static_dev[dev];
    if (d.ready)
        return MM_OK;
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_ws);
    if (e != cudaSuccess || !ptr) {
        MM_LOGE("static workspace: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return MM_ERR_CUDA;
    }
    if ((e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = static_cast<cudaError_t>(mmb_stream_init())) != cudaSuccess) {
        MM_LOGE("static workspace: device setup failed: %s", cudaGetErrorString(e));
        return MM_ERR_CUDA;
    }
    if (!g_static_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr);
        if (e != cudaSuccess || !fn || qr != cudaDriverEntryPointSuccess) {
            MM_LOGE("static workspace: cuTensorMapEncodeTiled not available");
            return MM_ERR_CUDA;
        }
        g_static_encode = reinterpret_cast<static_encode_fn>(fn);
    }
    d.ws = ptr;
    d.ready = true;
    return MM_OK;
}

bool static_encode(unsigned char out[128], CUtensorMapDataType dt, unsigned esize, const void *base,
                   uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                   CUtensorMapSwizzle sw)
{
    CUtensorMap map;
    cuuint64_t dims[2] = { inner, outer }, strides[1] = { inner * esize };
    cuuint32_t box[2] = { box_inner, box_outer }, estr[2] = { 1, 1 };
    if (g_static_encode(&map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    memcpy(out, &map, 128);
    return true;
}

} // namespace

extern "C" mm_status mm_f4_linear_static_ws(const void *x, const void *payload, const void *scale,
                                            float gs, void *y, uint32_t M, uint32_t K, uint32_t N,
                                            void *stream)
{
    if (!x || !payload || !scale || !y)
        return MM_ERR_STATE;
    if (M == 0 || N == 0 || K == 0 || K % 16 != 0)
        return MM_ERR_SHAPE;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MMB_STATIC_MAX_DEVICES)
        return MM_ERR_CUDA;
    mm_status st = static_ws_setup(dev);
    if (st != MM_OK)
        return st;
    const StaticWsDevice &d = g_static_dev[dev];

    mmb_args a;
    memset(&a, 0, sizeof a);
    a.x = x; a.payload = payload; a.scale = scale; a.y = y;
    a.gs = gs; a.M = M; a.K = K; a.N = N;
    a.ws = d.ws;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(payload) |
                           reinterpret_cast<uintptr_t>(scale) | reinterpret_cast<uintptr_t>(y) | 256u;
    /* the split the selector would choose with room to spare ... */
    mm_f4_shape sh = { M, K, N, static_cast<uint32_t>(d.sm_count),
                       static_cast<uint32_t>(bits & (~bits + 1u)), static_cast<size_t>(1) << 40 };
    st = mm_f4_select_variant(&sh, MM_F4_V_STREAM, &a.plan);
    if (st != MM_OK) {
        MM_LOGE("mm_f4_linear_static_ws serves the decode kernel only (M <= 32, K %% 256 == 0, "
                "16-byte aligned operands); M=%u K=%u N=%u: %s", M, K, N, mm_status_str(st));
        return st;
    }
    /* ... must fit the built-in array */
    if (a.plan.ws_needed > MMB_STATIC_WS_BYTES) {
        MM_LOGE("mm_f4_linear_static_ws: M=%u K=%u N=%u needs %zu bytes of split-K scratch, the "
                "built-in array holds %u", M, K, N, a.plan.ws_needed, MMB_STATIC_WS_BYTES);
        return MM_ERR_CAPACITY;
    }
    if (!static_encode(a.tm_payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, payload, K / 2, N, 128,
                       a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !static_encode(a.tm_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, scale, K / 16, N, 16,
                       a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !static_encode(a.tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, K, M, MMB_ST_KSTEP,
                       a.plan.tile_m, CU_TENSOR_MAP_SWIZZLE_NONE)) {
        MM_LOGE("mm_f4_linear_static_ws: tensor map encoding failed");
        return MM_ERR_CUDA;
    }
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    /* the array keeps what the last call left: the arrival counters must start at zero */
    if (a.plan.split_k > 1 &&
        cudaMemsetAsync(d.ws, 0, MMB_WS_COUNTER_B, cs) != cudaSuccess)
        return MM_ERR_CUDA;
    const int err = mmb_launch_stream(&a, cs);
    if (err) {
        MM_LOGE("mm_f4_linear_static_ws: launch failed: %s",
                cudaGetErrorString(static_cast<cudaError_t>(err)));
        return MM_ERR_CUDA;
    }
    return MM_OK;
}

/* Status word of the device, read on the caller's stream: for users of
 * mm_f4_linear_static_ws that run without the runtime shim.  Synchronises
 * `stream`, returns the MMB_DEV_* bits in *flags_out and clears them. */
extern "C" mm_status mm_f4_device_status_on(void *stream, unsigned *flags_out)
{
    if (!flags_out)
        return MM_ERR_STATE;
    unsigned *word = nullptr;
    if (mmb_status_word(&word) != 0 || !word)
        return MM_ERR_CUDA;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    unsigned v = 0;
    /* pageable destination: the copy has landed when the call returns */
    if (cudaMemcpyAsync(&v, word, sizeof v, cudaMemcpyDeviceToHost, cs) != cudaSuccess ||
        cudaStreamSynchronize(cs) != cudaSuccess)
        return MM_ERR_CUDA;
    if (v && (cudaMemsetAsync(word, 0, sizeof v, cs) != cudaSuccess || cudaStreamSynchronize(cs) != cudaSuccess))
        return MM_ERR_CUDA;
    *flags_out = v;
    return MM_OK;
}
