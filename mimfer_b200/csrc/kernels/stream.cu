/*
 * STREAM: the decode kernel of the NVFP4 linear op (M <= 32, HBM-bound).
 *
 * One CTA owns 256 weight rows and a contiguous range of 256-wide K steps.
 * A producer warp keeps a ring of stages full: per step one TMA box of packed
 * payload (256 rows x 128 B, 128-byte swizzle), one of block scales
 * (256 rows x 16 B), and the matching slice of the activations, which it
 * re-orders on the way into shared memory (see below).  Eight consumer warps
 * each take 32 rows: 16-byte shared loads of payload, nibble unpack and scale
 * in registers (fp4.cuh), bf16 warp MMAs with the weights as the 16-row
 * operand and up to 32 activation rows as the 8-wide operand, fp32
 * accumulators in registers.  With split-K the partial sums meet in the
 * workspace and the CTA that arrives last adds them in slice order, so the
 * result does not depend on scheduling (no atomics on data; the reference
 * demands order-faithful reductions, include/mimfer/kernels.h:14-15).
 *
 * Operand order inside a K step.  Lane (g, t) of a consumer warp (g = lane/4,
 * t = lane%4) owns the 64 weights [64t, 64t+64) of each of its rows, as eight
 * 32-bit words of eight nibbles.  A word is unpacked into the pairs (n0,n4)
 * (n1,n5) (n2,n6) (n3,n7) because both halves of such a pair need the same
 * shifts.  The MMA sums over K, so any order works as long as both operands
 * agree: the producer stores each group of eight activations as
 * (x0,x4,x1,x5,x2,x6,x3,x7), at [word][row][t], which also makes the
 * consumers' 16-byte reads conflict-free.
 *
 * It replaces the one-thread-per-output kernel of the reference
 * (src/kernels/cuda/cx.cu:345-356) for the decode regime.
 */
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

struct StreamParams {
    const uint16_t *x;
    uint16_t       *y;
    float          *partial;     /* workspace + MMB_WS_COUNTER_B, or NULL */
    unsigned       *counters;    /* workspace base, or NULL               */
    unsigned       *status;
    float           gs;
    uint32_t        M, K, N;
    uint32_t        k_steps, split_k, stages;
};

template <int MT>
__global__ void __launch_bounds__(MMB_ST_THREADS, 1)
f4_stream_kernel(const __grid_constant__ TmaDesc tm_payload,
                 const __grid_constant__ TmaDesc tm_scale, const StreamParams p)
{
    constexpr uint32_t MPAD = MT * 8;
    constexpr uint32_t STAGE_B = MMB_ST_STAGE_B(MT);
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t lut = base + p.stages * STAGE_B;
    const uint32_t bar_full = lut + 1024u;
    const uint32_t bar_empty = bar_full + 8u * p.stages;
    const uint32_t last_flag = bar_empty + 8u * p.stages;    /* split-K: "this CTA reduces" */

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t row0 = blockIdx.x * MMB_ST_ROWS;
    const uint32_t ks_begin = static_cast<uint32_t>(
        static_cast<uint64_t>(p.k_steps) * blockIdx.y / p.split_k);
    const uint32_t ks_end = static_cast<uint32_t>(
        static_cast<uint64_t>(p.k_steps) * (blockIdx.y + 1) / p.split_k);
    const uint32_t nsteps = ks_end - ks_begin;

    if (tid < 256u)
        sts32(lut + tid * 4u, scale_lut_entry(tid));
    if (tid == 0) {
        for (uint32_t s = 0; s < p.stages; s++) {
            mbar_init(bar_full + 8u * s, 33u);                 /* expect_tx + 32 lanes */
            mbar_init(bar_empty + 8u * s, MMB_ST_CONSUMERS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == MMB_ST_CONSUMERS) {
        /* ------------------------------ producer ------------------------- */
        const uint32_t t = lane & 3u, w = lane >> 2;          /* chunk = 8t + w */
        for (uint32_t it = 0; it < nsteps; it++) {
            const uint32_t s = it % p.stages, round = it / p.stages;
            const uint32_t stage = base + s * STAGE_B;
            if (round > 0)
                mbar_wait(bar_empty + 8u * s, (round - 1u) & 1u, p.status);
            const uint32_t ks = ks_begin + it;
            if (lane == 0) {
                mbar_expect_tx(bar_full + 8u * s, MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B);
                tma_load_2d(stage, &tm_payload, static_cast<int>(ks * 128u),
                            static_cast<int>(row0), bar_full + 8u * s);
                tma_load_2d(stage + MMB_ST_PAYLOAD_B, &tm_scale, static_cast<int>(ks * 16u),
                            static_cast<int>(row0), bar_full + 8u * s);
            }
            const uint32_t xs = stage + MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B;
            const uint16_t *xk = p.x + static_cast<size_t>(ks) * MMB_ST_KSTEP + (8u * t + w) * 8u;
#pragma unroll
            for (uint32_t m = 0; m < MPAD; m++) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (m < p.M)
                    v = __ldg(reinterpret_cast<const uint4 *>(xk + static_cast<size_t>(m) * p.K));
                uint4 o;
                o.x = prmt(v.x, v.z, 0x5410u);                 /* x0 x4 */
                o.y = prmt(v.x, v.z, 0x7632u);                 /* x1 x5 */
                o.z = prmt(v.y, v.w, 0x5410u);                 /* x2 x6 */
                o.w = prmt(v.y, v.w, 0x7632u);                 /* x3 x7 */
                sts128(xs + ((w * MPAD + m) * 4u + t) * 16u, o);
            }
            mbar_arrive(bar_full + 8u * s);
        }
        return;
    }

    /* --------------------------------- consumers ------------------------- */
    const uint32_t g = lane >> 2, t = lane & 3u;
    float acc[2][MT][4];
#pragma unroll
    for (int rt = 0; rt < 2; rt++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[rt][mt][i] = 0.0f;

    for (uint32_t it = 0; it < nsteps; it++) {
        const uint32_t s = it % p.stages, round = it / p.stages;
        const uint32_t stage = base + s * STAGE_B;
        mbar_wait(bar_full + 8u * s, round & 1u, p.status);
        const uint32_t pay = stage, scl = stage + MMB_ST_PAYLOAD_B;
        const uint32_t xs = scl + MMB_ST_SCALE_B;

        uint32_t scw[2][2];                                    /* 4 scale bytes per row */
#pragma unroll
        for (int rt = 0; rt < 2; rt++)
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                const uint32_t row = warp * 32u + rt * 16u + rr * 8u + g;
                scw[rt][rr] = lds32(scl + row * 16u + t * 4u);
            }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint4 pw[2][2];
#pragma unroll
            for (int rt = 0; rt < 2; rt++)
#pragma unroll
                for (int rr = 0; rr < 2; rr++) {
                    const uint32_t row = warp * 32u + rt * 16u + rr * 8u + g;
                    pw[rt][rr] = lds128(pay + row * 128u + (((2u * t + h) ^ g) << 4));
                }
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
                const uint32_t word = 4u * h + wi;
                uint4 xb[MT];
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
                    xb[mt] = lds128(xs + ((word * MPAD + mt * 8u + g) * 4u + t) * 16u);
#pragma unroll
                for (int rt = 0; rt < 2; rt++) {
                    uint32_t q0[4], q8[4];
                    const uint32_t sb = 2u * h + (wi >> 1);
                    const uint32_t c0 = lds32(lut + ((scw[rt][0] >> (8u * sb)) & 255u) * 4u);
                    const uint32_t c8 = lds32(lut + ((scw[rt][1] >> (8u * sb)) & 255u) * 4u);
                    const uint32_t w0 = wi == 0 ? pw[rt][0].x : wi == 1 ? pw[rt][0].y
                                      : wi == 2 ? pw[rt][0].z : pw[rt][0].w;
                    const uint32_t w8 = wi == 0 ? pw[rt][1].x : wi == 1 ? pw[rt][1].y
                                      : wi == 2 ? pw[rt][1].z : pw[rt][1].w;
                    unpack8_paired(w0, c0, q0);
                    unpack8_paired(w8, c8, q8);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        mma_bf16_16816(acc[rt][mt], q0[0], q8[0], q0[1], q8[1], xb[mt].x, xb[mt].y);
                        mma_bf16_16816(acc[rt][mt], q0[2], q8[2], q0[3], q8[3], xb[mt].z, xb[mt].w);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(bar_empty + 8u * s);
    }

    /* --------------------------------- epilogue -------------------------- */
    const float out_scale = p.gs * 256.0f;          /* undo the 2^-8 of the operand form */
    if (p.split_k == 1) {
#pragma unroll
        for (int rt = 0; rt < 2; rt++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t n = row0 + warp * 32u + rt * 16u + (i >> 1) * 8u + g;
                    const uint32_t m = mt * 8u + 2u * t + (i & 1);
                    if (n < p.N && m < p.M) {
                        __nv_bfloat16 hv = __float2bfloat16_rn(acc[rt][mt][i] * out_scale);
                        p.y[static_cast<size_t>(m) * p.N + n] = *reinterpret_cast<uint16_t *>(&hv);
                    }
                }
        return;
    }

    /* split-K: publish this slice, the last CTA of the row block reduces */
    float *mine = p.partial + static_cast<size_t>(blockIdx.y) * MPAD * p.N;
#pragma unroll
    for (int rt = 0; rt < 2; rt++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t n = row0 + warp * 32u + rt * 16u + (i >> 1) * 8u + g;
                const uint32_t m = mt * 8u + 2u * t + (i & 1);
                if (n < p.N && m < p.M)
                    __stcg(mine + static_cast<size_t>(m) * p.N + n, acc[rt][mt][i]);
            }
    __threadfence();
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (tid == 0) {
        const unsigned ticket = atomicAdd(p.counters + blockIdx.x, 1u);
        sts32(last_flag, (ticket == p.split_k - 1u) ? 1u : 0u);
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!lds32(last_flag))
        return;
    __threadfence();
#pragma unroll
    for (int rt = 0; rt < 2; rt++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t n = row0 + warp * 32u + rt * 16u + (i >> 1) * 8u + g;
                const uint32_t m = mt * 8u + 2u * t + (i & 1);
                if (n < p.N && m < p.M) {
                    float sum = 0.0f;
                    for (uint32_t sl = 0; sl < p.split_k; sl++)
                        sum += __ldcg(p.partial + (static_cast<size_t>(sl) * MPAD + m) * p.N + n);
                    __nv_bfloat16 hv = __float2bfloat16_rn(sum * out_scale);
                    p.y[static_cast<size_t>(m) * p.N + n] = *reinterpret_cast<uint16_t *>(&hv);
                }
            }
    if (tid == 0)
        p.counters[blockIdx.x] = 0u;                /* ready for the next launch */
}

template <int MT>
static int launch_mt(const mmb_args *a, unsigned *status, cudaStream_t st)
{
    StreamParams p;
    p.x = static_cast<const uint16_t *>(a->x);
    p.y = static_cast<uint16_t *>(a->y);
    p.counters = static_cast<unsigned *>(a->ws);
    p.partial = a->ws ? reinterpret_cast<float *>(static_cast<unsigned char *>(a->ws) + MMB_WS_COUNTER_B)
                      : nullptr;
    p.status = status;
    p.gs = a->gs;
    p.M = a->M; p.K = a->K; p.N = a->N;
    p.k_steps = a->plan.k_steps;
    p.split_k = a->plan.split_k;
    p.stages = a->plan.stages;
    TmaDesc tp, ts;
    memcpy(tp.bytes, a->tm_payload, 128);
    memcpy(ts.bytes, a->tm_scale, 128);
    dim3 grid(a->plan.grid_x, a->plan.grid_y), block(MMB_ST_THREADS);
    f4_stream_kernel<MT><<<grid, block, a->plan.smem_bytes, st>>>(tp, ts, p);
    return static_cast<int>(cudaGetLastError());
}

} // namespace mmb

extern "C" int mmb_stream_init(void)
{
    cudaError_t e;
    e = cudaFuncSetAttribute(mmb::f4_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             MMB_SMEM_MAX);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(mmb::f4_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             MMB_SMEM_MAX);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(mmb::f4_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             MMB_SMEM_MAX);
    return static_cast<int>(e);
}

extern "C" int mmb_launch_stream(const mmb_args *a, void *stream)
{
    unsigned *status = nullptr;
    int e = mmb_status_word(&status);
    if (e) return e;
    if (a->plan.split_k > 1 && !a->ws)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (a->plan.m_tiles) {
    case 1: return mmb::launch_mt<1>(a, status, st);
    case 2: return mmb::launch_mt<2>(a, status, st);
    case 4: return mmb::launch_mt<4>(a, status, st);
    default: return static_cast<int>(cudaErrorInvalidValue);
    }
}
