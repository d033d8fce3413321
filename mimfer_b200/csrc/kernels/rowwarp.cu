/*
 * Row-warp NVFP4 linear: the variant that takes every legal shape
 * (K % 16 == 0, any M and N).  One warp owns one weight row; its lanes walk
 * the row in 16-weight blocks (8 payload bytes + 1 scale byte per block),
 * dequantise in registers with the fp32 decode and keep one fp32 accumulator
 * per activation row; the K reduction is a warp shuffle tree.  It replaces
 * the thread-per-output kernel of the reference (src/kernels/cuda/cx.cu:345-356)
 * for shapes the TMA-fed kernels cannot take, and hosts the decode probe.
 */
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

__device__ unsigned int g_status_word;

constexpr int RW_MB = 4;    /* activation rows per pass */

__global__ void __launch_bounds__(256)
f4_rowwarp_kernel(const uint16_t *__restrict__ x, const uint8_t *__restrict__ payload,
                  const uint8_t *__restrict__ scale, uint16_t *__restrict__ y, float gs,
                  uint32_t M, uint32_t K, uint32_t N, uint32_t ldy, uint32_t col0)
{
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t r = blockIdx.x * 8u + warp;
    if (r >= N)
        return;
    const uint32_t nblk = K / 16u;
    const uint8_t *prow = payload + static_cast<size_t>(r) * (K / 2u);
    const uint8_t *srow = scale + static_cast<size_t>(r) * nblk;

    for (uint32_t m0 = blockIdx.y * RW_MB; m0 < M; m0 += gridDim.y * RW_MB) {
        float acc[RW_MB];
#pragma unroll
        for (int i = 0; i < RW_MB; i++) acc[i] = 0.0f;
        for (uint32_t b = lane; b < nblk; b += 32u) {
            const uint2 pw = *reinterpret_cast<const uint2 *>(prow + b * 8u);
            const float sc = e4m3_f32(srow[b]);
            float w[16];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                w[j] = e2m1_f32((pw.x >> (4 * j)) & 15u) * sc;
                w[8 + j] = e2m1_f32((pw.y >> (4 * j)) & 15u) * sc;
            }
#pragma unroll
            for (int i = 0; i < RW_MB; i++) {
                if (m0 + i < M) {
                    const uint4 *xp = reinterpret_cast<const uint4 *>(
                        x + static_cast<size_t>(m0 + i) * K + b * 16u);
                    const uint4 xa = xp[0], xb = xp[1];
                    const uint32_t xs[8] = { xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w };
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        acc[i] = fmaf(__uint_as_float(xs[j] << 16), w[2 * j], acc[i]);
                        acc[i] = fmaf(__uint_as_float(xs[j] & 0xffff0000u), w[2 * j + 1], acc[i]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < RW_MB; i++) {
            float v = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m0 + i < M) {
                __nv_bfloat16 h = __float2bfloat16_rn(v * gs);
                y[static_cast<size_t>(m0 + i) * ldy + col0 + r] = *reinterpret_cast<uint16_t *>(&h);
            }
        }
    }
}

/* index = s * 16 + n.  out_mma: the bf16 operand form, every one of the eight
 * nibble positions of a word must agree, else 0xdeadbeef is written.
 * out_f16: the fp16 operand form, same rule plus the column order check. */
__global__ void f4_decode_probe_kernel(uint32_t *out_mma, uint32_t *out_f32, uint32_t *out_f16)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 4096u)
        return;
    const uint32_t s = i >> 4, n = i & 15u;
    out_f32[i] = __float_as_uint(e2m1_f32(n) * e4m3_f32(s));

    const uint32_t c = scale_lut_entry(s);
    uint32_t q[4];
    unpack8_paired(n * 0x11111111u, c, q);
    const uint4 nat = unpack8_natural(n * 0x11111111u, c);
    const uint32_t first = q[0] & 0xffffu;
    bool same = true;
#pragma unroll
    for (int j = 0; j < 4; j++)
        same = same && (q[j] & 0xffffu) == first && (q[j] >> 16) == first;
    same = same && nat.x == q[0] && nat.y == q[0] && nat.z == q[0] && nat.w == q[0];
    const float v = __uint_as_float(first << 16) * 256.0f;
    out_mma[i] = same ? __float_as_uint(v) : 0xdeadbeefu;

    /* fp16 operand form: nibble n in all eight positions, then one position at a time */
    const uint4 hf = unpack8_natural_f16(n * 0x11111111u, scale_lut_entry_f16(s));
    const uint32_t h0 = hf.x & 0xffffu;
    bool same16 = hf.x == (h0 | (h0 << 16)) && hf.y == hf.x && hf.z == hf.x && hf.w == hf.x;
#pragma unroll
    for (int pos = 0; pos < 8; pos++) {          /* column order: nibble `pos` lands in slot `pos` */
        const uint4 one = unpack8_natural_f16(n << (4 * pos), scale_lut_entry_f16(s));
        const uint32_t regs[4] = { one.x, one.y, one.z, one.w };
        const uint32_t got = (regs[pos >> 1] >> (16 * (pos & 1))) & 0xffffu;
        same16 = same16 && got == h0;
    }
    const __half hv = *reinterpret_cast<const __half *>(&h0);
    out_f16[i] = same16 ? __float_as_uint(__half2float(hv)) : 0xdeadbeefu;
}

/* Bounded-wait self test: one thread waits on an mbarrier that nothing ever
 * completes.  The wait must give up after its limit, raise MMB_DEV_TIMEOUT in
 * the status word and let the kernel return normally. */
__global__ void f4_wait_selftest_kernel(unsigned *status, unsigned *done)
{
    __shared__ alignas(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1u);
        mbar_fence_init();
        const bool ok = mbar_wait(b, 0u, status);       /* never arrives */
        *done = ok ? 2u : 1u;
    }
}

} // namespace mmb

extern "C" int mmb_launch_wait_selftest(unsigned *status, unsigned *done, void *stream)
{
    mmb::f4_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, done);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mmb_launch_rowwarp(const mmb_args *a, void *stream)
{
    dim3 grid(a->plan.grid_x, a->plan.grid_y), block(a->plan.threads);
    /* tensor parallel: one launch per destination (this kernel is the untuned fallback) */
    const uint32_t nd = a->n_dst ? a->n_dst : 1u;
    for (uint32_t d = 0; d < nd; d++) {
        uint16_t *y = static_cast<uint16_t *>(a->n_dst ? a->y_dst[d] : a->y);
        mmb::f4_rowwarp_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint16_t *>(a->x), static_cast<const uint8_t *>(a->payload),
            static_cast<const uint8_t *>(a->scale), y, a->gs, a->M, a->K, a->N,
            a->n_dst ? a->ldy : a->N, a->n_dst ? a->col0 : 0u);
    }
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mmb_launch_decode_probe(uint32_t *out_mma, uint32_t *out_f32, uint32_t *out_f16,
                                       void *stream)
{
    mmb::f4_decode_probe_kernel<<<16, 256, 0, static_cast<cudaStream_t>(stream)>>>(out_mma, out_f32,
                                                                                  out_f16);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mmb_status_word(unsigned **dev_ptr)
{
    return static_cast<int>(cudaGetSymbolAddress(reinterpret_cast<void **>(dev_ptr),
                                                 mmb::g_status_word));
}
