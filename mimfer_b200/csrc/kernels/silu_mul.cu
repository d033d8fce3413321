/*
 * SILU_MUL: y = silu(gate) * up on bf16 vectors, the unfused form of the gated
 * MLP (mimfer: src/kernels/cpu/cx.c:155-167, src/kernels/cuda/cx.cu:264-273).
 * HBM-bound elementwise op: 16-byte loads and stores, grid-stride, a grid of a
 * few CTAs per SM.  The fused form lives in the epilogues of the linear
 * kernels; this one serves shapes they cannot take.
 */
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

__device__ __forceinline__ uint32_t silu_mul2(uint32_t g2, uint32_t u2)
{
    const float g0 = __uint_as_float(g2 << 16), g1 = __uint_as_float(g2 & 0xffff0000u);
    const float u0 = __uint_as_float(u2 << 16), u1 = __uint_as_float(u2 & 0xffff0000u);
    return pack_bf16x2(silu_approx(g0) * u0, silu_approx(g1) * u1);
}

__global__ void __launch_bounds__(256) silu_mul_kernel(const uint16_t *__restrict__ gate,
                                                       const uint16_t *__restrict__ up,
                                                       uint16_t *__restrict__ y, size_t n, int vec)
{
    grid_dep_wait();
    const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    if (vec) {
        const size_t n8 = n / 8;
        const uint4 *g4 = reinterpret_cast<const uint4 *>(gate), *u4 = reinterpret_cast<const uint4 *>(up);
        uint4 *y4 = reinterpret_cast<uint4 *>(y);
        for (size_t i = tid; i < n8; i += stride) {
            const uint4 g = g4[i], u = u4[i];
            uint4 o;
            o.x = silu_mul2(g.x, u.x);
            o.y = silu_mul2(g.y, u.y);
            o.z = silu_mul2(g.z, u.z);
            o.w = silu_mul2(g.w, u.w);
            y4[i] = o;
        }
        for (size_t i = n8 * 8 + tid; i < n; i += stride)
            y[i] = static_cast<uint16_t>(silu_mul2(gate[i], up[i]) & 0xffffu);
    } else {
        for (size_t i = tid; i < n; i += stride)
            y[i] = static_cast<uint16_t>(silu_mul2(gate[i], up[i]) & 0xffffu);
    }
    grid_dep_launch();
}

} // namespace mmb

extern "C" int mmb_launch_silu_mul(const void *gate, const void *up, void *y, size_t n, void *stream)
{
    const uintptr_t bits = reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                           reinterpret_cast<uintptr_t>(y);
    const int vec = (bits & 15u) == 0;
    size_t blocks = (n / (vec ? 8 : 1) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    mmb::silu_mul_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t *>(gate), static_cast<const uint16_t *>(up),
        static_cast<uint16_t *>(y), n, vec);
    return static_cast<int>(cudaGetLastError());
}
