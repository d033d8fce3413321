/*
 * ADD_RMSNORM: res += delta (in place), y = rmsnorm(res) * gain, on bf16 rows
 * (mimfer: src/kernels/cpu/cx.c:70-84,132-150; src/kernels/cuda/cx.cu:223-243,
 * one thread per row there).  The reference planner emits it after every
 * attention block and after every MLP, i.e. right behind the o and down
 * projections (src/plan/plan.c:440-449).
 *
 * One CTA per row, 16-byte loads.  The sum res + delta is rounded to bf16
 * first, exactly as the reference stores it, and the squares of the rounded
 * values are added in fp32: per thread in ascending order, then over the CTA
 * in a fixed tree, so the result is the same from run to run.  The reference
 * adds the H squares strictly left to right; the two orders differ in the
 * last bits of the fp32 sum, which moves an output by one bf16 step at most.
 * HBM/L2-bound and tiny: M rows of H values.
 */
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

#define MMB_NORM_THREADS 256u
#define MMB_NORM_KEEP    4u        /* 16-byte chunks a thread keeps in registers (H <= 8192) */

__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b, float &ss)
{
    const float s0 = __uint_as_float(a << 16) + __uint_as_float(b << 16);
    const float s1 = __uint_as_float(a & 0xffff0000u) + __uint_as_float(b & 0xffff0000u);
    const uint32_t r = pack_bf16x2(s0, s1);
    const float v0 = __uint_as_float(r << 16), v1 = __uint_as_float(r & 0xffff0000u);
    ss += v0 * v0;
    ss += v1 * v1;
    return r;
}

__device__ __forceinline__ uint32_t norm_bf16x2(uint32_t r, uint32_t g, float inv)
{
    const float y0 = __uint_as_float(r << 16) * inv * __uint_as_float(g << 16);
    const float y1 = __uint_as_float(r & 0xffff0000u) * inv * __uint_as_float(g & 0xffff0000u);
    return pack_bf16x2(y0, y1);
}

__global__ void __launch_bounds__(MMB_NORM_THREADS)
add_rmsnorm_kernel(uint16_t *__restrict__ res, const uint16_t *__restrict__ delta, uint16_t *__restrict__ y,
                   const uint16_t *__restrict__ gain, uint32_t H, float eps, int vec)
{
    __shared__ float s_part[MMB_NORM_THREADS / 32u];
    __shared__ float s_inv;
    grid_dep_wait();
    grid_dep_launch();
    const uint32_t tid = threadIdx.x;
    uint16_t *rr = res + static_cast<size_t>(blockIdx.x) * H;
    const uint16_t *dr = delta + static_cast<size_t>(blockIdx.x) * H;
    uint16_t *yr = y + static_cast<size_t>(blockIdx.x) * H;
    float ss = 0.0f;
    uint4 keep[MMB_NORM_KEEP];
    const uint32_t chunks = vec ? H / 8u : 0u;
    if (vec) {
        uint4 *r4 = reinterpret_cast<uint4 *>(rr);
        const uint4 *d4 = reinterpret_cast<const uint4 *>(dr);
#pragma unroll
        for (uint32_t j = 0; j < MMB_NORM_KEEP; j++) {
            const uint32_t i = tid + j * MMB_NORM_THREADS;
            if (i < chunks) {
                const uint4 a = r4[i], b = d4[i];
                uint4 o;
                o.x = add_bf16x2(a.x, b.x, ss);
                o.y = add_bf16x2(a.y, b.y, ss);
                o.z = add_bf16x2(a.z, b.z, ss);
                o.w = add_bf16x2(a.w, b.w, ss);
                r4[i] = o;
                keep[j] = o;
            }
        }
        for (uint32_t i = tid + MMB_NORM_KEEP * MMB_NORM_THREADS; i < chunks; i += MMB_NORM_THREADS) {
            const uint4 a = r4[i], b = d4[i];
            uint4 o;
            o.x = add_bf16x2(a.x, b.x, ss);
            o.y = add_bf16x2(a.y, b.y, ss);
            o.z = add_bf16x2(a.z, b.z, ss);
            o.w = add_bf16x2(a.w, b.w, ss);
            r4[i] = o;
        }
    }
    for (uint32_t i = chunks * 8u + tid; i < H; i += MMB_NORM_THREADS) {     /* tail, or everything when unaligned */
        float dummy = 0.0f;
        const uint32_t r = add_bf16x2(rr[i], dr[i], dummy) & 0xffffu;
        rr[i] = static_cast<uint16_t>(r);
        const float v = __uint_as_float(r << 16);
        ss += v * v;
    }
    /* fixed tree: lanes, then warps */
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31u) == 0)
        s_part[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
        for (uint32_t w = 0; w < MMB_NORM_THREADS / 32u; w++) t += s_part[w];
        s_inv = 1.0f / sqrtf(t / static_cast<float>(H) + eps);
    }
    __syncthreads();
    const float inv = s_inv;
    if (vec) {
        uint4 *y4 = reinterpret_cast<uint4 *>(yr);
        const uint4 *g4 = reinterpret_cast<const uint4 *>(gain);
        const uint4 *r4 = reinterpret_cast<const uint4 *>(rr);
#pragma unroll
        for (uint32_t j = 0; j < MMB_NORM_KEEP; j++) {
            const uint32_t i = tid + j * MMB_NORM_THREADS;
            if (i < chunks) {
                const uint4 g = g4[i];
                uint4 o;
                o.x = norm_bf16x2(keep[j].x, g.x, inv);
                o.y = norm_bf16x2(keep[j].y, g.y, inv);
                o.z = norm_bf16x2(keep[j].z, g.z, inv);
                o.w = norm_bf16x2(keep[j].w, g.w, inv);
                y4[i] = o;
            }
        }
        for (uint32_t i = tid + MMB_NORM_KEEP * MMB_NORM_THREADS; i < chunks; i += MMB_NORM_THREADS) {
            const uint4 r = r4[i], g = g4[i];       /* this thread's own stores of the first pass */
            uint4 o;
            o.x = norm_bf16x2(r.x, g.x, inv);
            o.y = norm_bf16x2(r.y, g.y, inv);
            o.z = norm_bf16x2(r.z, g.z, inv);
            o.w = norm_bf16x2(r.w, g.w, inv);
            y4[i] = o;
        }
    }
    for (uint32_t i = chunks * 8u + tid; i < H; i += MMB_NORM_THREADS)
        yr[i] = static_cast<uint16_t>(norm_bf16x2(rr[i], gain[i], inv) & 0xffffu);
}

} // namespace mmb

extern "C" int mmb_launch_add_rmsnorm(void *res, const void *delta, void *y, const void *gain, uint32_t M,
                                      uint32_t H, float eps, int pdl, void *stream)
{
    const uintptr_t bits = reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(delta) |
                           reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gain);
    const int vec = (bits & 15u) == 0 && H % 8u == 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(MMB_NORM_THREADS);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, mmb::add_rmsnorm_kernel, static_cast<uint16_t *>(res),
                                               static_cast<const uint16_t *>(delta), static_cast<uint16_t *>(y),
                                               static_cast<const uint16_t *>(gain), H, eps, vec));
}
