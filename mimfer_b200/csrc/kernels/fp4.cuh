/*
 * NVFP4 decode on the device.  Two forms, both bit-exact with the mimfer
 * decoders (include/mimfer/tensor.h:90-118):
 *
 *  fp32 form   e2m1_f32(n) * e4m3_f32(s), used by the row-warp kernel.
 *
 *  bf16 operand form, used by both tensor-core kernels.  A nibble's three
 *  magnitude bits (e1 e0 m) are placed at bits 8..6 of a bf16: the exponent
 *  field becomes e and the top mantissa bit m, which reads as the e2m1 value
 *  times 2^-126 for every code, the two subnormal codes (0, 0.5) included
 *  because a bf16 with exponent field 0 is subnormal in the same way.  One
 *  packed bf16 multiply by (e4m3 scale * 2^118), looked up from a 256-entry
 *  table so that 0x7f/0xff give 0 and the scale's sign is kept, yields
 *  value * scale * 2^-8 exactly: e2m1 x e4m3 needs at most 6 significant
 *  bits.  The 2^8 is returned in the epilogue together with the global scale.
 */
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace mmb {

__device__ __forceinline__ float e4m3_f32(uint32_t b)
{
    if ((b & 0x7fu) == 0x7fu)
        return 0.0f;
    uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float mag = e ? __uint_as_float(((e + 120u) << 23) | (m << 20))
                  : static_cast<float>(m) * 0.001953125f;          /* m * 2^-9 */
    return (b & 0x80u) ? -mag : mag;
}

__device__ __forceinline__ float e2m1_f32(uint32_t n)
{
    uint32_t e = (n >> 1) & 3u, m = n & 1u;
    float mag = e ? __uint_as_float(((e + 126u) << 23) | (m << 22)) : 0.5f * static_cast<float>(m);
    return (n & 8u) ? -mag : mag;
}

/* Table entry for scale byte b: bf16x2 (c, c) with c = e4m3(b) * 2^118. */
__device__ __forceinline__ uint32_t scale_lut_entry(uint32_t b)
{
    float c = e4m3_f32(b) * 3.3230699894622813e35f;                /* 2^118, exact */
    uint32_t hi = __float_as_uint(c) >> 16;                        /* <= 4 significant bits */
    return hi | (hi << 16);
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

/* Eight nibbles n0..n7 of `w` (n0 lowest) -> four bf16x2 registers holding
 * (n0,n4) (n1,n5) (n2,n6) (n3,n7), low half first, each already multiplied by
 * the scale entry c.  nibble * 0x1040 copies the nibble to bits 15..12 and
 * 9..6 of its half-word; the mask keeps the sign at bit 15 and the magnitude
 * at bits 8..6. */
__device__ __forceinline__ void unpack8_paired(uint32_t w, uint32_t c, uint32_t (&q)[4])
{
    const uint32_t keep = 0x81c081c0u;
    uint32_t hi = w >> 8;
    q[0] = mul_bf16x2(((w & 0x000f000fu) * 0x1040u) & keep, c);
    q[1] = mul_bf16x2(((w & 0x00f000f0u) * 0x0104u) & keep, c);
    q[2] = mul_bf16x2(((hi & 0x000f000fu) * 0x1040u) & keep, c);
    q[3] = mul_bf16x2(((hi & 0x00f000f0u) * 0x0104u) & keep, c);
}

/* Same eight weights in column order: (n0,n1) (n2,n3) (n4,n5) (n6,n7). */
__device__ __forceinline__ uint4 unpack8_natural(uint32_t w, uint32_t c)
{
    uint32_t q[4];
    unpack8_paired(w, c, q);
    uint4 r;
    r.x = prmt(q[0], q[1], 0x5410u);
    r.y = prmt(q[2], q[3], 0x5410u);
    r.z = prmt(q[0], q[1], 0x7632u);
    r.w = prmt(q[2], q[3], 0x7632u);
    return r;
}

/* ---- fp16 operand form -------------------------------------------------
 * cvt.rn.f16x2.e2m1x2 turns one payload byte (two nibbles) into two fp16
 * values, low nibble in the low half, i.e. already in column order.  e4m3
 * scales and the e2m1 x e4m3 products (at most 6 significant bits, magnitude
 * 2^-10 .. 2688) are exact fp16 normals, so one packed fp16 multiply by the
 * scale entry gives the dequantised weight exactly, with no exponent offset.
 * This is the main path of the CUDA-core decode kernel (stream.cu): a K step whose
 * activations all convert to fp16 exactly takes it.  The prefill kernel cannot:
 * tcgen05 kind::f16 wants both operands in one format and its activations stay
 * bf16. */
__device__ __forceinline__ uint32_t scale_lut_entry_f16(uint32_t b)
{
    const __half h = __float2half_rn(e4m3_f32(b));                 /* exact */
    const uint32_t u = *reinterpret_cast<const uint16_t *>(&h);
    return u | (u << 16);
}

/* The four e4m3 scales of `sc4` (byte j = scale j) as four fp16x2 registers
 * (c, c), by cvt.rn.f16x2.e4m3x2 instead of a table in shared memory: every
 * e4m3 value is an exact fp16, the sign is kept.  The two NaN codes 0x7f and
 * 0xff must read as 0.0 (include/mimfer/tensor.h:100-101): such bytes are
 * cleared first, 0x00 converts to +0. */
__device__ __forceinline__ void scales4_f16(uint32_t sc4, uint32_t (&c)[4])
{
    const uint32_t nan = (((sc4 & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) >> 7;   /* 1 per NaN byte */
    if (nan)
        sc4 &= ~(nan * 0xffu);
    uint32_t lo, hi;
    asm("{\n\t"
        ".reg .b16 a, b;\n\t"
        "mov.b32 {a, b}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, a;\n\t"
        "cvt.rn.f16x2.e4m3x2 %1, b;\n\t"
        "}"
        : "=r"(lo), "=r"(hi) : "r"(sc4));
    c[0] = prmt(lo, lo, 0x1010u);
    c[1] = prmt(lo, lo, 0x3232u);
    c[2] = prmt(hi, hi, 0x1010u);
    c[3] = prmt(hi, hi, 0x3232u);
}

__device__ __forceinline__ uint4 unpack8_natural_f16(uint32_t w, uint32_t c)
{
    uint4 r;
    asm("{\n\t"
        ".reg .b8 b0, b1, b2, b3;\n\t"
        ".reg .b32 t0, t1, t2, t3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 t0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 t1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 t2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 t3, b3;\n\t"
        "mul.rn.f16x2 %0, t0, %5;\n\t"
        "mul.rn.f16x2 %1, t1, %5;\n\t"
        "mul.rn.f16x2 %2, t2, %5;\n\t"
        "mul.rn.f16x2 %3, t3, %5;\n\t"
        "}"
        : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
        : "r"(w), "r"(c));
    return r;
}

/* silu(g) = g / (1 + exp(-g)) with the two special-function-unit approximations
 * (ex2.approx and rcp.approx, the non-flushing forms: full range, subnormal
 * results kept, relative error about 2^-22 each).  A few dozen fp32 ulps at the
 * ends of the range, far below half a bf16 step, so after the bf16 rounding that
 * follows it the result differs from an expf-and-divide evaluation only on
 * near-ties.  Limits as the division gives them: +inf -> +inf, -inf -> NaN,
 * large negative g -> small negative values down to -0. */
__device__ __forceinline__ float silu_approx(float g)
{
    float e, r;
    asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
    asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r;
}

/* Two outputs of silu(gate) * up on the two projections rounded to bf16 first:
 * the arithmetic of the reference's separate op (src/kernels/cpu/cx.c:155-167)
 * on the values its two GEMMs would have stored, for kernels that fuse the three
 * ops.  Returns the packed bf16 pair (first output in the low half). */
__device__ __forceinline__ uint32_t glu_out_bf16x2(float gate0, float gate1, float up0, float up1,
                                                   float gate_scale, float up_scale)
{
    const __nv_bfloat162 gq = __floats2bfloat162_rn(gate0 * gate_scale, gate1 * gate_scale);
    const __nv_bfloat162 uq = __floats2bfloat162_rn(up0 * up_scale, up1 * up_scale);
    const uint32_t gb = *reinterpret_cast<const uint32_t *>(&gq);
    const uint32_t ub = *reinterpret_cast<const uint32_t *>(&uq);
    const float y0 = silu_approx(__uint_as_float(gb << 16)) * __uint_as_float(ub << 16);
    const float y1 = silu_approx(__uint_as_float(gb & 0xffff0000u)) * __uint_as_float(ub & 0xffff0000u);
    const __nv_bfloat162 o = __floats2bfloat162_rn(y0, y1);
    return *reinterpret_cast<const uint32_t *>(&o);
}

__device__ __forceinline__ uint16_t glu_out_bf16(float gate_acc, float up_acc, float gate_scale,
                                                 float up_scale)
{
    return static_cast<uint16_t>(glu_out_bf16x2(gate_acc, 0.0f, up_acc, 0.0f, gate_scale, up_scale) & 0xffffu);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

} // namespace mmb
