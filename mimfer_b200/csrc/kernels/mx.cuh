/*
 * Pieces shared by the kernels of the block-scaled decode path (mx.cu: one op
 * per launch; mxg.cu: a group of independent ops per launch): the tcgen05
 * wrappers ptx.cuh does not have, the tensor-memory map and the plane sum.
 */
#pragma once
#include "fp4.cuh"
#include "ptx.cuh"

namespace mmb {

/* ---- tcgen05 pieces this file adds to ptx.cuh -------------------------------- */
/* one instruction for a whole 64-column slot: a tcgen05.st costs several hundred
 * cycles whatever its width (measured), so the slot goes out in one */
__device__ __forceinline__ void tmem_st_x64(uint32_t taddr, const uint32_t (&v)[64])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x64.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,"
        "%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,"
        "%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63,%64};"
        ::"r"(taddr),
          "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]),
          "r"(v[32]), "r"(v[33]), "r"(v[34]), "r"(v[35]), "r"(v[36]), "r"(v[37]), "r"(v[38]), "r"(v[39]),
          "r"(v[40]), "r"(v[41]), "r"(v[42]), "r"(v[43]), "r"(v[44]), "r"(v[45]), "r"(v[46]), "r"(v[47]),
          "r"(v[48]), "r"(v[49]), "r"(v[50]), "r"(v[51]), "r"(v[52]), "r"(v[53]), "r"(v[54]), "r"(v[55]),
          "r"(v[56]), "r"(v[57]), "r"(v[58]), "r"(v[59]), "r"(v[60]), "r"(v[61]), "r"(v[62]), "r"(v[63])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                   "=r"(r[7]) : "r"(taddr) : "memory");
}
/* D[tmem] (+)= A[smem] * B[smem]^T on e2m1 operands with one ue4m3 scale per 16
 * values of K for each row of A and of B (scale factors in tensor memory). */
__device__ __forceinline__ void umma_mxf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t sfa, uint32_t sfb)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
/* Instruction descriptor of kind::mxf4nvf4: e2m1 x e2m1 (format code 1 for both
 * operands), both K-major, N / 8 at bit 17, ue4m3 scales (bit 23 clear),
 * M / 16 at bit 24 (M = 128), K = 64 per instruction (bit 31 clear). */
__host__ __device__ constexpr uint32_t umma_idesc_mxf4(uint32_t n)
{
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (8u << 24);
}

/* tensor memory map (512 columns): accumulators of the two 128-row halves at
 * 0 and nb; scale-factor slots from 384 on, 64 columns each */
#define MMB_MX_SF_COL   384u
#define MMB_MX_SF_SLOT  64u
#define MMB_MX_SFB_OFF  32u

/* Sum of the six plane columns of one activation row, smallest plane first. */
__device__ __forceinline__ float mx_row_sum(const uint32_t (&c)[24], int r)
{
    float v = __uint_as_float(c[6 * r]);
#pragma unroll
    for (int q = 1; q < MMB_MX_PLANES; q++) v += __uint_as_float(c[6 * r + q]);
    return v;
}

/* ---- activation slicing ------------------------------------------------------ */
__device__ __forceinline__ uint32_t quant_e2m1(float t)
{
    /* nearest e2m1 code of t (round to nearest even, saturating); the second
     * operand is zero, so whichever nibble holds t is found by folding */
    uint32_t u;
    asm("{\n\t.reg .b8 q;\n\tcvt.rn.satfinite.e2m1x2.f32 q, %1, %2;\n\tmov.b32 %0, {q, q, q, q};\n\t}"
        : "=r"(u) : "f"(t), "f"(0.0f));
    return (u | (u >> 4)) & 15u;
}

__device__ __forceinline__ float dequant_e2m1(uint32_t code)
{
    uint32_t h2;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t}" : "=r"(h2) : "r"(code));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

/* shift s_p of plane p: its digit v stands for v * 2^(s_p + 1) units */
__host__ __device__ constexpr int mx_shift(int plane)
{
    return plane == 0 ? 0 : 3 * plane - 1;       /* 0, 2, 5, 8, 11, 14 */
}

/* Thread = four consecutive activations (a quarter of a 16-wide block); one CTA of
 * 256 threads covers 1024 values of activation row m, starting at 1024 * cta_x. */
/* Largest magnitude (bf16 bits without the sign) of the 1024 values of row m that
 * start at 1024 * cta_x: the first pass of the two-pass slicing of a group. */
__device__ __forceinline__ void xamax_cta(const uint16_t *x, uint32_t *chunk_max, uint32_t M, uint32_t K,
                                          uint32_t m, uint32_t cta_x)
{
    __shared__ uint32_t s_cm[8];
    const uint32_t tid = threadIdx.x, quarter = cta_x * 256u + tid;
    uint32_t a = 0;
    if (quarter < K / 4u && m < M) {
        const uint2 v = __ldcg(reinterpret_cast<const uint2 *>(x + static_cast<size_t>(m) * K) + quarter);
        a = max(max(v.x & 0x7fffu, (v.x >> 16) & 0x7fffu), max(v.y & 0x7fffu, (v.y >> 16) & 0x7fffu));
    }
    a = __reduce_max_sync(0xffffffffu, a);
    if ((tid & 31u) == 0)
        s_cm[tid >> 5] = a;
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int i = 1; i < 8; i++) a = max(a, s_cm[i]);
        chunk_max[m * MMB_MX_MAX_CHUNKS + cta_x] = a;
    }
}

/* chunk_max: the row's chunk maxima from xamax_cta (NULL: this CTA scans the row itself). */
__device__ __forceinline__ void xslice_cta(const uint16_t *x, uint8_t *planes, uint8_t *sfb, float *row_scale,
                                           uint32_t M, uint32_t K, uint32_t m, uint32_t cta_x,
                                           const uint32_t *chunk_max = nullptr)
{
    __shared__ uint32_t s_max[8];
    const uint32_t tid = threadIdx.x;
    const uint32_t blocks = K / 16u;

    /* this thread's four values, fetched while the row is scanned */
    const uint32_t quarter = cta_x * 256u + tid;         /* index of the four values in the row */
    const uint32_t blk = quarter >> 2;
    uint32_t w0 = 0, w1 = 0;
    if (blk < blocks && m < M) {
        const uint2 v = __ldcg(reinterpret_cast<const uint2 *>(x + static_cast<size_t>(m) * K) + quarter);
        w0 = v.x; w1 = v.y;                  /* written by the kernel in front: not the read-only path */
    }
    /* largest magnitude of the row: every CTA of the row scans all of it, eight
     * 16-byte loads in flight per thread */
    uint32_t amax = 0;
    if (chunk_max) {
        if (m < M && tid < (K + 1023u) / 1024u)
            amax = __ldcg(chunk_max + m * MMB_MX_MAX_CHUNKS + tid);
    } else if (m < M) {
        const uint4 *row = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(m) * K);
        const uint32_t n8 = K / 8u;
        for (uint32_t base8 = 0; base8 < n8; base8 += 2048u) {
            uint4 v[8];
#pragma unroll
            for (uint32_t j = 0; j < 8u; j++) {
                const uint32_t i = base8 + j * 256u + tid;
                v[j] = i < n8 ? __ldcg(row + i) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (uint32_t j = 0; j < 8u; j++) {
                const uint32_t w[4] = { v[j].x, v[j].y, v[j].z, v[j].w };
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    amax = max(amax, w[q] & 0x7fffu);
                    amax = max(amax, (w[q] >> 16) & 0x7fffu);
                }
            }
        }
    }
    amax = __reduce_max_sync(0xffffffffu, amax);
    if ((tid & 31u) == 0)
        s_max[tid >> 5] = amax;
    __syncthreads();
    amax = s_max[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = max(amax, s_max[i]);

    /* G = 9 - floor(log2(row maximum)): the largest block's top digit plane gets
     * the largest power of two a ue4m3 holds */
    const bool finite = amax < 0x7f80u;
    int e_max = static_cast<int>(amax >> 7) - 127;           /* exponent field 0: subnormal, below 2^-126 */
    if ((amax >> 7) == 0)
        e_max = amax ? (31 - __clz(amax)) - 133 : -126;       /* top bit of the 7-bit fraction x 2^-133 */
    const int G = 9 - e_max;
    if (cta_x == 0 && tid == 0) {
        const int g1 = G >> 1, g2 = G - g1;
        float f1 = __int_as_float((127 - g1) << 23), f2 = __int_as_float((127 - g2) << 23);
        if (!finite)
            f1 = __int_as_float(0x7fc00000);                  /* a row with inf or NaN gives NaN outputs */
        row_scale[2u * m] = f1;
        row_scale[2u * m + 1u] = f2;
    }

    const bool live = blk < blocks && m < M && finite && amax;
    if (!live)
        w0 = w1 = 0u;
    /* largest magnitude of the 16-wide block: the four threads of a block are neighbours */
    uint32_t bmax = max(max(w0 & 0x7fffu, (w0 >> 16) & 0x7fffu), max(w1 & 0x7fffu, (w1 >> 16) & 0x7fffu));
    bmax = max(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
    bmax = max(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
    if (blk >= blocks)
        return;
    int e_b = static_cast<int>(bmax >> 7) - 127;
    if ((bmax >> 7) == 0)
        e_b = bmax ? (31 - __clz(bmax)) - 133 : -200;
    const int U = max(e_b - 16, -10 - G);                      /* the block's unit is 2^U */
    uint32_t codes[MMB_MX_PLANES];
#pragma unroll
    for (int q = 0; q < MMB_MX_PLANES; q++) codes[q] = 0u;
    if (live) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t bits = ((i < 2 ? w0 : w1) >> (16 * (i & 1))) & 0xffffu;
            const uint32_t ef = (bits >> 7) & 0xffu, mant = bits & 0x7fu;
            const uint32_t sig = ef ? 128u + mant : mant;
            const int e = ef ? static_cast<int>(ef) - 127 : -126;
            const int sh = e - 7 - U;                          /* value = sig * 2^sh units */
            uint32_t V;
            if (sh >= 0)
                V = sig << sh;                                  /* sh <= 9 by the choice of U */
            else
                V = sh < -10 ? 0u : (sig + (1u << (-sh - 1))) >> (-sh);
            float R = static_cast<float>(V);
            if (bits & 0x8000u)
                R = -R;
#pragma unroll
            for (int q = MMB_MX_PLANES - 1; q >= 0; q--) {
                const float wgt = __int_as_float((127 + mx_shift(q) + 1) << 23);
                const float inv = __int_as_float((127 - mx_shift(q) - 1) << 23);
                const uint32_t code = quant_e2m1(R * inv);
                R = fmaf(-dequant_e2m1(code), wgt, R);
                codes[q] |= code << (4 * i);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < MMB_MX_PLANES; q++) {
        const size_t n = static_cast<size_t>(m) * MMB_MX_PLANES + q;
        *reinterpret_cast<uint16_t *>(planes + n * (K / 2u) + quarter * 2u) = static_cast<uint16_t>(codes[q]);
        if ((tid & 3u) == 0) {
            /* block scale of the plane, stored with the row's 2^G: 2^(U + 1 + s + G) in [2^-9, 2^8] */
            const int sfe = U + 1 + mx_shift(q) + G;
            const uint32_t byte = live ? (sfe >= -6 ? static_cast<uint32_t>(sfe + 7) << 3 : 1u << (sfe + 9)) : 0u;
            sfb[n * blocks + blk] = static_cast<uint8_t>(byte);
        }
    }
}

/* ---- one thread per 16-wide block ----------------------------------------------
 * The slicing of xslice_cta with a whole block in one thread: no shuffles, two
 * 16-byte loads, one 8-byte store per plane.  Row exponent and liveness come from
 * the caller (row_amax: largest magnitude of the row as bf16 bits without sign). */
struct RowFrame {
    int  G;          /* 9 - floor(log2(row maximum)) */
    bool finite;     /* no inf or NaN in the row */
    bool any;        /* the row has a non-zero value */
};

__device__ __forceinline__ RowFrame row_frame(uint32_t row_amax)
{
    RowFrame f;
    f.finite = row_amax < 0x7f80u;
    f.any = row_amax != 0u;
    int e_max = static_cast<int>(row_amax >> 7) - 127;
    if ((row_amax >> 7) == 0)
        e_max = row_amax ? (31 - __clz(row_amax)) - 133 : -126;
    f.G = 9 - e_max;
    return f;
}

__device__ __forceinline__ void row_factors(const RowFrame &f, float *row_scale, uint32_t m)
{
    const int g1 = f.G >> 1, g2 = f.G - g1;
    float f1 = __int_as_float((127 - g1) << 23), f2 = __int_as_float((127 - g2) << 23);
    if (!f.finite)
        f1 = __int_as_float(0x7fc00000);                      /* a row with inf or NaN gives NaN outputs */
    row_scale[2u * m] = f1;
    row_scale[2u * m + 1u] = f2;
}

/* w[8]: the block's sixteen bf16 values, two per word; plane row n0 = 6 * m. */
__device__ __forceinline__ void xslice_block(const uint32_t (&w)[8], const RowFrame &f, bool live, uint8_t *planes,
                                             uint8_t *sfb, uint32_t K, uint32_t m, uint32_t blk)
{
    uint32_t bmax = 0;
#pragma unroll
    for (int i = 0; i < 8; i++)
        bmax = max(bmax, max(w[i] & 0x7fffu, (w[i] >> 16) & 0x7fffu));
    live = live && f.finite && f.any;
    int e_b = static_cast<int>(bmax >> 7) - 127;
    if ((bmax >> 7) == 0)
        e_b = bmax ? (31 - __clz(bmax)) - 133 : -200;
    const int U = max(e_b - 16, -10 - f.G);
    float R[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint32_t bits = live ? (w[i >> 1] >> (16 * (i & 1))) & 0xffffu : 0u;
        const uint32_t ef = (bits >> 7) & 0xffu, mant = bits & 0x7fu;
        const uint32_t sig = ef ? 128u + mant : mant;
        const int e = ef ? static_cast<int>(ef) - 127 : -126;
        const int sh = e - 7 - U;
        uint32_t V;
        if (sh >= 0)
            V = sig << sh;
        else
            V = sh < -10 ? 0u : (sig + (1u << (-sh - 1))) >> (-sh);
        const float r = static_cast<float>(V);
        R[i] = (bits & 0x8000u) ? -r : r;
    }
    const uint32_t blocks = K / 16u;
#pragma unroll
    for (int q = MMB_MX_PLANES - 1; q >= 0; q--) {
        const float wgt = __int_as_float((127 + mx_shift(q) + 1) << 23);
        const float inv = __int_as_float((127 - mx_shift(q) - 1) << 23);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            /* a byte of the plane: high nibble = odd column, low nibble = even column */
            uint32_t byte, h2;
            asm("{\n\t.reg .b8 q;\n\tcvt.rn.satfinite.e2m1x2.f32 q, %1, %2;\n\tmov.b32 %0, {q, q, q, q};\n\t}"
                : "=r"(byte) : "f"(R[2 * j + 1] * inv), "f"(R[2 * j] * inv));
            byte &= 0xffu;
            asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %1;\n\t"
                "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t}" : "=r"(h2) : "r"(byte));
            const __half2 d = *reinterpret_cast<const __half2 *>(&h2);
            R[2 * j] = fmaf(-__low2float(d), wgt, R[2 * j]);
            R[2 * j + 1] = fmaf(-__high2float(d), wgt, R[2 * j + 1]);
            if (j < 4) lo |= byte << (8 * j); else hi |= byte << (8 * (j - 4));
        }
        const size_t n = static_cast<size_t>(m) * MMB_MX_PLANES + q;
        *reinterpret_cast<uint2 *>(planes + n * (K / 2u) + static_cast<size_t>(blk) * 8u) = make_uint2(lo, hi);
        const int sfe = U + 1 + mx_shift(q) + f.G;
        const uint32_t byte = live ? (sfe >= -6 ? static_cast<uint32_t>(sfe + 7) << 3 : 1u << (sfe + 9)) : 0u;
        sfb[n * blocks + blk] = static_cast<uint8_t>(byte);
    }
}

} // namespace mmb
