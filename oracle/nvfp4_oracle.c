/*
 * CPU oracle for the NVFP4 linear op.  TEST INFRASTRUCTURE ONLY: it is the
 * checker for tests/, the smoke check and the benchmark's CPU-baseline leg;
 * nothing in the product library links or calls it.
 *
 * It restates, in plain C, the arithmetic of the mimfer CPU reference kernel:
 *
 *   orc_e2m1_decode      include/mimfer/tensor.h:90-95   (8-entry magnitude LUT, bit 3 = sign)
 *   orc_e4m3_decode      include/mimfer/tensor.h:98-118  (0x7f/0xff -> +0.0f, sign honoured,
 *                                                         exp 0 -> m/8 * 2^-6, else (1+m/8)*2^(e-7))
 *   orc_wget             include/mimfer/tensor.h:130-139 (low nibble = even column, one scale per
 *                                                         16 columns, row-major by output feature)
 *   orc_silu_mul         src/kernels/cpu/cx.c:155-167    (silu(gate) * up on bf16, fp32 maths)
 *   orc_bf16_from_f32    include/mimfer/tensor.h:146-152 (RNE by +0x7fff + lsb)
 *   orc_f32_from_bf16    include/mimfer/tensor.h:154-159
 *   orc_gemm_f4          src/kernels/cpu/cx.c:197-216    (fp32 accumulate, k ascending,
 *                                                         separate multiply and add, one bf16
 *                                                         round at the end; K % 16 != 0 -> error)
 *
 * One extension: a global scale `gs` multiplies the fp32 accumulator before
 * the single bf16 rounding.  With gs == 1.0f the result is the reference's,
 * bit for bit (x * 1.0f is exact).  The reference has no global scale, so that
 * one multiply is not pinned by reference code; everything else is pinned by
 * tests/test_oracle.py against the compiled reference (oracle/_ref) and
 * against fixtures generated from it (tests/golden).
 *
 * Build: gcc -std=c11 -O2 -fopenmp (no -march=native, no -ffast-math); -std=c11
 * keeps floating-point contraction off, so no FMA is formed, as in the
 * reference host build.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

float orc_e2m1_decode(unsigned nibble)
{
    static const float mag[8] = { 0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f };
    float v = mag[nibble & 7u];
    return (nibble & 8u) ? -v : v;
}

float orc_e4m3_decode(unsigned char b)
{
    if (b == 0x7f || b == 0xff)
        return 0.0f;
    int neg = b & 0x80, e = (b >> 3) & 15, m = b & 7;
    float v = (float)m / 8.0f;
    if (e == 0) {
        v *= 0.015625f;
    } else {
        v += 1.0f;
        float p = 1.0f;
        for (int i = e - 7; i > 0; i--) p *= 2.0f;
        for (int i = e - 7; i < 0; i++) p *= 0.5f;
        v *= p;
    }
    return neg ? -v : v;
}

uint16_t orc_bf16_from_f32(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float orc_f32_from_bf16(uint16_t b)
{
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

float orc_wget(const uint8_t *payload, const uint8_t *scale, uint32_t K,
               uint32_t row, uint32_t col)
{
    unsigned byte = payload[(size_t)row * (K / 2) + (col >> 1)];
    unsigned nib = (col & 1) ? (byte >> 4) : (byte & 15u);
    float sc = orc_e4m3_decode(scale[(size_t)row * (K / 16) + (col >> 4)]);
    return orc_e2m1_decode(nib) * sc;
}

/* table[s * 16 + n] = fp32 bits of e2m1(n) * e4m3(s) */
void orc_decode_table(uint32_t *table4096)
{
    for (unsigned s = 0; s < 256; s++)
        for (unsigned n = 0; n < 16; n++) {
            float v = orc_e2m1_decode(n) * orc_e4m3_decode((unsigned char)s);
            memcpy(&table4096[s * 16 + n], &v, 4);
        }
}

/* Dequantise one weight row into fp32 (each element exactly orc_wget). */
static void dequant_row(const uint8_t *payload, const uint8_t *scale, uint32_t K,
                        uint32_t row, float *w)
{
    const uint8_t *p = payload + (size_t)row * (K / 2);
    const uint8_t *s = scale + (size_t)row * (K / 16);
    for (uint32_t b = 0; b < K / 16; b++) {
        float sc = orc_e4m3_decode(s[b]);
        for (uint32_t j = 0; j < 8; j++) {
            unsigned byte = p[b * 8 + j];
            w[b * 16 + 2 * j] = orc_e2m1_decode(byte & 15u) * sc;
            w[b * 16 + 2 * j + 1] = orc_e2m1_decode(byte >> 4) * sc;
        }
    }
}

static float dot_row(const uint16_t *xr, const float *w, uint32_t K)
{
    float acc = 0.0f;
    for (uint32_t k = 0; k < K; k++) {
        float prod = orc_f32_from_bf16(xr[k]) * w[k];
        acc += prod;
    }
    return acc;
}

/*
 * Columns [n_begin, n_end) of y for activation rows listed in m_idx (NULL =
 * all rows 0..M-1, n_m = M).  y_out is [n_m][n_end - n_begin] bf16 and, when
 * acc_out != NULL, the un-scaled fp32 accumulators go there with the same
 * shape.  Parallel over weight rows; every element is computed by the same
 * scalar sequence whatever the thread count.  Returns 0, or 4 (the
 * reference's MM_ERR_SHAPE) when K % 16 != 0.
 */
int orc_gemm_f4_block(const uint16_t *x, const uint8_t *payload, const uint8_t *scale,
                      float gs, uint16_t *y_out, float *acc_out,
                      uint32_t M, uint32_t K, uint32_t N,
                      const uint32_t *m_idx, uint32_t n_m,
                      uint32_t n_begin, uint32_t n_end, int threads)
{
    if (K % 16 != 0)
        return 4;
    if (!m_idx) n_m = M;
    if (n_end > N) n_end = N;
    uint32_t width = n_end > n_begin ? n_end - n_begin : 0;
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
    {
        float *w = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (long r = (long)n_begin; r < (long)n_end; r++) {
            dequant_row(payload, scale, K, (uint32_t)r, w);
            for (uint32_t i = 0; i < n_m; i++) {
                uint32_t m = m_idx ? m_idx[i] : i;
                float acc = dot_row(x + (size_t)m * K, w, K);
                size_t o = (size_t)i * width + ((uint32_t)r - n_begin);
                if (acc_out) acc_out[o] = acc;
                float scaled = acc * gs;
                y_out[o] = orc_bf16_from_f32(scaled);
            }
        }
        free(w);
    }
    return 0;
}

/* y[i] = bf16(silu(gate[i]) * up[i]) on bf16 inputs: the reference's SILU_MUL
 * (src/kernels/cpu/cx.c:155-167): s = g / (1 + expf(-g)) in fp32, one multiply,
 * one rounding. */
void orc_silu_mul(const uint16_t *gate, const uint16_t *up, uint16_t *y, size_t n)
{
    for (size_t i = 0; i < n; i++) {
        float g = orc_f32_from_bf16(gate[i]);
        float s = g / (1.0f + expf(-g));
        float prod = s * orc_f32_from_bf16(up[i]);
        y[i] = orc_bf16_from_f32(prod);
    }
}

/* Residual add + RMSNorm, the reference's OP_ADD_RMSNORM
 * (src/kernels/cpu/cx.c:70-84 and 132-150): per row, res[i] = bf16(res[i] +
 * delta[i]) in place; ss = sum of squares of the rounded row, fp32, ascending;
 * inv = 1 / sqrtf(ss / H + eps); y[i] = bf16(res[i] * inv * gain[i]), multiplied
 * left to right. */
void orc_add_rmsnorm(uint16_t *res, const uint16_t *delta, uint16_t *y, const uint16_t *gain,
                     uint32_t M, uint32_t H, float eps)
{
    for (uint32_t m = 0; m < M; m++) {
        uint16_t *rr = res + (size_t)m * H;
        const uint16_t *dr = delta + (size_t)m * H;
        uint16_t *yr = y + (size_t)m * H;
        for (uint32_t i = 0; i < H; i++) {
            float s = orc_f32_from_bf16(rr[i]) + orc_f32_from_bf16(dr[i]);
            rr[i] = orc_bf16_from_f32(s);
        }
        float ss = 0.0f;
        for (uint32_t i = 0; i < H; i++) {
            float v = orc_f32_from_bf16(rr[i]);
            float sq = v * v;
            ss += sq;
        }
        float mean = ss / (float)H;
        float inv = 1.0f / sqrtf(mean + eps);
        for (uint32_t i = 0; i < H; i++) {
            float t = orc_f32_from_bf16(rr[i]) * inv;
            float o = t * orc_f32_from_bf16(gain[i]);
            yr[i] = orc_bf16_from_f32(o);
        }
    }
}

/* Whole op, reference operand order: y[M][N]. */
int orc_gemm_f4(const uint16_t *x, const uint8_t *payload, const uint8_t *scale,
                float gs, uint16_t *y, uint32_t M, uint32_t K, uint32_t N, int threads)
{
    return orc_gemm_f4_block(x, payload, scale, gs, y, NULL, M, K, N, NULL, M, 0, N, threads);
}
