/*
 * NVFP4 quantising packer and the seeded input generator (host C).
 *
 * The mimfer tree has a container writer but no quantiser; its weight view is
 * payload + block scales only (include/mimfer/tensor.h:121-126).  This file
 * produces exactly that layout (tensor.h:17-19: payload [N][K/2], low nibble =
 * even column; scales [N][K/16] e4m3) from fp32 weights, plus the per-tensor
 * fp32 global scale that NVFP4 checkpoints carry:
 *
 *   gs            = max|W| / (6 * 448)             (1.0f for an all-zero tensor)
 *   scale(block)  = e4m3_rne_sat(amax_block / (6 * gs))
 *   nibble(w)     = e2m1_rne_sat(w / (e4m3_value(scale) * gs))
 *
 * so that W ~= gs * e4m3_value(scale) * e2m1_value(nibble).  Encoders round to
 * nearest, ties to the code with an even mantissa bit, and saturate (448, 6).
 *
 * The generator is splitmix64 (include/mimfer/mimfer.h:149-155, the tree's
 * only RNG) feeding Box-Muller in double; every row restarts the stream from
 * (seed, row) so rows can be produced in any order or in parallel.
 */
#include "../core/core.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---- format values (encoder side; the decoders live with their users) --- */

static float e4m3_value(unsigned code)   /* code 0..0x7e, positive */
{
    unsigned e = (code >> 3) & 15u, m = code & 7u;
    return e ? ldexpf(1.0f + (float)m / 8.0f, (int)e - 7) : ldexpf((float)m / 8.0f, -6);
}

static uint8_t e4m3_encode_pos(float f)
{
    if (!(f > 0.0f))
        return 0;
    if (f >= 448.0f)
        return 0x7e;
    unsigned lo = 0, hi = 0x7e;                 /* value(lo) <= f < value(hi) */
    while (hi - lo > 1) {
        unsigned mid = (lo + hi) / 2;
        if (e4m3_value(mid) <= f) lo = mid; else hi = mid;
    }
    float dl = f - e4m3_value(lo), dh = e4m3_value(hi) - f;
    if (dl < dh) return (uint8_t)lo;
    if (dh < dl) return (uint8_t)hi;
    return (uint8_t)((lo & 1u) ? hi : lo);      /* tie: even mantissa bit */
}

static unsigned e2m1_encode(float v)
{
    unsigned sign = signbit(v) ? 8u : 0u;
    float a = fabsf(v);
    unsigned code;
    if (!(a == a))       code = 0;              /* NaN never occurs; map to 0 */
    else if (a <= 0.25f) code = 0;
    else if (a < 0.75f)  code = 1;
    else if (a <= 1.25f) code = 2;
    else if (a < 1.75f)  code = 3;
    else if (a <= 2.5f)  code = 4;
    else if (a < 3.5f)   code = 5;
    else if (a <= 5.0f)  code = 6;
    else                 code = 7;
    return sign | code;
}

static void pack_row(const float *w, uint32_t K, float gs, uint8_t *p, uint8_t *s)
{
    for (uint32_t b = 0; b < K / 16; b++) {
        const float *wb = w + (size_t)b * 16;
        float amax = 0.0f;
        for (int j = 0; j < 16; j++) {
            float a = fabsf(wb[j]);
            if (a > amax) amax = a;
        }
        uint8_t code = e4m3_encode_pos(amax / (6.0f * gs));
        float denom = e4m3_value(code) * gs;
        s[b] = code;
        for (int j = 0; j < 8; j++) {
            unsigned lo = 0, hi = 0;
            if (denom > 0.0f) {
                lo = e2m1_encode(wb[2 * j] / denom);
                hi = e2m1_encode(wb[2 * j + 1] / denom);
            }
            p[b * 8 + j] = (uint8_t)(lo | (hi << 4));
        }
    }
}

mm_status mm_f4_pack(const float *W, uint32_t N, uint32_t K,
                     uint8_t *payload, uint8_t *scales, float *gs_out)
{
    MM_REQUIRE(W && payload && scales && gs_out, MM_ERR_STATE);
    MM_REQUIRE(N > 0 && K > 0 && K % 16 == 0, MM_ERR_SHAPE);
    float wmax = 0.0f;
#pragma omp parallel for reduction(max : wmax) schedule(static)
    for (long r = 0; r < (long)N; r++)
        for (uint32_t k = 0; k < K; k++) {
            float a = fabsf(W[(size_t)r * K + k]);
            if (a > wmax) wmax = a;
        }
    float gs = wmax > 0.0f ? wmax / (6.0f * 448.0f) : 1.0f;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)N; r++)
        pack_row(W + (size_t)r * K, K, gs, payload + (size_t)r * (K / 2),
                 scales + (size_t)r * (K / 16));
    *gs_out = gs;
    return MM_OK;
}

/* ---- seeded generator ---------------------------------------------------- */

static inline uint64_t splitmix64(uint64_t *st)
{
    uint64_t z = (*st += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

static void normal_row(float *out, uint64_t cols, uint64_t seed, uint64_t row,
                       float mean, float std)
{
    uint64_t st = seed * 0xd1342543de82ef95ull + row * 0x2545f4914f6cdd1dull + 1u;
    (void)splitmix64(&st);
    for (uint64_t i = 0; i < cols; i += 2) {
        double u1 = (double)((splitmix64(&st) >> 11) + 1u) * (1.0 / 9007199254740992.0);
        double u2 = (double)(splitmix64(&st) >> 11) * (1.0 / 9007199254740992.0);
        double r = sqrt(-2.0 * log(u1));
        double a = 6.283185307179586476925 * u2;
        out[i] = (float)((double)mean + (double)std * (r * cos(a)));
        if (i + 1 < cols)
            out[i + 1] = (float)((double)mean + (double)std * (r * sin(a)));
    }
}

void mm_fill_normal_f32(float *out, uint64_t rows, uint64_t cols, uint64_t seed,
                        float mean, float std)
{
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; r++)
        normal_row(out + (size_t)r * cols, cols, seed, (uint64_t)r, mean, std);
}

void mm_f32_to_bf16(const float *in, uint16_t *out, uint64_t n)
{
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; i++) {
        uint32_t u;
        memcpy(&u, &in[i], 4);
        u += 0x7fffu + ((u >> 16) & 1u);        /* round to nearest even */
        out[i] = (uint16_t)(u >> 16);
    }
}

void mm_bf16_to_f32(const uint16_t *in, float *out, uint64_t n)
{
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; i++) {
        uint32_t u = (uint32_t)in[i] << 16;
        memcpy(&out[i], &u, 4);
    }
}

mm_status mm_f4_make_weight(uint32_t N, uint32_t K, uint64_t seed, float std,
                            uint8_t *payload, uint8_t *scales, float *gs_out)
{
    MM_REQUIRE(payload && scales && gs_out, MM_ERR_STATE);
    MM_REQUIRE(N > 0 && K > 0 && K % 16 == 0, MM_ERR_SHAPE);
    float wmax = 0.0f;
    int failed = 0;
#pragma omp parallel reduction(max : wmax)
    {
        float *row = (float *)malloc((size_t)K * sizeof(float));
        if (!row) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(static)
        for (long r = 0; r < (long)N; r++) {
            if (!row) continue;
            normal_row(row, K, seed, (uint64_t)r, 0.0f, std);
            for (uint32_t k = 0; k < K; k++) {
                float a = fabsf(row[k]);
                if (a > wmax) wmax = a;
            }
        }
        free(row);
    }
    if (failed)
        return MM_ERR_NOMEM;
    float gs = wmax > 0.0f ? wmax / (6.0f * 448.0f) : 1.0f;
#pragma omp parallel
    {
        float *row = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (long r = 0; r < (long)N; r++) {
            if (!row) continue;
            normal_row(row, K, seed, (uint64_t)r, 0.0f, std);
            pack_row(row, K, gs, payload + (size_t)r * (K / 2), scales + (size_t)r * (K / 16));
        }
        if (!row) {
#pragma omp atomic write
            failed = 1;
        }
        free(row);
    }
    *gs_out = gs;
    return failed ? MM_ERR_NOMEM : MM_OK;
}
