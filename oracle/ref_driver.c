/*
 * Thin driver around the UNMODIFIED mimfer CPU reference kernel.  TEST
 * INFRASTRUCTURE ONLY.  It is compiled together with the reference's own
 * sources (src/kernels/cpu/cx.c, src/core/mimfer.c), taken in place from the
 * read-only reference tree, into oracle/_ref/libmimfer_ref.so; no reference
 * source is copied into this repository.
 *
 * ref_silu_mul     one call of the reference kx_op_silu_mul.
 * ref_gemm_f4      one call of the reference kx_op_gemm_f4
 *                  (src/kernels/cpu/cx.c:197-216), single thread, as shipped.
 * ref_gemm_f4_mt   the same function called once per thread on a contiguous
 *                  slice of output features (weight rows are contiguous in both
 *                  buffers, include/mimfer/tensor.h:17-19), results scattered
 *                  back into y[M][N].  Per-element arithmetic is untouched.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "mimfer_abi.h"

mm_status kx_op_gemm_f4(const mm_kcall *kc);   /* the reference's symbols */
mm_status kx_op_silu_mul(const mm_kcall *kc);

/* One call of the reference kx_op_silu_mul (src/kernels/cpu/cx.c:155-167) over n
 * bf16 elements. */
int ref_silu_mul(const uint16_t *gate, const uint16_t *up, uint16_t *y, uint32_t n)
{
    mm_op_desc op;
    mm_kcall kc;
    memset(&op, 0, sizeof op);
    op.op = OP_SILU_MUL;
    op.layer = -1;
    op.a = gate; op.b = up; op.c = y;
    op.n0 = 1; op.n1 = n;
    kc.op = &op; kc.e = NULL; kc.stream = NULL;
    return (int)kx_op_silu_mul(&kc);
}

int ref_gemm_f4(const uint16_t *x, const uint8_t *payload, const uint8_t *scale,
                uint16_t *y, uint32_t M, uint32_t K, uint32_t N)
{
    mm_op_desc op;
    mm_kcall kc;
    memset(&op, 0, sizeof op);
    op.op = OP_GEMM_F4;
    op.layer = -1;
    op.a = x; op.b = payload; op.c = y; op.d = scale;
    op.n0 = M; op.n1 = K; op.n2 = N;
    kc.op = &op; kc.e = NULL; kc.stream = NULL;
    return (int)kx_op_gemm_f4(&kc);
}

int ref_gemm_f4_mt(const uint16_t *x, const uint8_t *payload, const uint8_t *scale,
                   uint16_t *y, uint32_t M, uint32_t K, uint32_t N, int threads)
{
    int rc = 0;
    if (threads < 1) threads = 1;
    if (K % 16 != 0)
        return ref_gemm_f4(x, payload, scale, y, M, K, N);
#pragma omp parallel num_threads(threads)
    {
        int nt = 1, id = 0;
#ifdef _OPENMP
        extern int omp_get_num_threads(void);
        extern int omp_get_thread_num(void);
        nt = omp_get_num_threads();
        id = omp_get_thread_num();
#endif
        uint32_t n0 = (uint32_t)((uint64_t)N * id / nt);
        uint32_t n1 = (uint32_t)((uint64_t)N * (id + 1) / nt);
        uint32_t w = n1 - n0;
        if (w) {
            uint16_t *tmp = (uint16_t *)malloc((size_t)M * w * 2);
            int r = ref_gemm_f4(x, payload + (size_t)n0 * (K / 2),
                                scale + (size_t)n0 * (K / 16), tmp, M, K, w);
            if (r) {
#pragma omp critical
                rc = r;
            }
            for (uint32_t m = 0; m < M; m++)
                memcpy(y + (size_t)m * N + n0, tmp + (size_t)m * w, (size_t)w * 2);
            free(tmp);
        }
    }
    return rc;
}
