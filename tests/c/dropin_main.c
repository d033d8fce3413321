/*
 * C host program that drives the NVFP4 linear op the way mimfer's own C code
 * does: an mm_op_desc dispatched through mm_kx_invoke (reference call stack:
 * src/plan/plan.c:119-130 -> src/kernels/kx.c:15-47 -> kx_op_gemm_f4).
 *
 * Built two ways by tests/test_dropin_c.py:
 *   -DUSE_REFERENCE_HEADERS  against the reference's own headers (compile + link
 *                            only: proves the library satisfies the symbols and
 *                            types an unmodified mimfer translation unit uses)
 *   default                  against include/mimfer_b200.h, run on a GPU; prints
 *                            the FNV-1a checksum of y for comparison with the
 *                            Python path.
 * usage: dropin_main M K N
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <cuda_runtime_api.h>

#ifdef USE_REFERENCE_HEADERS
#define MM_WITH_CUDA 1
#include "mimfer/mimfer.h"
#include "mimfer/plan.h"
#include "mimfer/kernels.h"
#include "mimfer/cuda_rt.h"
/* new surface of the B200 library, not in the reference headers */
mm_status mm_f4_make_weight(uint32_t N, uint32_t K, uint64_t seed, float std, uint8_t *payload,
                            uint8_t *scales, float *gs_out);
void mm_fill_normal_f32(float *out, uint64_t rows, uint64_t cols, uint64_t seed, float mean, float std);
void mm_f32_to_bf16(const float *in, uint16_t *out, uint64_t n);
mm_status mm_f4_gscale_set(const void *scale_base, float gs);
mm_status mm_f4_workspace_set(void *dev_ptr, size_t bytes);
#else
#include "mimfer_b200.h"
#endif

static uint64_t fnv1a64(const void *data, size_t n)
{
    const unsigned char *p = (const unsigned char *)data;
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < n; i++) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}

#define CU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
    fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_)); return 2; } } while (0)
#define MM(call) do { mm_status s_ = (call); if (s_ != MM_OK) { \
    fprintf(stderr, "%s: status %d\n", #call, (int)s_); return 3; } } while (0)

int main(int argc, char **argv)
{
    if (argc != 4) { fprintf(stderr, "usage: %s M K N\n", argv[0]); return 1; }
    uint32_t M = (uint32_t)atoi(argv[1]), K = (uint32_t)atoi(argv[2]), N = (uint32_t)atoi(argv[3]);
    size_t pb = (size_t)N * K / 2, sb = (size_t)N * K / 16, xb = (size_t)M * K * 2, yb = (size_t)M * N * 2;

    uint8_t *payload = malloc(pb), *scales = malloc(sb);
    float *xf = malloc((size_t)M * K * 4), gs = 0.0f;
    uint16_t *x = malloc(xb), *y = malloc(yb);
    if (!payload || !scales || !xf || !x || !y) return 1;
    MM(mm_f4_make_weight(N, K, 0, 0.02f, payload, scales, &gs));
    mm_fill_normal_f32(xf, M, K, 1, 0.0f, 1.0f);
    mm_f32_to_bf16(xf, x, (uint64_t)M * K);

    MM(mm_cuda_init(0));
    void *d_payload, *d_scales, *d_x, *d_y, *d_ws;
    const size_t ws_bytes = 32u << 20;
    CU(cudaMalloc(&d_payload, pb)); CU(cudaMalloc(&d_scales, sb)); CU(cudaMalloc(&d_x, xb));
    CU(cudaMalloc(&d_y, yb)); CU(cudaMalloc(&d_ws, ws_bytes));
    CU(cudaMemcpy(d_payload, payload, pb, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(d_scales, scales, sb, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(d_x, x, xb, cudaMemcpyHostToDevice));
    CU(cudaMemset(d_y, 0, yb));
    MM(mm_f4_workspace_set(d_ws, ws_bytes));
    MM(mm_f4_gscale_set(d_scales, gs));

    mm_op_desc op;
    memset(&op, 0, sizeof op);
    op.op = OP_GEMM_F4; op.layer = 0;
    op.a = d_x; op.b = d_payload; op.c = d_y; op.d = d_scales;
    op.n0 = M; op.n1 = K; op.n2 = N;
    strcpy(op.note, "dropin");
    mm_kcall kc;
    kc.op = &op; kc.e = (const mm_engine *)&op;   /* any non-NULL engine: never dereferenced */
    kc.stream = 0;
    MM(mm_kx_invoke(&kc));                       /* synchronises, like the reference launcher */

    CU(cudaMemcpy(y, d_y, yb, cudaMemcpyDeviceToHost));
    printf("%016llx\n", (unsigned long long)fnv1a64(y, yb));
    MM(mm_cuda_shutdown());
    return 0;
}
