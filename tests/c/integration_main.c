/*
 * One OP_GEMM_F4 through mimfer's OWN dispatcher and CUDA runtime shim into this
 * library's launcher: the program is written against the reference headers and
 * linked from the reference's src/kernels/kx.c, src/cuda/cuda_rt.c and
 * src/core/mimfer.c (compiled where they lie, -DMM_WITH_CUDA) plus this
 * library's objects without csrc/cuda/rt.c and csrc/core/core.c
 * (oracle/build.py: build_integration).
 *
 * usage: integration_main M K N gs x.bin payload.bin scales.bin y.bin
 *   x bf16 [M][K], payload u8 [N][K/2], scales u8 [N][K/16] -> y bf16 [M][N]
 */
#define MM_WITH_CUDA 1
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <cuda_runtime_api.h>
#include "mimfer/mimfer.h"
#include "mimfer/plan.h"
#include "mimfer/kernels.h"
#include "mimfer/cuda_rt.h"

/* the library's additions to the reference surface */
mm_status mm_f4_gscale_set(const void *scale_base, float gs);
mm_status mm_f4_workspace_set(void *dev_ptr, size_t bytes);
mm_status mm_f4_device_status(unsigned *flags_out);

static void *slurp(const char *path, size_t n)
{
    FILE *f = fopen(path, "rb");
    void *p = malloc(n ? n : 1);
    if (!f || !p || fread(p, 1, n, f) != n) { fprintf(stderr, "cannot read %zu bytes of %s\n", n, path); exit(4); }
    fclose(f);
    return p;
}

#define CU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
    fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_)); return 2; } } while (0)
#define MM(call) do { mm_status s_ = (call); if (s_ != MM_OK) { \
    fprintf(stderr, "%s: %s\n", #call, mm_status_str(s_)); return 3; } } while (0)

int main(int argc, char **argv)
{
    if (argc != 9) { fprintf(stderr, "usage: %s M K N gs x payload scales y\n", argv[0]); return 1; }
    const uint32_t M = (uint32_t)atoi(argv[1]), K = (uint32_t)atoi(argv[2]), N = (uint32_t)atoi(argv[3]);
    const float gs = (float)atof(argv[4]);
    const size_t xb = (size_t)M * K * 2, pb = (size_t)N * K / 2, sb = (size_t)N * K / 16, yb = (size_t)M * N * 2;
    void *x = slurp(argv[5], xb), *payload = slurp(argv[6], pb), *scales = slurp(argv[7], sb), *y = malloc(yb);
    void *dx, *dp, *ds, *dy, *ws;
    const size_t ws_bytes = (size_t)64 << 20;

    MM(mm_cuda_init(0));                                   /* mimfer's shim owns the streams */
    CU(cudaMalloc(&dx, xb)); CU(cudaMalloc(&dp, pb)); CU(cudaMalloc(&ds, sb)); CU(cudaMalloc(&dy, yb));
    CU(cudaMalloc(&ws, ws_bytes));
    CU(cudaMemcpy(dx, x, xb, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(dp, payload, pb, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(ds, scales, sb, cudaMemcpyHostToDevice));
    CU(cudaMemset(dy, 0, yb));
    MM(mm_f4_workspace_set(ws, ws_bytes));
    MM(mm_f4_gscale_set(ds, gs));

    mm_op_desc op;
    memset(&op, 0, sizeof op);
    op.op = OP_GEMM_F4;
    op.a = dx; op.b = dp; op.d = ds; op.c = dy;
    op.n0 = M; op.n1 = K; op.n2 = N;
    mm_kcall kc;
    memset(&kc, 0, sizeof kc);
    kc.op = &op;
    kc.e = (const mm_engine *)&kc;                         /* the dispatcher only tests it for NULL */
    MM(mm_kx_invoke(&kc));                                 /* src/kernels/kx.c -> kx_op_gemm_f4 of this library */

    op.op = OP_ROPE;                                       /* an op the library does not own stays unserved */
    if (mm_kx_invoke(&kc) != MM_ERR_UNSUPPORTED) { fprintf(stderr, "OP_ROPE was not refused\n"); return 5; }

    MM(mm_stream_sync(MM_ST_COMPUTE));
    unsigned flags = 1;
    MM(mm_f4_device_status(&flags));
    if (flags) { fprintf(stderr, "device status 0x%x\n", flags); return 6; }
    CU(cudaMemcpy(y, dy, yb, cudaMemcpyDeviceToHost));
    FILE *f = fopen(argv[8], "wb");
    if (!f || fwrite(y, 1, yb, f) != yb) { fprintf(stderr, "cannot write %s\n", argv[8]); return 4; }
    fclose(f);
    printf("integration_main: OP_GEMM_F4 M=%u K=%u N=%u through mm_kx_invoke: ok\n", M, K, N);
    return 0;
}
