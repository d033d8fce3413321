/*
 * Driver for the reference's residual add + RMSNorm op.  TEST INFRASTRUCTURE
 * ONLY, compiled with the reference's own headers and sources in place (see
 * oracle/build.py); nothing of the reference is copied here.
 *
 * ref_add_rmsnorm   one call of the reference kx_op_add_rmsnorm
 *                   (src/kernels/cpu/cx.c:132-150): res += delta in place, then
 *                   y = rmsnorm(res) * gain.  The op reads its epsilon from the
 *                   engine's model configuration (kc->e->mc.norm_eps), so the
 *                   driver passes a zeroed engine with that one field set.
 */
#define _POSIX_C_SOURCE 200809L      /* the reference headers use clock_gettime */
#include <stdint.h>
#include <string.h>
#include "mimfer/engine.h"
#include "mimfer/kernels.h"

int ref_add_rmsnorm(uint16_t *res, const uint16_t *delta, uint16_t *y, const uint16_t *gain,
                    uint32_t M, uint32_t H, float eps)
{
    static mm_engine e;
    mm_op_desc op;
    mm_kcall kc;
    memset(&e, 0, sizeof e);
    memset(&op, 0, sizeof op);
    e.mc.norm_eps = eps;
    op.op = OP_ADD_RMSNORM;
    op.layer = -1;
    op.a = res; op.b = delta; op.c = y; op.d = gain;
    op.n0 = M; op.n1 = H;
    kc.op = &op; kc.e = &e; kc.stream = NULL;
    return (int)kx_op_add_rmsnorm(&kc);
}
