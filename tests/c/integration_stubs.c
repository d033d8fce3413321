/*
 * The launchers of the mimfer dispatcher (src/kernels/kx.c:15-47) that the NVFP4
 * linear library does not own, as a GPU build of mimfer without its cx.cu would
 * need them to link: each reports that it is not served.
 */
#include "mimfer/kernels.h"

#define NOT_SERVED(name) mm_status name(const mm_kcall *kc) { (void)kc; return MM_ERR_UNSUPPORTED; }
NOT_SERVED(kx_op_embed)
NOT_SERVED(kx_op_rmsnorm)
NOT_SERVED(kx_op_gemm_bf16)
NOT_SERVED(kx_op_rope)
NOT_SERVED(kx_op_kvstore)
NOT_SERVED(kx_op_att_decode)
NOT_SERVED(kx_op_att_prefill)
NOT_SERVED(kx_op_softmax_causal)
NOT_SERVED(kx_op_conv4)
NOT_SERVED(kx_op_lin_dec)
NOT_SERVED(kx_op_lin_pre)
NOT_SERVED(kx_op_copy)
NOT_SERVED(kx_op_sample)

/* src/kernels/kx.h:43, defined in mimfer's cx.cu: which ops the GPU build prefers */
int kx_cuda_oppref(int op)
{
    return op == OP_GEMM_F4 || op == OP_QKV || op == OP_LMHEAD || op == OP_SILU_MUL || op == OP_ADD_RMSNORM;
}
