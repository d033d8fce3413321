/*
 * mimfer operator ABI, as seen by the NVFP4 linear launcher.
 *
 * The B200 library is a drop-in for one launcher of the mimfer appliance:
 * kx_op_gemm_f4 (reference: src/kernels/cuda/cx.cu:358-376, CPU twin
 * src/kernels/cpu/cx.c:197-216).  That launcher is called with a
 * `const mm_kcall *` whose `op` member points at an `mm_op_desc`.  This header
 * restates exactly the types that cross that call, with the same member order,
 * widths and enumerator values as the reference headers, so an object file
 * built here links against an unmodified mimfer tree:
 *
 *   mm_status     include/mimfer/mimfer.h:50-66
 *   mm_op         include/mimfer/plan.h:46-69
 *   mm_op_desc    include/mimfer/plan.h:73-82
 *   mm_kcall      include/mimfer/kernels.h:73-80
 *   mm_wt         include/mimfer/tensor.h:121-126
 *   mm_dtype      include/mimfer/tensor.h:33-42
 *   mm_stream_id  include/mimfer/cuda_rt.h:32-36
 *
 * tests/test_abi.py compiles this header next to the reference's own
 * headers (when the reference tree is mounted) and compares every sizeof and
 * offsetof; the _Static_asserts below pin the same numbers for builds without
 * the mount.
 */
#ifndef MIMFER_ABI_H
#define MIMFER_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (values are part of the ABI) ------------------------- */
typedef enum mm_status {
    MM_OK = 0,
    MM_ERR_NOMEM = 1,
    MM_ERR_IO = 2,
    MM_ERR_CORRUPT = 3,
    MM_ERR_SHAPE = 4,        /* K not a multiple of 16, zero extents        */
    MM_ERR_CUDA = 5,         /* launch or synchronise failed                */
    MM_ERR_DEVICE = 6,       /* not an sm_100 device                        */
    MM_ERR_UNSUPPORTED = 7,
    MM_ERR_RANGE = 8,
    MM_ERR_STATE = 9,        /* NULL operand, runtime not initialised       */
    MM_ERR_BUSY = 10,
    MM_ERR_TIMEOUT = 11,     /* a bounded device-side wait ran out          */
    MM_ERR_CAPACITY = 12,
    MM_ERR_EOF = 13,
    MM_ERR_LAST = 14
} mm_status;

const char *mm_status_str(mm_status s);

/* ---- opcodes ------------------------------------------------------------ */
typedef enum mm_op {
    OP_EMBED = 0,
    OP_LMHEAD = 1,
    OP_RMSNORM = 2,
    OP_ADD_RMSNORM = 3,
    OP_GEMM_F4 = 4,          /* y = x @ W^T, W in NVFP4 -- the op built here */
    OP_GEMM_BF16 = 5,
    OP_QKV = 6,
    OP_ROPE = 7,
    OP_KVSTORE = 8,
    OP_ATT_DECODE = 9,
    OP_ATT_PREFILL = 10,
    OP_SOFTMAX_CAUSAL = 11,
    OP_SILU_MUL = 12,
    OP_CONV4 = 13,
    OP_LIN_DEC = 14,
    OP_LIN_PRE = 15,
    OP_COPY = 16,
    OP_SAMPLE = 17,
    OP_NOP = 18,
    OP_N = 19
} mm_op;

/* ---- the op descriptor --------------------------------------------------
 * For OP_GEMM_F4 (operand table: include/mimfer/kernels.h:89-92):
 *   a  = x, bf16, [n0][n1] row-major                (M x K)
 *   b  = W payload, e2m1 nibbles, [n2][n1/2] bytes, low nibble = even column
 *   d  = W block scales, e4m3, [n2][n1/16] bytes, one per 16 columns
 *   c  = y, bf16, [n0][n2] row-major                (M x N)
 *   n0 = M, n1 = K (multiple of 16), n2 = N
 */
typedef struct mm_op_desc {
    int         op;
    int         layer;
    const void *a;
    const void *b;
    void       *c;
    const void *d;
    uint32_t    n0, n1, n2;
    char        note[24];
} mm_op_desc;

struct mm_engine;                       /* opaque to every launcher here   */
typedef struct mm_engine mm_engine;
typedef void *mm_stream_h;

typedef struct mm_kcall {
    const mm_op_desc *op;
    const mm_engine  *e;                /* never dereferenced by GEMM_F4    */
    mm_stream_h       stream;           /* passed as 0 and ignored, as in
                                           src/plan/plan.c:121              */
} mm_kcall;

typedef enum mm_dtype {
    MM_DT_U8 = 0,
    MM_DT_I32 = 1,
    MM_DT_I64 = 2,
    MM_DT_F32 = 3,
    MM_DT_BF16 = 4,
    MM_DT_FP4E2M1 = 5,
    MM_DT_FP8E4M3 = 6,
    MM_DT_N = 7
} mm_dtype;

/* NVFP4 weight view (rows = output features, cols = input features). */
typedef struct mm_wt {
    const void *data;
    const void *scale;
    uint32_t    rows;
    uint32_t    cols;
} mm_wt;

typedef enum mm_stream_id {
    MM_ST_COMPUTE = 0,
    MM_ST_XFER = 1,
    MM_ST_N = 2
} mm_stream_id;

#ifndef __cplusplus
_Static_assert(sizeof(mm_op_desc) == 80, "mm_op_desc layout");
_Static_assert(offsetof(mm_op_desc, a) == 8, "mm_op_desc.a");
_Static_assert(offsetof(mm_op_desc, d) == 32, "mm_op_desc.d");
_Static_assert(offsetof(mm_op_desc, n0) == 40, "mm_op_desc.n0");
_Static_assert(offsetof(mm_op_desc, note) == 52, "mm_op_desc.note");
_Static_assert(sizeof(mm_kcall) == 24, "mm_kcall layout");
_Static_assert(sizeof(mm_wt) == 24, "mm_wt layout");
#endif

#ifdef __cplusplus
}
#endif
#endif /* MIMFER_ABI_H */
