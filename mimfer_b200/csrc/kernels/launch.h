/*
 * Launch interface between the C launcher (csrc/cuda/kx_gemm_f4.c) and the
 * kernels (the .cu files under csrc/kernels).  One POD argument block per op; the tile and
 * grid numbers come from the selector (csrc/plan/select.c) and the smem
 * footprints below are the single definition both sides use.
 */
#ifndef MMB_LAUNCH_H
#define MMB_LAUNCH_H

#include <stddef.h>
#include "mimfer_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- STREAM (decode) geometry ------------------------------------------- */
#define MMB_ST_ROWS        256    /* weight rows per CTA (16 warps x 16 rows)  */
#define MMB_ST_KSTEP       256u   /* weights along K per pipeline stage        */
#define MMB_ST_CONSUMERS   16     /* MMA warps                                  */
#ifndef MMB_ST_XFORM_WARPS
#define MMB_ST_XFORM_WARPS 4u     /* activation transform warps                 */
#endif
#define MMB_ST_THREADS     ((MMB_ST_CONSUMERS + 1u + MMB_ST_XFORM_WARPS) * 32u)
#define MMB_ST_PAYLOAD_B   (MMB_ST_ROWS * 128u)            /* SW128 box        */
#define MMB_ST_SCALE_B     (MMB_ST_ROWS * 16u)
#define MMB_ST_X_RAW_B(mt) ((mt) * 8u * MMB_ST_KSTEP * 2u)     /* bytes TMA delivers         */
#define MMB_ST_X_B(mt)     ((mt) * 5120u)                       /* slot: 8 rows x 576 B, padded */
#define MMB_ST_STAGE_B(mt) (MMB_ST_PAYLOAD_B + MMB_ST_SCALE_B + MMB_ST_X_B(mt))
#define MMB_ST_FIXED_B     (2048u /* scale LUT */ + 512u /* barriers, flags */ + 1024u /* align slack */)


/* ---- MX (decode on the block-scaled tensor path) ---------------------------- */
#define MMB_MX_PLANES       6      /* signed e2m1 digits per activation                      */
#define MMB_MX_THREADS      352u   /* TMA, MMA (half 0), 2 x 4 scale-factor warps (four also run the epilogue), MMA (half 1) */
#define MMB_MX_MAX_NB       192u   /* B rows: 6 x (M padded to a multiple of 4), M <= 32     */
/* one pipeline stage: payload (rows x 128 B, padded to 1024) | digit planes (nb x 128 B)
 * | block scales (rows x 16 B) | plane scales (nb x 16 B), padded so that every stage
 * and both swizzled tiles start on a 1024-byte boundary.  `rows` is any multiple of 4 up
 * to 256: the selector sizes the tiles so that the grid fills the SMs. */
/* An MMA half always reads 128 rows of 128 bytes, valid or not, so the payload area
 * spans every byte the halves can touch: one half for a plain tile of up to 128
 * rows, two otherwise (the second half of a gated pair starts at rows / 2). */
#define MMB_MX_PAY_B(rows, glu)  (((glu) || (rows) > 128u) ? 32768u : 16384u)
#define MMB_MX_SC_B(rows)   ((((rows) * 16u) + 127u) & ~127u)      /* TMA destinations are 128-byte aligned */
#define MMB_MX_STAGE_B(rows, nb, glu) ((MMB_MX_PAY_B(rows, glu) + (nb) * 144u + MMB_MX_SC_B(rows) + 1023u) & ~1023u)
#define MMB_MX_FIXED_B      (512u /* barriers, flags */ + 1024u /* align slack */)
/* activation scratch of one op, inside its workspace region after the arrival
 * counters: row factors (32 rows x 2 floats), chunk maxima, digit planes [nb][K/2],
 * plane scales [nb][K/16] */
#define MMB_MX_ROWSCALE_OFF 0u
#define MMB_MX_CHUNKMAX_OFF 1024u  /* [32 rows][64] largest magnitude of every 1024-value chunk (group slicing) */
#define MMB_MX_MAX_CHUNKS   64u
#define MMB_MX_PLANES_OFF   16384u
#define MMB_MX_PLANES_B(nb, K) ((((size_t)(nb) * ((K) / 2u)) + 1023u) & ~(size_t)1023u)
#define MMB_MX_XS_B(nb, K)  (MMB_MX_PLANES_OFF + MMB_MX_PLANES_B(nb, K) + ((((size_t)(nb) * ((K) / 16u)) + 1023u) & ~(size_t)1023u))

/* ---- MXG (a group of independent decode linears in one persistent launch) ------- */
#define MMB_MXG_THREADS     480u   /* TMA, 2 x MMA, 8 x scale copy, 4 x epilogue                       */
#define MMB_MXG_MAX_OPS     48u    /* the op list travels in the kernel's parameter space (32 KB)      */
#define MMB_MXG_ACC_STRIDE  192u   /* tensor-memory columns between the two accumulator buffers        */
#define MMB_MXG_FIXED_B     (512u + 1024u)

/* ---- UMMA (prefill) geometry ---------------------------------------------- */
#define MMB_UM_KBLOCK      64u    /* bf16 elements per smem row (128 B swizzle) */
#define MMB_UM_KGROUP      256u   /* weights covered by one scale box (16 B)    */
#define MMB_UM_DEQ_WARPS   8u
#define MMB_UM_THREADS     ((2u + MMB_UM_DEQ_WARPS) * 32u)
#define MMB_UM_PAY_SLOTS(bn) ((bn) >= 256u ? 2u : 4u)
#define MMB_UM_SC_SLOTS    2u
#define MMB_UM_A_B(bm)     ((bm) * MMB_UM_KBLOCK * 2u)
#define MMB_UM_B_B(bn)     ((bn) * MMB_UM_KBLOCK * 2u)
#define MMB_UM_PAY_B(bn)   ((bn) * 32u)
#define MMB_UM_SC_B(bn)    ((bn) * 16u)
#define MMB_UM_FIXED_B     (1024u /* scale LUT */ + 512u /* barriers, tmem slot */ + 1024u /* align slack */)
#define MMB_UM_SMEM_B(bm, bn, st)                                              \
    ((st) * (MMB_UM_A_B(bm) + MMB_UM_B_B(bn)) + MMB_UM_PAY_SLOTS(bn) * MMB_UM_PAY_B(bn) + \
     MMB_UM_SC_SLOTS * MMB_UM_SC_B(bn) + MMB_UM_FIXED_B)

#define MMB_SMEM_MAX       232448u   /* 227 KiB opt-in limit per CTA on sm_100 */

/* Workspace layout: [counters: MMB_WS_COUNTER_B bytes][fp32 partials]. */
#define MMB_WS_COUNTER_B   16384u
#define MMB_WS_MAX_TILES   (MMB_WS_COUNTER_B / 4u)

#define MMB_MAX_PEERS      8u

/* Flag block of the cross-rank barrier (mm_f4_tp_barrier): one arrival slot per
 * peer, then the owner's epoch counter; 64 bytes, zeroed before first use. */
#define MMB_TPB_EPOCH      MMB_MAX_PEERS
#define MMB_TPB_WORDS      16u

/* Programmatic dependent launch, per op.  C(k) = completion of kernel k of the
 * stream, T(k) = the moment all its CTAs have triggered their dependents.
 *   OFF           plain launch: starts after C(prev).
 *   TRIGGER_FIRST every CTA triggers in its prologue, then waits for C(prev)
 *                 before the first activation load.  Safe on its own; gives no
 *                 ordering guarantee to an INDEPENDENT successor.
 *   WAIT_FIRST    wait for C(prev), then trigger: T(k) >= C(k-1).
 *   INDEPENDENT   the op touches nothing that any kernel since (and including)
 *                 the last WAIT_FIRST/OFF kernel reads or writes, workspace
 *                 included: trigger at once, never wait before loading, wait for
 *                 C(prev) just before the CTA exits, so completions stay ordered
 *                 (C(k) >= C(k-1)) and a later waiting kernel still sees
 *                 everything before it.  Only the decode kernel has this form.
 * INDEPENDENT must only follow WAIT_FIRST, OFF or INDEPENDENT kernels. */
#define MMB_PDL_OFF           0
#define MMB_PDL_TRIGGER_FIRST 1
#define MMB_PDL_WAIT_FIRST    2
#define MMB_PDL_INDEPENDENT   3

/* Measurement modes of the streaming decode kernel (mmb_args.dbg, mm_f4_tune
 * key 4).  They split a launch time into its parts: the weight stream alone,
 * the arithmetic alone, the split-K exchange; results are not meaningful with
 * any of them set.  Only a build with -DMMB_MEASURE_MODES has them: in the
 * shipped library the bits read as zero and key 4 is an unknown key. */
#ifdef MMB_MEASURE_MODES
#define MMB_DBG_NO_MATH      1u   /* consumers release every stage untouched        */
#define MMB_DBG_NO_LOADS     2u   /* no TMA traffic and no waits: arithmetic on whatever shared memory holds */
#define MMB_DBG_NO_EXCHANGE  4u   /* split-K slices store their own sums, no partials, no ticket */
#else
#define MMB_DBG_NO_MATH      0u
#define MMB_DBG_NO_LOADS     0u
#define MMB_DBG_NO_EXCHANGE  0u
#endif

/* Device status word bits. */
#define MMB_DEV_TIMEOUT    1u
#define MMB_DEV_BADARG     2u

typedef struct mmb_args {
    const void *x;        /* bf16 [M][K]        */
    const void *payload;  /* u8   [N][K/2]      */
    const void *scale;    /* u8   [N][K/16]     */
    void       *y;        /* bf16 [M][N]        */
    /* Tensor-parallel output: when n_dst > 0 the result goes to y_dst[0..n_dst-1]
     * (this GPU's and its peers' copies of the full output) with row pitch ldy
     * elements and column offset col0, instead of to y. */
    void       *y_dst[MMB_MAX_PEERS];
    uint32_t    n_dst, ldy, col0;
    /* Prefill, tensor parallel: CTA i of the first `stagger_ctas` starts i / stagger_ctas
     * of stagger_ns late (0 = all together), see umma.cu. */
    uint32_t    stagger_ns, stagger_ctas;
    float       gs;
    uint32_t    M, K, N;
    /* Gated pair (glu != 0): `payload`/`scale` are the lower-addressed of the gate
     * and up projections, tm_payload/tm_scale are 3-D maps whose third
     * coordinate selects the projection (plane 0 = lower address), N counts the
     * output features (rows of each projection), and the kernel writes
     * y[m][j] = bf16(silu(bf16(gate)) * bf16(up)) with pitch N.  gate_plane says
     * which plane is the gate; gs scales the gate, gs_up the up projection. */
    int         glu, gate_plane;
    float       gs_up;
    void       *ws;       /* workspace base or NULL */
    /* MX: activation scratch of this op (inside its own workspace region, or the
     * region of the op in front when both read the same activations) and where the
     * split-K partials start inside `ws` */
    void       *mx_x_ws;
    size_t      mx_partial_off;
    mm_f4_plan  plan;
    int         pdl;      /* MMB_PDL_*: how the launch is ordered against its predecessor */
    uint32_t    dbg;      /* MMB_DBG_* (decode kernel), 0 in production */
    /* 128-byte TMA descriptors, filled by the launcher (opaque here) */
    unsigned char tm_payload[128] __attribute__((aligned(64)));
    unsigned char tm_scale[128] __attribute__((aligned(64)));
    unsigned char tm_x[128] __attribute__((aligned(64)));     /* MX: the digit planes */
    unsigned char tm_sfb[128] __attribute__((aligned(64)));   /* MX: the planes' block scales */
} mmb_args;

/* One op of a group launch, and the group (host side; mxg.cu turns it into the
 * kernel's parameter block). */
typedef struct mmb_gop {
    const void *x;            /* bf16 [M][K] */
    void       *y;            /* bf16 [M][N] */
    void       *x_ws;         /* activation scratch (row factors, digit planes, plane scales) */
    int         slice_here;   /* this op is the first of the group to read x: slice it        */
    void       *y_dst[MMB_MAX_PEERS]; /* tensor parallel: every rank's copy of the full output (n_dst > 0) */
    uint32_t    n_dst, ldy, col0;     /* ... its row pitch, and this op's first column in it */
    void       *partial;
    uint32_t    counters_idx;         /* first arrival counter of the op (mmb_group.counters) */
    float       gs, gs_up;
    int         glu, gate_plane;
    uint32_t    M, K, N;
    uint32_t    rows, nb, k_steps, split_k, tiles, unit0;
    unsigned char tm_payload[128] __attribute__((aligned(64)));
    unsigned char tm_scale[128] __attribute__((aligned(64)));
    unsigned char tm_planes[128] __attribute__((aligned(64)));
    unsigned char tm_sfb[128] __attribute__((aligned(64)));
} mmb_gop;

typedef struct mmb_group {
    uint32_t n_ops, n_units, stages, acc_bufs, stage_b, smem_bytes, grid;
    int      pdl;
    void    *counters;       /* arrival counters of the region */
    void    *sched;          /* two zeroed words in the workspace: units are handed out as CTAs ask (NULL: round-robin) */
    void    *l2_base;        /* persisting L2 access window over the scratch (planes, partials); NULL = none */
    size_t   l2_bytes;
    mmb_gop  op[MMB_MXG_MAX_OPS];
} mmb_group;

int mmb_launch_mxg(const mmb_group *g, void *stream, uint32_t *kernels_launched);

/* Each returns a cudaError_t value (0 = success) from the launch. `stream`
 * is a cudaStream_t. */
int mmb_launch_rowwarp(const mmb_args *a, void *stream);
int mmb_launch_stream(const mmb_args *a, void *stream);
int mmb_launch_umma(const mmb_args *a, void *stream);
int mmb_launch_xslice(const mmb_args *a, void *stream);     /* activations -> digit planes (a->mx_x_ws) */
int mmb_launch_mx(const mmb_args *a, void *stream);
/* Buffers one launch of the upload kernel takes (host_gather.cu). */
#define MMB_GATHER_MAX 32u
int mmb_launch_host_gather(const void *const *src_host, void *const *dst_dev, const size_t *bytes,
                           uint32_t n, void *stream);
int mmb_launch_host_scatter(const void *const *src_dev, void *const *dst_host, const size_t *bytes,
                            uint32_t n, void *stream);
int mmb_launch_tp_barrier(unsigned *const *flags, uint32_t n_ranks, uint32_t rank, void *stream);
int mmb_launch_silu_mul(const void *gate, const void *up, void *y, size_t n, void *stream);
int mmb_launch_add_rmsnorm(void *res, const void *delta, void *y, const void *gain, uint32_t M, uint32_t H,
                           float eps, int pdl, void *stream);
int mmb_launch_wait_selftest(unsigned *status, unsigned *done, void *stream);
int mmb_launch_decode_probe(uint32_t *out_mma, uint32_t *out_f32, uint32_t *out_f16, void *stream);
/* STREAM plan with the rows per CTA and the K split given (0 = the selector's
 * own choice for that number); experiments and the selector's tests. */
mm_status mmb_plan_stream_with(const mm_f4_shape *s, uint32_t rows, uint32_t split, mm_f4_plan *p);
/* mm_f4_select_glu with the block-scaled decode path allowed or not. */
mm_status mmb_select_glu(const mm_f4_shape *s, int allow_mx, mm_f4_plan *p);
mm_status mmb_plan_mx_group(const mm_f4_shape *s, int glu, uint32_t split_k, mm_f4_plan *p);
mm_status mmb_plan_mx_with(const mm_f4_shape *s, uint32_t rows, uint32_t split, mm_f4_plan *p);
/* One-time per-process setup (smem opt-in attributes). */
int mmb_kernels_init(void);
/* Address of the device status word. */
int mmb_status_word(unsigned **dev_ptr);

#ifdef __cplusplus
}
#endif
#endif
