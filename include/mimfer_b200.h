/*
 * C-ABI of the B200 NVFP4 linear library (libmimfer_b200.so).
 *
 * Everything here has C linkage and takes plain pointers and sizes.  The
 * first group keeps the names, argument meaning and error behaviour of the
 * mimfer appliance so the library drops in behind its dispatcher; each
 * declaration cites the reference interface it replaces (paths are relative
 * to the mimfer source tree).  The second group is new surface the reference
 * has no counterpart for (global scale, split-K workspace, tile selection,
 * the quantising packer, the op-list engine); it is named mm_f4_* / mm_lin_*.
 *
 * Threading: one host thread per process drives one device, exactly like the
 * reference runtime (src/cuda/cuda_rt.c:15-18 keeps process-global statics).
 */
#ifndef MIMFER_B200_H
#define MIMFER_B200_H

#include "mimfer_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ======================================================================
 * 1. Reference-named surface
 * ====================================================================== */

/* Replaces kx_op_gemm_f4 in src/kernels/cuda/cx.cu:358-376 (CPU twin
 * src/kernels/cpu/cx.c:197-216).  y = bf16(gs * sum_k x[m][k] * W[r][k]),
 * fp32 accumulation; gs is the weight's global scale (1.0f unless registered
 * with mm_f4_gscale_set).  Launches on the compute stream of the runtime
 * below.  Outside graph capture it synchronises that stream and reports
 * launch / device errors (reference: kx_sync, cx.cu:83-100); while capturing
 * it only enqueues.  Returns MM_ERR_SHAPE when n1 % 16 != 0 or an extent is
 * zero, MM_ERR_STATE on NULL operands or an uninitialised runtime,
 * MM_ERR_CUDA on launch/sync failure, MM_ERR_TIMEOUT when a bounded
 * device-side wait gave up.  Allocates nothing. */
mm_status kx_op_gemm_f4(const mm_kcall *kc);

/* Replaces kx_op_qkv in src/kernels/cuda/cx.cu:327-335.  The reference
 * planner hands this op the NVFP4 payload and scale pointers of a fused qkv
 * weight (src/plan/plan.c:272-275) but both reference kernel sets read them
 * as bf16; here a non-NULL `d` operand routes to the NVFP4 kernels with the
 * GEMM_F4 operand meaning, and a NULL `d` returns MM_ERR_UNSUPPORTED (the
 * bf16 GEMM is outside this library). */
mm_status kx_op_qkv(const mm_kcall *kc);

/* Replaces kx_op_lmhead in src/kernels/cuda/cx.cu:332-335 the same way: the
 * operands are a GEMM's (a = x, b = W, c = logits, n0 = M, n1 = K, n2 = N,
 * src/kernels/cpu/cx.c:187-190); a non-NULL `d` (block scales) makes it the
 * NVFP4 op, a NULL `d` returns MM_ERR_UNSUPPORTED. */
mm_status kx_op_lmhead(const mm_kcall *kc);

/* Replaces kx_op_silu_mul in src/kernels/cuda/cx.cu:275-284 (CPU twin
 * src/kernels/cpu/cx.c:155-167): c[i] = bf16(silu(a[i]) * b[i]) over n0 * n1
 * bf16 elements.  Served so that the op list of a whole MLP can run here, and
 * as the unfused form of mm_f4_mlp_gate_up. */
mm_status kx_op_silu_mul(const mm_kcall *kc);

/* Replaces kx_op_add_rmsnorm in src/kernels/cuda/cx.cu:223-260 (CPU twin
 * src/kernels/cpu/cx.c:132-150): a[m][i] = bf16(a[m][i] + b[m][i]) in place, then
 * c[m][i] = bf16(a[m][i] * inv * d[i]) with inv = 1 / sqrt(mean(a[m]^2) + eps) over
 * n0 rows of n1 bf16 values.  The reference planner emits it right behind the o
 * and down projections (src/plan/plan.c:440-449), so an op list of a whole layer's
 * linears runs here without leaving the library.  eps is the value registered with
 * mm_norm_eps_set (the reference reads kc->e->mc.norm_eps; the engine is opaque
 * here). */
mm_status kx_op_add_rmsnorm(const mm_kcall *kc);

/* Replaces mm_kx_invoke in src/kernels/kx.c:15-47 for the opcodes this
 * library owns: OP_GEMM_F4, OP_QKV and OP_LMHEAD (fp4 forms), OP_SILU_MUL, OP_ADD_RMSNORM and OP_NOP.  Same NULL checks
 * (kc, kc->op, kc->e -> MM_ERR_STATE); any other opcode returns
 * MM_ERR_UNSUPPORTED. */
mm_status mm_kx_invoke(const mm_kcall *kc);

/* Replaces kx_cuda_oppref in src/kernels/cuda/cx.cu (declared in
 * src/kernels/kx.h:43): 1 for the opcodes listed above, else 0. */
int kx_cuda_oppref(int op);

/* Runtime shim, replacing the parts of src/cuda/cuda_rt.c the launcher and
 * the engine use (declared in include/mimfer/cuda_rt.h:38-106).  Two
 * non-blocking streams, capture on the compute stream, no device allocation.
 * When this library is linked into a mimfer build these come from mimfer's
 * own cuda_rt.c instead (leave csrc/cuda/rt.c out of the link). */
int        mm_cuda_enabled(void);                       /* cuda_rt.h:42 */
mm_status  mm_cuda_device_count(int *n_out);            /* cuda_rt.h:44 */
mm_status  mm_cuda_init(int device_ordinal);            /* cuda_rt.h:47 */
mm_status  mm_cuda_shutdown(void);                      /* cuda_rt.h:48 */
void      *mm_cuda_stream_raw(mm_stream_id id);         /* cuda_rt.h:106 (cudaStream_t) */
int        mm_cuda_capturing(void);                     /* cuda_rt.h:94 */
#define MM_N_EVENTS 16                                  /* cuda_rt.h:55: fixed event pool */
mm_status  mm_event_record(int ev, mm_stream_id st);    /* cuda_rt.h:56 */
mm_status  mm_event_wait(int ev, mm_stream_id st);      /* cuda_rt.h:57 */
mm_status  mm_stream_sync(mm_stream_id st);             /* cuda_rt.h:58 */
mm_status  mm_h2d_async(void *dst, const void *src, size_t n, mm_stream_id st); /* :61 */
mm_status  mm_d2h_async(void *dst, const void *src, size_t n, mm_stream_id st); /* :62 */
mm_status  mm_mset_async(void *dst, int value, size_t n, mm_stream_id st);      /* :63 */

typedef struct mm_graph mm_graph;                       /* cuda_rt.h:66 */
mm_status  mm_graph_create(mm_graph **out);             /* :67 */
mm_status  mm_graph_capture_begin(mm_graph *g);         /* :69 */
mm_status  mm_graph_commit(mm_graph *g, const void *window_base,
                           size_t window_bytes, int hit_ratio_pct); /* :72 */
mm_status  mm_graph_launch(mm_graph *g, mm_stream_id st);           /* :74 */
void       mm_graph_destroy(mm_graph *g);                           /* :75 */

/* Logging, replacing mm_log in src/core/mimfer.c:37-60. Level 0 = errors
 * only ... 3 = debug; default 1. */
void mm_log_set_level(int level);

/* ======================================================================
 * 2. New surface (no counterpart in the reference)
 * ====================================================================== */

/* ---- global scale ------------------------------------------------------
 * The reference weight view carries payload + block scales only
 * (include/mimfer/tensor.h:121-126); NVFP4 checkpoints add one fp32 scale per
 * tensor.  The descriptor has no free slot for it, so it is registered per
 * weight, keyed by the block-scale base pointer (`d` of the descriptor).
 * Unregistered weights use 1.0f, which is bit-for-bit the reference maths. */
mm_status mm_f4_gscale_set(const void *scale_base, float gs);
float     mm_f4_gscale_get(const void *scale_base);
void      mm_f4_gscale_unset(const void *scale_base);   /* back to 1.0f; unknown keys are ignored */
uint32_t  mm_f4_gscale_room(void);                      /* registrations the table still takes  */
void      mm_f4_gscale_clear(void);

/* ---- split-K workspace ---------------------------------------------------
 * The launcher allocates nothing (reference rule: include/mimfer/alloc.h:4-29);
 * split-K variants need fp32 partials plus arrival counters.  The owner of the
 * activation arena donates a block once (the role the reference reserves as
 * e->ab.part, include/mimfer/engine.h:98).  Without a workspace the selector
 * only returns variants that need none.  The block is zeroed here, on the
 * compute stream; it must be 256-byte aligned device memory. */
mm_status mm_f4_workspace_set(void *dev_ptr, size_t bytes);
size_t    mm_f4_workspace_bytes(void);

/* ---- tile / variant selection (pure host C, no CUDA) ---------------------- */
typedef enum mm_f4_variant {
    MM_F4_V_ROWWARP = 0,  /* any K%16==0: one warp per weight row, shuffles  */
    MM_F4_V_STREAM  = 1,  /* decode: TMA-staged weight stream + warp MMA     */
    MM_F4_V_UMMA    = 2,  /* prefill: tcgen05 kind::f16, TMEM accumulators   */
    MM_F4_V_MX      = 4   /* decode: block-scaled tcgen05 MMA on the packed  */
                          /*   payload and its e4m3 scales as they lie in    */
                          /*   memory; activations as e2m1 digit planes      */
} mm_f4_variant;

typedef struct mm_f4_shape {
    uint32_t M, K, N;
    uint32_t sm_count;        /* SMs of the device (148 on B200)            */
    uint32_t ptr_align;       /* min alignment in bytes of x/payload/scale/y */
    size_t   ws_bytes;        /* workspace available (0 = none)              */
} mm_f4_shape;

typedef struct mm_f4_plan {
    int      variant;         /* mm_f4_variant                                */
    uint32_t m_tiles;         /* STREAM: 8-row activation tiles (1 to 4); MX: */
                              /*   groups of four activation rows (1 to 8);   */
                              /*   UMMA: tiles of the last, partial wave that */
                              /*   are cut into split_k K slices (0 = none)   */
    uint32_t tile_m, tile_n;  /* UMMA: CTA tile; STREAM/MX: tile_n =  */
                              /*   W rows per CTA, tile_m = padded activation */
                              /*   rows (MX: digit-plane rows, 24 per group)  */
    uint32_t split_k;         /* >= 1; UMMA: slices of each of those tiles    */
    uint32_t k_steps;         /* K / 256 (STREAM) or K / 64 (UMMA)            */
    uint32_t stages;          /* smem pipeline depth                          */
    uint32_t grid_x, grid_y, grid_z;
    uint32_t threads;
    uint32_t smem_bytes;      /* dynamic shared memory per CTA                */
    size_t   ws_needed;       /* bytes of workspace this plan uses            */
} mm_f4_plan;

/* Deterministic: the same shape always yields the same plan.  Returns
 * MM_ERR_SHAPE for K%16 != 0 or a zero extent. */
mm_status mm_f4_select(const mm_f4_shape *s, mm_f4_plan *out);
/* Force a variant (tests, sweeps); MM_ERR_UNSUPPORTED if the shape cannot run
 * on it. */
mm_status mm_f4_select_variant(const mm_f4_shape *s, int variant, mm_f4_plan *out);
/* Plan of the gated pair (mm_f4_mlp_gate_up): s->N = output features.
 * MM_ERR_UNSUPPORTED when only the unfused three-op form can run the shape. */
mm_status mm_f4_select_glu(const mm_f4_shape *s, mm_f4_plan *out);
/* Override for kx_op_gemm_f4: -1 = automatic (default). */
void      mm_f4_force_variant(int variant);

/* ---- flat launch ---------------------------------------------------------
 * Same maths as kx_op_gemm_f4 with the operands spelled out; enqueues on
 * `stream` (a cudaStream_t; NULL = the compute stream) and does not
 * synchronise.  Device pointers. */
mm_status mm_f4_linear(const void *x, const void *payload, const void *scale,
                       float gs, void *y, uint32_t M, uint32_t K, uint32_t N,
                       void *stream);

/* The activation side of the block-scaled decode kernel (no counterpart in the
 * reference, which keeps activations in bf16, src/kernels/cpu/cx.c:211).  The tensor
 * core multiplies e2m1 by e2m1, so the bf16 activations x [M][K] (M <= 32, K a
 * multiple of 256) are rewritten as six signed e2m1 digit planes per row with
 * power-of-two block scales.  A 16-wide block's unit is 2^-16 of its largest
 * magnitude's power of two (2^-19 of the row's, if that is larger): every value
 * that is a multiple of the unit is kept exactly - all values within 2^9 of the
 * block's largest - and the rest is rounded to the nearest multiple.  mm_f4_linear does
 * this itself in front of its kernel; an owner of a whole op list does it once per
 * distinct activation tensor per step, ahead of the ops (the op-list engine does,
 * in overlap mode, into the upper half of the workspace).  `scratch`: device
 * memory, 256-byte aligned, mm_f4_xslice_bytes(M, K) bytes.  Its layout, with
 * R = 6 * (M rounded up to a multiple of 4) plane rows:
 *   byte 0       float f[2 * m], f[2 * m + 1]: row m's value = (sum of its planes) * f1 * f2
 *   byte 1024    scratch of the two-pass slicing of an op group
 *   byte 16384   planes  [R][K / 2]   row 6 * m + p = digit plane p of activation row m,
 *                                     e2m1 codes, low nibble = even column
 *   then         scales  [R][K / 16]  one ue4m3 byte (a power of two) per 16-wide block
 * x[m][k] ~= f1 * f2 * sum over p of e2m1(planes[6m+p][k]) * ue4m3(scales[6m+p][k/16]);
 * rows m >= M are zero. */
size_t    mm_f4_xslice_bytes(uint32_t M, uint32_t K);
mm_status mm_f4_xslice(const void *x, uint32_t M, uint32_t K, void *scratch, size_t scratch_bytes, void *stream);

/* Gated MLP front half in one kernel (no single counterpart in the reference):
 * replaces the three ops the reference planner emits per layer
 * (src/plan/plan.c:223-247: OP_GEMM_F4 "gate", OP_GEMM_F4 "up", OP_SILU_MUL)
 *     y[m][j] = bf16( silu(G) * U ),  G = bf16(x . Wgate[j]),  U = bf16(x . Wup[j]),
 * i.e. the arithmetic of kx_op_silu_mul (src/kernels/cpu/cx.c:155-167) on the
 * values the two GEMMs would have stored; the [M][inter] gate and up buffers are
 * never written.  The two projections are separate NVFP4 tensors ([inter][K/2]
 * payload, [inter][K/16] scales each) anywhere in device memory, as long as the
 * payload and the scale tensors lie in the same order (both gate-first or both
 * up-first) and their distances are multiples of 16 bytes below 2^40 - true for
 * tensors staged one after the other into one weight arena.  M <= 32 runs the
 * decode kernel (split-K through the workspace), larger M the tcgen05 kernel.
 * MM_ERR_UNSUPPORTED if the shape needs the fallback kernel (K % 256 != 0,
 * unaligned operands) or the layout rule fails: run the three ops then. */
mm_status mm_f4_mlp_gate_up(const void *x, const void *gate_payload, const void *gate_scale,
                            float gs_gate, const void *up_payload, const void *up_scale,
                            float gs_up, void *y, uint32_t M, uint32_t K, uint32_t inter,
                            void *stream);
/* y = silu(gate) * up, elementwise on bf16 [n] (src/kernels/cuda/cx.cu:264-273):
 * the unfused form, enqueued on `stream`. */
mm_status mm_silu_mul(const void *gate, const void *up, void *y, size_t n, void *stream);

/* res += delta in place, y = rmsnorm(res) * gain on M rows of H bf16 values
 * (src/kernels/cuda/cx.cu:223-243), enqueued on `stream`; epsilon as registered
 * (default 1e-6, the value of the reference's model configurations). */
mm_status mm_add_rmsnorm(void *res, const void *delta, void *y, const void *gain, uint32_t M, uint32_t H,
                         void *stream);
mm_status mm_norm_eps_set(float eps);
float     mm_norm_eps_get(void);

/* Tensor-parallel form (no counterpart in the reference, which is single-GPU).
 * This rank owns output features [col0, col0 + N_local) of a layer with `ldy`
 * output features in total; payload/scale point at that row slice.  The
 * kernel's epilogue stores the slice into all `n_ranks` copies of the full
 * output y_all[r] ([M][ldy] bf16; y_all[0] is this GPU's own, the others are
 * peer-mapped device pointers, e.g. from a symmetric-memory rendezvous), so
 * the exchange rides on the compute kernel as unicast peer writes over NVLink
 * (stores at decode sizes; at prefill sizes one bulk copy from shared memory per
 * output-tile row and destination, and the CTAs of the first wave start spread over
 * the time the link needs for one wave's tiles, mm_f4_tune key 12).
 * The caller must run a cross-rank barrier on `stream` after the op before any
 * rank reads its copy, and must not let a rank start the next write into a
 * buffer its peers still read.  n_ranks <= 8; col0 and ldy multiples of 8. */
mm_status mm_f4_linear_tp(const void *x, const void *payload, const void *scale, float gs,
                          void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0,
                          uint32_t M, uint32_t K, uint32_t N_local, void *stream);

/* Cross-rank barrier for the tensor-parallel form (no counterpart in the
 * reference): one small kernel on `stream` (NULL = the compute stream).
 * flags_all[r] points at rank r's flag block: 64 bytes of memory every rank can
 * write (r == rank: this GPU's own block, the others peer-mapped), zeroed once
 * before the first barrier, indexed by rank.  After the kernel, every store any
 * rank issued on its stream before its own call of the same barrier is visible
 * here.  No argument changes between calls, so the call can be captured into a
 * graph.  A peer that does not arrive within about two seconds makes the wait give
 * up with MMB_DEV_TIMEOUT in the device status word (mm_f4_device_status,
 * MM_ERR_TIMEOUT from the synchronising calls) instead of hanging the GPU. */
mm_status mm_f4_tp_barrier(void *const *flags_all, uint32_t n_ranks, uint32_t rank, void *stream);

/* The exchange by the copy engines instead of the epilogue's stores (no counterpart in
 * the reference).  A rank runs mm_f4_linear_tp with n_ranks = 1 (its own copy only), on
 * the whole activations or on a chunk of rows, and then pushes what that call wrote:
 * columns [col0, col0 + cols) of rows [row0, row0 + rows) of y_all[0] go to the same
 * place in y_all[1 .. n_ranks - 1], one two-dimensional copy per peer, each on a side
 * stream of its own that waits for the compute stream's work up to this call.  The
 * compute stream itself goes on, so the next chunk's GEMM runs while the copy engines
 * drain this one over NVLink.  mm_f4_tp_push_join makes the compute stream wait for every
 * push since the last join; call it before mm_f4_tp_barrier.  ldy, col0 and cols are
 * multiples of 8 (16-byte rows); MM_ERR_SHAPE otherwise.  Issue both calls eagerly: they
 * have not been exercised inside a stream capture. */
mm_status mm_f4_tp_push(void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0, uint32_t cols,
                        uint32_t row0, uint32_t rows);
mm_status mm_f4_tp_push_join(void);

/* No counterpart in the reference.  The decode kernel of mm_f4_linear with its
 * split-K scratch built in, for callers that cannot hand over a workspace and
 * may not allocate one: code that runs under mimfer's rule that device memory
 * is claimed by a few cudaMalloc calls at start-up and never afterwards
 * (include/mimfer/alloc.h:4-29), or a serving loop that must not touch the
 * allocator.  Calls no cudaMalloc/cudaFree and no allocating library routine;
 * x, payload, scale and y are still the caller's (device pointers), `stream`
 * is a cudaStream_t (NULL = the legacy default stream) and the call does not
 * synchronise.
 *  - Scratch is one file-scope device array of 16 KiB + 4 MiB, resident on
 *    every GPU that loads the library until the process exits.  A shape whose
 *    split needs more returns MM_ERR_CAPACITY (the log names both numbers);
 *    shapes the decode kernel cannot take (M > 32, K % 256 != 0, operands not
 *    16-byte aligned) return MM_ERR_UNSUPPORTED.
 *  - The first call on each device looks the array's device address up
 *    (cudaGetSymbolAddress) and sets kernel attributes; make that first call
 *    outside any stream capture, with the device current.
 *  - All calls share the array and it keeps the previous call's contents; the
 *    arrival counters are zeroed on `stream` before each launch.  Two calls of
 *    one process that overlap on the GPU (issued on different streams) race on
 *    it: keep the calls on one stream or order them with events.  Separate
 *    processes have separate copies.
 *  - A device-side wait that gave up (the kernel's waits are bounded) raises a
 *    bit in the device status word and the output is then not valid.  A caller
 *    that uses the runtime shim reads it with mm_f4_device_status; one that does
 *    not reads it with mm_f4_device_status_on(stream, &flags), which synchronises
 *    the caller's own stream, returns the bits (1 = a wait timed out) and clears
 *    them.  Check it wherever the stream is synchronised anyway. */
mm_status mm_f4_linear_static_ws(const void *x, const void *payload, const void *scale,
                                 float gs, void *y, uint32_t M, uint32_t K, uint32_t N,
                                 void *stream);
mm_status mm_f4_device_status_on(void *stream, unsigned *flags_out);

/* Host-buffer form: copies x (pinned or pageable host memory) to `x_dev`,
 * runs the op on resident device weights, copies y back to `y_host` and
 * synchronises.  This is the call the end-to-end benchmark times. */
mm_status mm_f4_linear_host(const void *x_host, void *x_dev,
                            const void *payload_dev, const void *scale_dev,
                            float gs, void *y_dev, void *y_host,
                            uint32_t M, uint32_t K, uint32_t N);

/* Reads and clears the device-side status word that bounded waits set. */
mm_status mm_f4_device_status(unsigned *flags_out);
/* Count of kernels this library launched since the last call (then reset). */
unsigned long long mm_f4_launch_count(int reset);

/* Device decode probe: for every (nibble n, scale byte s) writes the fp32
 * bits of the dequantised weight as each kernel family computes it, to three
 * device arrays of 4096 uint32 (index s*16+n): the bf16 tensor-core operand
 * form (rescaled), the row-warp fp32 form, and the fp16 tensor-core operand
 * form. */
mm_status mm_f4_decode_probe(uint32_t *out_bf16_dev, uint32_t *out_f32_dev,
                             uint32_t *out_f16_dev);

/* Self test of the bounded device-side waits: launches one thread that waits on
 * a barrier nothing completes.  The wait must expire (about one second), the
 * kernel must return, and this call must report MM_ERR_TIMEOUT with
 * *done_dev == 1; the device stays usable.  done_dev: one device uint32. */
mm_status mm_f4_wait_selftest(unsigned *done_dev);

/* Knobs for tests and sweeps; the defaults are what the benchmark uses.
 * Returns the previous value, or -1 for an unknown key.
 *   key 1  programmatic dependent launch: an op's weight prefetch overlaps the
 *          tail of the kernel in front of it in the stream (1 = on, default)
 *   key 2  weight rows per CTA of the decode kernels (0 = the planner's choice)
 *   key 3  K slices of the decode kernels (0 = the planner's choice)
 *   key 5  decode ops on the block-scaled tensor kernel (1, default) or on the
 *          CUDA-core streaming kernel (0)
 *   key 6  cap on the pipeline stages of a group launch (0 = as many as fit, default)
 *   key 10 the work units of a group launch are handed out as its CTAs ask for them
 *          (1, default) or dealt round-robin in advance (0)
 *   key 11 copy streams per peer of mm_f4_tp_push (0 = about eight over all peers, default)
 *   key 12 tensor-parallel prefill launches start the CTAs of their first wave spread over
 *          this many percent of the time NVLink needs for one wave's tiles (100, default;
 *          0 = all together; at most 400)
 *   key 9  the ops of a group launch run in order of activation rows, most first
 *          (1, default), or in list order (0)
 *   key 8  the prefill kernel cuts the tiles of its last, partial wave into K slices
 *          (1, default) or runs them whole (0)
 *   key 7  group launches carry a persisting L2 access-policy window over the digit
 *          planes of their activations (0 = off, default; sets the context's persisting
 *          L2 carve-out to 32 MiB on first use)
 * Key 4 (measurement modes that skip loads, arithmetic or the split-K exchange)
 * exists only in a library built with -DMMB_MEASURE_MODES. */
int mm_f4_tune(int key, int value);

/* ---- timing on the compute stream (events with timing enabled) ----------- */
mm_status mm_time_begin(void);
mm_status mm_time_end(float *ms_out);        /* synchronises */

/* ---- quantising packer + seeded generator (host) --------------------------
 * W fp32 [N][K] row-major -> payload [N][K/2], scales [N][K/16], *gs.
 * gs = max|W| / (6*448); block scale = e4m3_rne_sat(amax_block / (6*gs));
 * nibble = e2m1_rne_sat(w / (decode(scale) * gs)).  Layout as
 * include/mimfer/tensor.h:17-19. */
mm_status mm_f4_pack(const float *W, uint32_t N, uint32_t K,
                     uint8_t *payload, uint8_t *scales, float *gs_out);
/* out[i] = mean + std * normal(), splitmix64 (include/mimfer/mimfer.h:149-155)
 * + Box-Muller, one stream per row of `cols` values so rows can be generated
 * in parallel with identical results. */
void mm_fill_normal_f32(float *out, uint64_t rows, uint64_t cols,
                        uint64_t seed, float mean, float std);
void mm_f32_to_bf16(const float *in, uint16_t *out, uint64_t n);
void mm_bf16_to_f32(const uint16_t *in, float *out, uint64_t n);
/* Generate + pack one weight without materialising fp32 W (row blocks). gs is
 * computed in a first pass over the same stream. */
mm_status mm_f4_make_weight(uint32_t N, uint32_t K, uint64_t seed, float std,
                            uint8_t *payload, uint8_t *scales, float *gs_out);

/* ---- NVFP4 tensors in a weights section -----------------------------------
 * The reference loader walks the tensor index of the artifact's weights
 * section and stages every tensor into the weight arena
 * (src/model/tensor_registry.c:372-560; layout in tensor_registry.h:86-120) but
 * rejects MM_DT_FP4E2M1 entries (tensor_registry.c:468-474).  These calls read
 * the same index with fp4 entries admitted.  An fp4 entry's bytes are payload
 * (rows*cols/2), block scales (rows*cols/16) and the fp32 global scale (4),
 * back to back; cols % 16 == 0.  Errors as in the reference: MM_ERR_CORRUPT
 * for a bad header, truncated index, wrong nbytes, bytes outside the payload or
 * a duplicate name; MM_ERR_UNSUPPORTED for any other dtype; MM_ERR_SHAPE for an
 * fp4 tensor with cols % 16 != 0. */
typedef struct mm_f4_went {
    char     name[48];
    uint32_t rows, cols;
    uint8_t  dtype;           /* MM_DT_BF16 or MM_DT_FP4E2M1 */
    uint64_t off, nbytes;     /* within the section payload   */
} mm_f4_went;
typedef struct mm_f4_wreg mm_f4_wreg;

/* rows*cols/2 + rows*cols/16 + 4 */
uint64_t  mm_f4_tensor_bytes(uint32_t rows, uint32_t cols);
/* Validate the index; ents may be NULL to count only (cap ignored then). */
mm_status mm_f4_weights_parse(const uint8_t *data, size_t len, mm_f4_went *ents, uint32_t cap,
                              uint32_t *n_out);
/* Device bytes the tensors take when bump-placed on 256-byte boundaries. */
size_t    mm_f4_weights_arena_bytes(const mm_f4_went *ents, uint32_t n);
/* Copy every tensor into the caller's device block (256-byte aligned, at least
 * mm_f4_weights_arena_bytes; no allocation here), in index order, an fp4 tensor
 * as [payload | scales]; register each fp4 tensor's global scale
 * (mm_f4_gscale_set) and return a name -> view registry.  Copies run on the
 * transfer stream and are complete on return.  mm_cuda_init first. */
mm_status mm_f4_weights_stage(const uint8_t *data, size_t len, void *arena_dev, size_t arena_bytes,
                              mm_f4_wreg **out);
uint32_t  mm_f4_weights_count(const mm_f4_wreg *r);
size_t    mm_f4_weights_used(const mm_f4_wreg *r);
/* The reference's mm_tens_find (include/mimfer/engine.h:86) for this registry:
 * MM_ERR_RANGE when the name is absent, MM_ERR_UNSUPPORTED when the tensor is of
 * the other kind. */
mm_status mm_f4_weights_find(const mm_f4_wreg *r, const char *name, mm_wt *w_out, float *gs_out);
mm_status mm_f4_weights_find_bf16(const mm_f4_wreg *r, const char *name, const void **data_out,
                                  uint32_t *rows_out, uint32_t *cols_out);
void      mm_f4_weights_free(mm_f4_wreg *r);

/* ---- op-list engine (graph-captured sequence of linears) ------------------ */
typedef struct mm_lin_engine mm_lin_engine;
mm_status mm_lin_engine_create(mm_lin_engine **out, uint32_t max_ops);
mm_status mm_lin_engine_add(mm_lin_engine *e, const mm_op_desc *op);
/* Tensor-parallel form of an OP_GEMM_F4 (no counterpart in the reference): op->n2 output
 * features are this rank's shard of a wider output; the kernel stores them at column
 * `col0` of every rank's [M][ldy] copy of it, y_all[0] == op->c being this rank's own
 * (peer-mapped pointers for the others, as for mm_f4_linear_tp).  Such ops join group
 * launches like any decode op; close a step with mm_f4_tp_barrier.  Such an op takes no
 * host output buffer (mm_lin_engine_bind_host and mm_lin_engine_launch_host refuse one):
 * its output is a column slice of a buffer the other ranks complete. */
mm_status mm_lin_engine_add_tp(mm_lin_engine *e, const mm_op_desc *op, void *const *y_all, uint32_t n_ranks,
                               uint32_t ldy, uint32_t col0);
uint32_t  mm_lin_engine_n_ops(const mm_lin_engine *e);
/* on != 0: an OP_SILU_MUL added right after the two OP_GEMM_F4 that produce its
 * operands from the same activations (the MLP front half as the reference
 * planner emits it, src/plan/plan.c:223-247) replaces the three ops by one
 * fused kernel (mm_f4_mlp_gate_up) whenever that kernel can take them; the op
 * count drops by two and the gate/up buffers are no longer written.  Off by
 * default. */
mm_status mm_lin_engine_fuse_mlp(mm_lin_engine *e, int on);
/* on != 0: dependency-aware launch order.  The engine compares the memory every
 * op reads and writes (activations, outputs, split-K scratch) with the ops still
 * in flight before it; an op that shares nothing with them is launched so that
 * it starts while they drain (programmatic dependent launch without the leading
 * wait) and still completes after them; every other op waits for its
 * predecessor as before.  Results are identical; only ops served by the decode
 * kernel run ahead.  Needs a workspace of at least 16 MiB to let split-K ops
 * overlap (each of four regions serves one op in flight).  Off by default.
 * on == 2 additionally lets an op that runs ahead take fewer, longer K slices
 * than it would alone (it shares the SMs with its predecessors, so about half
 * of them is its fair share): faster, still the same bits from run to run,
 * but no longer the bits of the serial order, because the fp32 partial sums are
 * cut at other places.
 * mm_lin_engine_n_independent: how many ops of the last dispatch or capture ran
 * ahead. */
mm_status mm_lin_engine_overlap(mm_lin_engine *e, int on);
uint32_t  mm_lin_engine_n_independent(const mm_lin_engine *e);
/* Overlap mode, block-scaled decode path: how many distinct activation tensors of
 * the last dispatch or capture were turned into digit planes ahead of the ops, on
 * the transfer stream (inputs of the step that no earlier op of the list writes). */
uint32_t  mm_lin_engine_n_sliced_ahead(const mm_lin_engine *e);
/* on != 0 (the default): group mode.  Runs of consecutive decode linears (M <= 32)
 * that share no memory with each other - q, k and v of a layer, gate and up, a
 * benchmark's stand-alone linears - become ONE persistent launch of the
 * block-scaled kernel: the CTAs take the ops' work units one after the other from
 * a shared counter and the weight stream does not stop between ops (up to 48 ops
 * per launch; an activation tensor several ops read is sliced once; inside a launch
 * the ops run in order of activation rows, most first).  Results are those of the
 * single launches up to the places where K is cut.  Needs a workspace of at least
 * 32 MiB; without one, and for ops the block-scaled kernel does not take, the ops
 * are dispatched one by one.  Before capture.
 * mm_lin_engine_n_group_launches: group launches of the last dispatch or capture. */
mm_status mm_lin_engine_group(mm_lin_engine *e, int on);
uint32_t  mm_lin_engine_n_group_launches(const mm_lin_engine *e);
/* Capture all ops into one CUDA graph (reference pattern:
 * src/plan/plan.c:479-507). */
mm_status mm_lin_engine_capture(mm_lin_engine *e);
/* Replay the graph (or dispatch op by op if not captured); no sync. */
mm_status mm_lin_engine_launch(mm_lin_engine *e);
/* One step with host buffers, the shape of a serving round in the reference
 * engine (src/engine/engine.c:233-357: inputs up, one graph launch, results
 * down, one host sync): for every op i with x_host[i] != NULL the activations
 * are copied from (pinned) host memory into the op's device operand `a`, the
 * graph is replayed (or the ops dispatched), every y_host[i] != NULL receives
 * the op's output, then the compute stream is synchronised and the device
 * status word checked.  Arrays have mm_lin_engine_n_ops entries; either may be
 * NULL as a whole. */
mm_status mm_lin_engine_launch_host(mm_lin_engine *e, const void *const *x_host,
                                    void *const *y_host);
/* The same step with the copies inside the graph.  Bind pinned host buffers to
 * the op list before mm_lin_engine_capture (entries as in
 * mm_lin_engine_launch_host; the pointers are baked into the graph, so the
 * caller refills and reads the same buffers every step, the way the reference
 * engine keeps its pinned staging for a round).  The captured graph then
 * uploads every op's activations on the transfer stream ahead of the kernels
 * (op i waits only for its own upload) and downloads every output right after
 * its kernel while the next kernels run.  mm_lin_engine_step_bound replays
 * that graph, synchronises once and checks the device status word; with
 * buffers bound, mm_lin_engine_launch_host returns MM_ERR_BUSY. */
mm_status mm_lin_engine_bind_host(mm_lin_engine *e, const void *const *x_host, void *const *y_host);
mm_status mm_lin_engine_step_bound(mm_lin_engine *e);
/* How many consecutive ops share one upload-complete event in the bound graph
 * (default 1: every op waits for its own upload only).  A copy node costs
 * several microseconds whatever its size and a cross-stream dependency a few
 * more per kernel, so a list of short ops does better with larger groups: the
 * first op of a group waits for the uploads of the whole group, the others for
 * nothing.  With group launches on, a launch ends where an upload group ends, so
 * that one launch's downloads and the next one's uploads overlap the kernels
 * between them (measured on the ten-op decode sweep, whose kernels alone take
 * 0.138 ms: 0.282 ms per step with one group of 10, 0.250 with groups of 5,
 * 0.229 with groups of 4, 0.242 with groups of 3, 0.273 with groups of 2).
 * Before capture. */
mm_status mm_lin_engine_upload_group(mm_lin_engine *e, uint32_t ops_per_event);
/* on != 0 (default): the uploads of a group go up as ONE kernel that reads the
 * pinned host buffers over PCIe (they must be mapped for the device, which
 * cudaHostAlloc memory is, and 16-byte aligned; other buffers and groups of
 * more than 32 buffers fall back to copy nodes), and the outputs of a group
 * launch go down the same way: one kernel that writes the pinned host buffers.
 * on == 0: always copy nodes.  Before capture. */
mm_status mm_lin_engine_upload_kernel(mm_lin_engine *e, int on);
void      mm_lin_engine_destroy(mm_lin_engine *e);

#ifdef __cplusplus
}
#endif
#endif /* MIMFER_B200_H */
