/* Internal helpers shared by the host C sources: logging and the
 * check-and-return macros (policy as in include/mimfer/mimfer.h:100-118 of the
 * mimfer tree: log once, return the status, no unwinding). */
#ifndef MMB_CORE_H
#define MMB_CORE_H

#include "mimfer_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

void mmb_log(int lvl, const char *file, int line, const char *fmt, ...)
    __attribute__((format(printf, 4, 5)));

#define MM_LOGE(...) mmb_log(0, __FILE__, __LINE__, __VA_ARGS__)
#define MM_LOGW(...) mmb_log(1, __FILE__, __LINE__, __VA_ARGS__)
#define MM_LOGI(...) mmb_log(2, __FILE__, __LINE__, __VA_ARGS__)
#define MM_LOGD(...) mmb_log(3, __FILE__, __LINE__, __VA_ARGS__)

#define MM_CHECK(expr)                                                   \
    do {                                                                 \
        mm_status s_ = (expr);                                           \
        if (s_ != MM_OK) {                                               \
            MM_LOGE("%s: %s", #expr, mm_status_str(s_));                 \
            return s_;                                                   \
        }                                                                \
    } while (0)

#define MM_REQUIRE(cond, code)                                           \
    do {                                                                 \
        if (!(cond)) {                                                   \
            MM_LOGE("required: %s", #cond);                              \
            return (code);                                               \
        }                                                                \
    } while (0)

/* The gated pair as an op: `op` is the gate projection's OP_GEMM_F4 descriptor
 * with c = the output of silu(gate) * up, the up projection comes beside it.
 * Same synchronisation and error behaviour as kx_op_gemm_f4. */
mm_status mmb_op_mlp_gate_up(const mm_op_desc *op, const void *up_payload, const void *up_scale);
/* Would mm_f4_mlp_gate_up take these operands?  Host-only check. */
int mmb_gate_up_fusable(const void *x, const void *gate_payload, const void *gate_scale,
                        const void *up_payload, const void *up_scale, const void *y,
                        uint32_t M, uint32_t K, uint32_t inter);

/* Engine -> launcher, for the next op only: how to order the launch against its
 * predecessor (MMB_PDL_* of kernels/launch.h, -1 = the launcher's default),
 * which workspace region its scratch lives in, whether an op that runs ahead
 * may take fewer, longer K slices than it would alone, and whether it reads the
 * activations the op before it already turned into digit planes (block-scaled
 * decode path: the planes are shared instead of made again). */
void mmb_next_op_context(int pdl_mode, int ws_region, int shallow_split, int share_x);
/* For the next op only: its activations' digit planes already lie at `planes_ws`
 * (made by mm_f4_xslice into the plane cache), so the op launches no slicing
 * kernel and waits for none. */
void mmb_next_op_planes(void *planes_ws);
/* The part of the workspace set aside for digit planes made ahead of their ops
 * (NULL / 0 when the workspace is too small to divide). */
void *mmb_plane_cache(size_t *bytes_out);
/* A run of mutually independent decode linears as one persistent launch of the
 * block-scaled kernel.  begin: open a group (launch mode and workspace region as
 * for a single op); add: MM_OK, MM_ERR_CAPACITY (full: launch and open another)
 * or MM_ERR_UNSUPPORTED (the op does not run on that kernel); launch: enqueue the
 * slicing of the group's activations and the kernel, then synchronise like an op. */
mm_status mmb_group_begin(int pdl_mode, int ws_region);
mm_status mmb_group_add(const mm_op_desc *op, int glu, const void *up_payload, const void *up_scale);
mm_status mmb_group_add_tp(const mm_op_desc *op, void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0);
mm_status mmb_op_linear_tp(const mm_op_desc *op, void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0);
mm_status mmb_group_launch(void);
uint32_t  mmb_group_size(void);
/* Regions the workspace is cut into, so that ops in flight together never share
 * scratch (1 when the workspace is too small to divide). */
int mmb_ws_regions(void);
/* Drop the launcher's per-device state (runtime shutdown or re-initialisation). */
void mmb_launcher_reset(void);
/* Grow the runtime shim's event pool (mm_event_record / mm_event_wait indices)
 * to at least n events; set-up time only. */
mm_status mmb_event_pool_reserve(int n);
/* The plan the launcher would pick for this op (glu: the op is a fused gate/up
 * pair, n2 = output features). */
mm_status mmb_plan_for_op(const mm_op_desc *op, int glu, mm_f4_plan *out);

static inline size_t mmb_align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

#ifdef __cplusplus
}
#endif
#endif
