/*
 * Op-list engine: a fixed sequence of NVFP4 linear ops, dispatched one by one
 * or captured once into a CUDA graph and replayed.
 *
 * In mimfer the planner fills a flat array of address-fixed descriptors
 * (src/plan/plan.c:386-473), runs them through the dispatcher
 * (plan_run_ops, plan.c:119-130) and captures that walk into a graph at load
 * (capture_one, plan.c:479-507; launch, plan.c:132-138).  This engine is the
 * same mechanism restricted to the ops this library serves; the descriptors
 * are the reference's mm_op_desc, so a reference plan's linear ops can be
 * appended unchanged.
 */
#include "../core/core.h"
#include "../kernels/launch.h"
#include <stdlib.h>
#include <string.h>

/* Engine-private opcode: gate projection, up projection and silu(gate) * up as
 * one kernel.  The descriptor is the gate GEMM's with c = the SILU_MUL output;
 * the up projection's tensors sit in the side array. */
#define MMB_OP_GATE_UP ((mm_op)(OP_N + 1))

typedef struct up_operands { const void *payload, *scale; } up_operands;
/* tensor-parallel linear: every rank's copy of the full output, its row pitch, this op's first column */
typedef struct tp_dst { void *y[8]; uint32_t n, ldy, col0; } tp_dst;

struct mm_lin_engine {
    mm_op_desc  *ops;
    up_operands *up;            /* [max_ops], used by MMB_OP_GATE_UP entries */
    tp_dst      *tp;            /* [max_ops], n > 0 for ops added with mm_lin_engine_add_tp */
    uint32_t     n_ops, max_ops;
    mm_graph    *graph;
    int          captured;
    int          fuse_mlp;
    int          overlap;
    int          group;             /* runs of independent decode linears as one persistent launch */
    uint32_t     n_group_launches;  /* group launches of the last walk */
    uint32_t     n_independent;     /* ops of the last walk launched without a leading wait */
    /* host buffers bound before capture: the copies become nodes of the graph */
    const void **x_bound;           /* [max_ops] pinned host source of op i's activations, or NULL */
    void       **y_bound;           /* [max_ops] pinned host destination of op i's output, or NULL  */
    int          bound, bound_captured;
    void       **planes;            /* [max_ops] op i's digit planes in the plane cache, or NULL    */
    int         *plane_ev;          /* [max_ops] event that says they are there (-1: already waited) */
    uint32_t     n_plane_slots;     /* distinct activation tensors sliced ahead in the last walk    */
    uint32_t     upload_group;      /* ops whose uploads share one event (>= 1) */
    int          upload_kernel;     /* uploads of a group as one kernel instead of copy nodes */
};

mm_status mm_lin_engine_create(mm_lin_engine **out, uint32_t max_ops)
{
    MM_REQUIRE(out && max_ops > 0, MM_ERR_STATE);
    mm_lin_engine *e = (mm_lin_engine *)calloc(1, sizeof *e);
    if (!e)
        return MM_ERR_NOMEM;
    e->ops = (mm_op_desc *)calloc(max_ops, sizeof(mm_op_desc));
    e->up = (up_operands *)calloc(max_ops, sizeof(up_operands));
    e->tp = (tp_dst *)calloc(max_ops, sizeof(tp_dst));
    if (!e->ops || !e->up || !e->tp) {
        free(e->ops);
        free(e->up);
        free(e->tp);
        free(e);
        return MM_ERR_NOMEM;
    }
    e->x_bound = (const void **)calloc(max_ops, sizeof(void *));
    e->y_bound = (void **)calloc(max_ops, sizeof(void *));
    e->planes = (void **)calloc(max_ops, sizeof(void *));
    e->plane_ev = (int *)calloc(max_ops, sizeof(int));
    if (!e->x_bound || !e->y_bound || !e->planes || !e->plane_ev) {
        mm_lin_engine_destroy(e);
        return MM_ERR_NOMEM;
    }
    e->max_ops = max_ops;
    e->upload_group = 1;
    e->upload_kernel = 1;
    e->group = 1;
    *out = e;
    return MM_OK;
}

mm_status mm_lin_engine_upload_group(mm_lin_engine *e, uint32_t ops_per_event)
{
    MM_REQUIRE(e && ops_per_event >= 1, MM_ERR_STATE);
    MM_REQUIRE(!e->captured, MM_ERR_BUSY);
    e->upload_group = ops_per_event;
    return MM_OK;
}

mm_status mm_lin_engine_upload_kernel(mm_lin_engine *e, int on)
{
    MM_REQUIRE(e, MM_ERR_STATE);
    MM_REQUIRE(!e->captured, MM_ERR_BUSY);
    e->upload_kernel = on ? 1 : 0;
    return MM_OK;
}

mm_status mm_lin_engine_bind_host(mm_lin_engine *e, const void *const *x_host, void *const *y_host)
{
    MM_REQUIRE(e && e->n_ops > 0, MM_ERR_STATE);
    MM_REQUIRE(!e->captured, MM_ERR_BUSY);
    e->bound = 0;
    /* the output of a tensor-parallel op is a column slice of a wider buffer, completed by
     * the other ranks: it has no host destination of its own (read the full buffer after
     * the step's barrier) */
    for (uint32_t i = 0; y_host && i < e->n_ops; i++)
        if (e->tp[i].n && y_host[i])
            return MM_ERR_UNSUPPORTED;
    for (uint32_t i = 0; i < e->n_ops; i++) {
        e->x_bound[i] = x_host ? x_host[i] : NULL;
        e->y_bound[i] = y_host ? y_host[i] : NULL;
        if (e->ops[i].op != OP_NOP && (e->x_bound[i] || e->y_bound[i]))
            e->bound = 1;
    }
    return MM_OK;
}

mm_status mm_lin_engine_fuse_mlp(mm_lin_engine *e, int on)
{
    MM_REQUIRE(e, MM_ERR_STATE);
    MM_REQUIRE(!e->captured, MM_ERR_BUSY);
    e->fuse_mlp = on ? 1 : 0;
    return MM_OK;
}

/* The reference planner's MLP front half (src/plan/plan.c:223-247) is
 * GEMM_F4 x -> gate, GEMM_F4 x -> up, SILU_MUL (gate, up) -> y.  When the SILU_MUL
 * arrives and the two ops before it are exactly that pair, and the fused kernel
 * can take the operands, the three collapse into one MMB_OP_GATE_UP; the gate and
 * up buffers are then never written. */
static int try_fuse_mlp(mm_lin_engine *e, const mm_op_desc *silu)
{
    if (!e->fuse_mlp || e->n_ops < 2)
        return 0;
    mm_op_desc *g = &e->ops[e->n_ops - 2], *u = &e->ops[e->n_ops - 1];
    if (g->op != OP_GEMM_F4 || u->op != OP_GEMM_F4)
        return 0;
    if (g->c == silu->b && u->c == silu->a) {           /* emitted up first */
        mm_op_desc *t = g; g = u; u = t;
    }
    if (g->c != silu->a || u->c != silu->b || g->a != u->a || g->n0 != u->n0 || g->n1 != u->n1 ||
        g->n2 != u->n2 || silu->n0 != g->n0 || silu->n1 != g->n2)
        return 0;
    if (!mmb_gate_up_fusable(g->a, g->b, g->d, u->b, u->d, silu->c, g->n0, g->n1, g->n2))
        return 0;
    mm_op_desc f = *g;
    up_operands upo = { u->b, u->d };
    f.op = MMB_OP_GATE_UP;
    f.c = silu->c;
    memcpy(f.note, "gate+up+silu", 13);
    e->n_ops -= 2;
    e->ops[e->n_ops] = f;
    e->up[e->n_ops] = upo;
    e->n_ops++;
    return 1;
}

mm_status mm_lin_engine_add(mm_lin_engine *e, const mm_op_desc *op)
{
    MM_REQUIRE(e && op, MM_ERR_STATE);
    MM_REQUIRE(!e->captured, MM_ERR_BUSY);
    MM_REQUIRE(e->n_ops < e->max_ops, MM_ERR_CAPACITY);
    MM_REQUIRE(kx_cuda_oppref(op->op), MM_ERR_UNSUPPORTED);
    if (op->op == OP_SILU_MUL) {
        MM_REQUIRE(op->a && op->b && op->c, MM_ERR_STATE);
        if (op->n0 == 0 || op->n1 == 0)
            return MM_ERR_SHAPE;
        if (try_fuse_mlp(e, op))
            return MM_OK;
    } else if (op->op == OP_ADD_RMSNORM) {
        MM_REQUIRE(op->a && op->b && op->c && op->d, MM_ERR_STATE);
        if (op->n0 == 0 || op->n1 == 0)
            return MM_ERR_SHAPE;
    } else if (op->op != OP_NOP) {
        MM_REQUIRE(op->a && op->b && op->c && op->d, MM_ERR_STATE);
        if (op->n0 == 0 || op->n1 == 0 || op->n2 == 0 || op->n1 % 16 != 0)
            return MM_ERR_SHAPE;
    }
    memset(&e->tp[e->n_ops], 0, sizeof(tp_dst));
    e->ops[e->n_ops++] = *op;
    return MM_OK;
}

/* bytes of the op's first input and of its output (host-buffer step) */
/* A linear whose n2 output features are this rank's shard of a wider output: the kernel
 * stores them at column col0 of every rank's [M][ldy] copy (y_all[0] = op->c, this rank's).
 * Inside a group launch, or as mm_f4_linear_tp when it runs on its own. */
mm_status mm_lin_engine_add_tp(mm_lin_engine *e, const mm_op_desc *op, void *const *y_all, uint32_t n_ranks,
                               uint32_t ldy, uint32_t col0)
{
    MM_REQUIRE(e && op && y_all, MM_ERR_STATE);
    MM_REQUIRE(n_ranks >= 1 && n_ranks <= 8, MM_ERR_RANGE);
    MM_REQUIRE(op->op == OP_GEMM_F4 && y_all[0] == op->c, MM_ERR_STATE);
    MM_REQUIRE((uint64_t)col0 + op->n2 <= ldy, MM_ERR_SHAPE);
    for (uint32_t d = 0; d < n_ranks; d++)
        MM_REQUIRE(y_all[d] && ((uintptr_t)y_all[d] & 15u) == 0, MM_ERR_STATE);
    const uint32_t at = e->n_ops;
    MM_CHECK(mm_lin_engine_add(e, op));
    if (e->n_ops != at + 1u)
        return MM_ERR_STATE;
    tp_dst *t = &e->tp[at];
    for (uint32_t d = 0; d < n_ranks; d++) t->y[d] = y_all[d];
    t->n = n_ranks; t->ldy = ldy; t->col0 = col0;
    return MM_OK;
}

static size_t op_in_bytes(const mm_op_desc *op) { return (size_t)op->n0 * op->n1 * 2u; }
static size_t op_out_bytes(const mm_op_desc *op)
{
    return (size_t)op->n0 * (op->op == OP_SILU_MUL || op->op == OP_ADD_RMSNORM ? op->n1 : op->n2) * 2u;
}

uint32_t mm_lin_engine_n_ops(const mm_lin_engine *e) { return e ? e->n_ops : 0; }

mm_status mm_lin_engine_overlap(mm_lin_engine *e, int on)
{
    MM_REQUIRE(e, MM_ERR_STATE);
    MM_REQUIRE(!e->captured, MM_ERR_BUSY);
    e->overlap = on < 0 ? 0 : (on > 2 ? 2 : on);
    return MM_OK;
}

uint32_t mm_lin_engine_n_independent(const mm_lin_engine *e) { return e ? e->n_independent : 0; }
uint32_t mm_lin_engine_n_sliced_ahead(const mm_lin_engine *e) { return e ? e->n_plane_slots : 0; }

mm_status mm_lin_engine_group(mm_lin_engine *e, int on)
{
    MM_REQUIRE(e, MM_ERR_STATE);
    MM_REQUIRE(!e->captured, MM_ERR_BUSY);
    e->group = on ? 1 : 0;
    return MM_OK;
}

uint32_t mm_lin_engine_n_group_launches(const mm_lin_engine *e) { return e ? e->n_group_launches : 0; }

/* ---- which ops may run ahead of their predecessors --------------------------
 * The reference engine serialises its ops on one stream (src/plan/plan.c:119-130)
 * although many neighbours do not depend on each other: q, k and v read the same
 * activations, as do gate and up.  With overlap on, an op that neither reads nor
 * writes anything a kernel still in flight touches is launched in the
 * INDEPENDENT form of kernels/launch.h: it starts streaming weights and
 * activations while its predecessors drain, fills the SMs they leave idle, and
 * still completes after them.  "In flight" = every op since, and including, the
 * last op that waited for its predecessor; split-K scratch counts as touched
 * memory, so ops in flight together use different workspace regions. */
typedef struct span { uintptr_t lo, hi; } span;

static span mk_span(const void *p, size_t bytes)
{
    span s = { (uintptr_t)p, (uintptr_t)p + bytes };
    return s;
}
static int spans_meet(span a, span b) { return a.lo < b.hi && b.lo < a.hi; }

/* reads[0..1] and writes[0..1] of an op (weights and gains are never written, so
 * they do not count).  ADD_RMSNORM updates its first operand in place. */
static void op_spans(const mm_lin_engine *e, const mm_op_desc *op, span reads[2], span writes[2])
{
    size_t in = op_in_bytes(op);
    const int two = op->op == OP_SILU_MUL || op->op == OP_ADD_RMSNORM;
    reads[0] = mk_span(op->a, in);
    reads[1] = two ? mk_span(op->b, in) : mk_span(op->a, 0);
    writes[0] = mk_span(op->c, op_out_bytes(op));
    if (op >= e->ops && op < e->ops + e->n_ops && e->tp[op - e->ops].n)      /* a column slice of [M][ldy] */
        writes[0] = mk_span(op->c, (size_t)op->n0 * e->tp[op - e->ops].ldy * 2u);
    writes[1] = op->op == OP_ADD_RMSNORM ? mk_span(op->a, in) : mk_span(op->c, 0);
}

static int ops_independent(const mm_lin_engine *e, const mm_op_desc *p, const mm_op_desc *q)
{
    span pr[2], qr[2], pw[2], qw[2];
    op_spans(e, p, pr, pw);
    op_spans(e, q, qr, qw);
    for (int i = 0; i < 2; i++)
        for (int j = 0; j < 2; j++)
            if (spans_meet(pw[i], qw[j]) || spans_meet(pw[i], qr[j]) || spans_meet(qw[i], pr[j]))
                return 0;
    return 1;
}

/* Events of the runtime shim's pool used while capturing a bound step. */
enum { EV_FORK = 0, EV_Y = 1, EV_JOIN = 2, EV_OP0 = 4 };   /* EV_OP0 + i: op i's upload */

/* Launch the open group (ops [first, end) that joined it).  With bound host
 * buffers the group waits for the uploads of all its ops and every output goes
 * down after the launch. */
static mm_status engine_close_group(mm_lin_engine *e, uint32_t first, uint32_t end, int with_copies, uint32_t grp)
{
    if (mmb_group_size() == 0)
        return mmb_group_launch();
    if (with_copies)
        for (uint32_t k = first / grp; k <= (end - 1) / grp; k++)
            MM_CHECK(mm_event_wait(EV_OP0 + (int)k, MM_ST_COMPUTE));
    MM_CHECK(mmb_group_launch());
    e->n_group_launches++;
    if (with_copies) {
        MM_CHECK(mm_event_record(EV_Y, MM_ST_COMPUTE));
        MM_CHECK(mm_event_wait(EV_Y, MM_ST_XFER));
        /* the group's outputs go down as one kernel per MMB_GATHER_MAX buffers that
         * writes the pinned host buffers itself; what it cannot take uses copy nodes */
        const void *src[MMB_GATHER_MAX];
        void *dst[MMB_GATHER_MAX];
        size_t len[MMB_GATHER_MAX];
        uint32_t pending = 0;
        for (uint32_t i = first; i <= end; i++) {
            const mm_op_desc *op = i < end ? &e->ops[i] : NULL;
            if (op && e->y_bound[i] && op->op != OP_NOP) {
                src[pending] = op->c;
                dst[pending] = e->y_bound[i];
                len[pending] = op_out_bytes(op);
                pending++;
            }
            if (pending == MMB_GATHER_MAX || (i == end && pending)) {
                int rc = e->upload_kernel
                             ? mmb_launch_host_scatter(src, dst, len, pending, mm_cuda_stream_raw(MM_ST_XFER))
                             : -1;
                if (rc > 0) {
                    MM_LOGE("engine: download kernel launch failed (cuda error %d)", rc);
                    return MM_ERR_CUDA;
                }
                if (rc < 0)
                    for (uint32_t j = 0; j < pending; j++)
                        MM_CHECK(mm_d2h_async(dst[j], src[j], len[j], MM_ST_XFER));
                pending = 0;
            }
        }
    }
    return MM_OK;
}

static mm_status run_ops(mm_lin_engine *e)
{
    /* Bound host buffers, while capturing: the copies ride on the transfer stream
     * as nodes of the same graph.  All uploads are enqueued first, none of them
     * depending on a kernel, so the first op of a group only waits for the
     * activations of its group and the copy engine works ahead of the kernels; each download follows its kernel
     * and overlaps the next ones. */
    const int with_copies = e->bound && mm_cuda_capturing();
    const uint32_t grp = e->upload_group;
    if (with_copies) {
        MM_CHECK(mmb_event_pool_reserve((int)(e->n_ops / grp) + 1 + EV_OP0));
        MM_CHECK(mm_event_record(EV_FORK, MM_ST_COMPUTE));
        MM_CHECK(mm_event_wait(EV_FORK, MM_ST_XFER));
        /* a group's uploads go up as one kernel that reads the pinned buffers over
         * PCIe (kernels/host_gather.cu); buffers it cannot take, and groups larger
         * than one launch holds, use copy nodes */
        const void *src[MMB_GATHER_MAX];
        void *dst[MMB_GATHER_MAX];
        size_t len[MMB_GATHER_MAX];
        uint32_t pending = 0, first = 0;
        for (uint32_t i = 0; i < e->n_ops; i++) {
            const mm_op_desc *op = &e->ops[i];
            if (e->x_bound[i] && op->op != OP_NOP) {
                if (pending == 0)
                    first = i;
                if (pending < MMB_GATHER_MAX) {
                    src[pending] = e->x_bound[i];
                    dst[pending] = (void *)(uintptr_t)op->a;
                    len[pending] = op_in_bytes(op);
                }
                pending++;
            }
            /* one event per group of ops, after the group's last upload */
            if (i % grp == grp - 1 || i + 1 == e->n_ops) {
                int rc = pending && pending <= MMB_GATHER_MAX && e->upload_kernel
                             ? mmb_launch_host_gather(src, dst, len, pending, mm_cuda_stream_raw(MM_ST_XFER))
                             : -1;
                if (rc > 0) {
                    MM_LOGE("engine: upload kernel launch failed (cuda error %d)", rc);
                    return MM_ERR_CUDA;
                }
                if (rc < 0)
                    for (uint32_t j = first; pending && j <= i; j++)
                        if (e->x_bound[j] && e->ops[j].op != OP_NOP)
                            MM_CHECK(mm_h2d_async((void *)(uintptr_t)e->ops[j].a, e->x_bound[j],
                                                  op_in_bytes(&e->ops[j]), MM_ST_XFER));
                pending = 0;
                MM_CHECK(mm_event_record(EV_OP0 + (int)(i / grp), MM_ST_XFER));
            }
        }
    }
    /* Block-scaled decode path, overlap mode: activations that no earlier op of the
     * list writes (inputs of the step; the same tensor read by several ops) are
     * turned into digit planes once, on the transfer stream ahead of the ops, into
     * the plane cache.  The ops that read them launch no slicing kernel of their
     * own, wait only for that event, and may run ahead of their predecessors like
     * any op whose inputs are ready. */
    enum { MAX_PLANE_SLOTS = 64 };
    struct { const void *x; uint32_t M, K; void *ws; } slot[MAX_PLANE_SLOTS];
    uint32_t n_slots = 0;
    const int ev_x0 = EV_OP0 + (int)(e->n_ops / grp) + 1;
    for (uint32_t i = 0; i < e->n_ops; i++) {
        e->planes[i] = NULL;
        e->plane_ev[i] = -1;
    }
    if (e->overlap && !(e->group && mmb_ws_regions() > 1)) {
        size_t cap = 0, used = 0;
        unsigned char *cache = (unsigned char *)mmb_plane_cache(&cap);
        for (uint32_t i = 0; cache && i < e->n_ops; i++) {
            const mm_op_desc *op = &e->ops[i];
            if (op->op == OP_NOP || op->op == OP_SILU_MUL || op->op == OP_ADD_RMSNORM)
                continue;
            mm_f4_plan plan;
            MM_CHECK(mmb_plan_for_op(op, op->op == MMB_OP_GATE_UP, &plan));
            if (plan.variant != MM_F4_V_MX)
                continue;
            int external = 1;
            const span xs = mk_span(op->a, op_in_bytes(op));
            for (uint32_t j = 0; external && j < i; j++) {
                span r[2], w[2];
                if (e->ops[j].op == OP_NOP)
                    continue;
                op_spans(e, &e->ops[j], r, w);
                if (spans_meet(w[0], xs) || spans_meet(w[1], xs))
                    external = 0;
            }
            if (!external)
                continue;
            uint32_t k = 0;
            while (k < n_slots && !(slot[k].x == op->a && slot[k].M == op->n0 && slot[k].K == op->n1))
                k++;
            if (k == n_slots) {
                const size_t need = (mm_f4_xslice_bytes(op->n0, op->n1) + 1023u) & ~(size_t)1023u;
                if (n_slots == MAX_PLANE_SLOTS || need == 0 || used + need > cap)
                    continue;                     /* no room: the op slices for itself */
                slot[k].x = op->a; slot[k].M = op->n0; slot[k].K = op->n1;
                slot[k].ws = cache + used;
                used += need;
                n_slots++;
            }
            e->planes[i] = slot[k].ws;
            e->plane_ev[i] = ev_x0 + (int)k;
        }
    }
    e->n_plane_slots = n_slots;
    if (n_slots) {
        MM_CHECK(mmb_event_pool_reserve(ev_x0 + (int)n_slots));
        if (!with_copies) {
            MM_CHECK(mm_event_record(EV_FORK, MM_ST_COMPUTE));
            MM_CHECK(mm_event_wait(EV_FORK, MM_ST_XFER));
        }
        for (uint32_t k = 0; k < n_slots; k++) {
            MM_CHECK(mm_f4_xslice(slot[k].x, slot[k].M, slot[k].K, slot[k].ws,
                                  mm_f4_xslice_bytes(slot[k].M, slot[k].K), mm_cuda_stream_raw(MM_ST_XFER)));
            MM_CHECK(mm_event_record(ev_x0 + (int)k, MM_ST_XFER));
        }
        for (uint32_t i = 0; i < e->n_ops; i++) {                /* only a tensor's first reader waits */
            if (e->plane_ev[i] < 0)
                continue;
            int first = 1;
            for (uint32_t j = 0; j < i; j++)
                if (e->plane_ev[j] == e->plane_ev[i] || (e->planes[j] == e->planes[i] && e->planes[j]))
                    first = 0;
            if (!first)
                e->plane_ev[i] = -1;
        }
    }
    mm_kcall kc;
    kc.e = (const mm_engine *)e;      /* the dispatcher only tests it for NULL */
    kc.stream = NULL;
    uint32_t first_in_flight = 0;     /* the last op that waited for its predecessor */
    unsigned regions_in_flight = 0;   /* workspace regions used since then */
    int next_region = 0;
    const int n_regions = e->overlap ? mmb_ws_regions() : 1;
    e->n_independent = 0;
    int prev_mx = -1;                 /* index of the op in front when it made digit planes, else -1 */
    uint32_t group_first = 0;         /* first op of the open group */
    int group_open = 0, group_region = 0;
    e->n_group_launches = 0;
    for (uint32_t i = 0; i < e->n_ops; i++) {
        const mm_op_desc *op = &e->ops[i];
        const int linear = op->op != OP_NOP && op->op != OP_SILU_MUL && op->op != OP_ADD_RMSNORM;
        if (e->group && mmb_ws_regions() > 1) {
            /* Group mode: an op joins the open group when it runs on the block-scaled
             * kernel and shares no memory with the group's ops; anything else closes
             * the group (one persistent launch for all its ops) first. */
            int joined = 0;
            if (linear) {
                int indep = 1;
                for (uint32_t j = group_first; group_open && indep && j < i; j++)
                    if (e->ops[j].op != OP_NOP && !ops_independent(e, op, &e->ops[j]))
                        indep = 0;
                for (int attempt = 0; attempt < 2 && !joined; attempt++) {
                    if (!group_open) {
                        MM_CHECK(mmb_group_begin(MMB_PDL_WAIT_FIRST, group_region));
                        group_region = (group_region + 1) % mmb_ws_regions();
                        group_open = 1;
                        group_first = i;
                        indep = 1;
                    }
                    mm_status gs = !indep ? MM_ERR_CAPACITY
                                   : e->tp[i].n ? mmb_group_add_tp(op, e->tp[i].y, e->tp[i].n, e->tp[i].ldy, e->tp[i].col0)
                                                : mmb_group_add(op, op->op == MMB_OP_GATE_UP, e->up[i].payload,
                                                                e->up[i].scale);
                    if (gs == MM_OK) {
                        joined = 1;
                    } else if (gs == MM_ERR_CAPACITY && mmb_group_size() > 0) {
                        MM_CHECK(engine_close_group(e, group_first, i, with_copies, grp));
                        group_open = 0;
                    } else if (gs == MM_ERR_UNSUPPORTED || gs == MM_ERR_CAPACITY) {
                        break;                      /* not a block-scaled op: dispatched on its own below */
                    } else {
                        return gs;
                    }
                }
            }
            if (joined) {
                if (i > group_first)
                    e->n_independent++;
                /* with bound host buffers a launch ends where an upload group ends: its
                 * outputs go down, and the next launch's activations come up, while the
                 * neighbouring launch computes */
                if (i + 1 == e->n_ops || (with_copies && (i + 1) % grp == 0)) {
                    MM_CHECK(engine_close_group(e, group_first, i + 1, with_copies, grp));
                    group_open = 0;
                }
                continue;
            }
            if (group_open && op->op != OP_NOP) {
                MM_CHECK(engine_close_group(e, group_first, i, with_copies, grp));
                group_open = 0;
            }
        }
        mm_f4_plan plan;
        int share = 0;
        if (linear) {
            MM_CHECK(mmb_plan_for_op(op, op->op == MMB_OP_GATE_UP, &plan));
            /* block-scaled decode path: an op that reads the activations the op in
             * front already turned into digit planes takes those planes (q, k and v;
             * gate and up), unless that op wrote into them */
            if (plan.variant == MM_F4_V_MX && prev_mx >= 0) {
                const mm_op_desc *q = &e->ops[prev_mx];
                span qr[2], qw[2];
                op_spans(e, q, qr, qw);
                share = q->a == op->a && q->n0 == op->n0 && q->n1 == op->n1 &&
                        !spans_meet(qw[0], mk_span(op->a, op_in_bytes(op)));
            }
            prev_mx = plan.variant == MM_F4_V_MX ? (int)i : -1;
        } else if (op->op != OP_NOP) {
            prev_mx = -1;
        }
        if (e->overlap && op->op != OP_NOP) {
            int independent = 0, region = 0, scratch = 0;
            if (linear) {
                /* split-K partials and digit planes live in the op's workspace region */
                scratch = plan.split_k > 1 || plan.variant == MM_F4_V_MX;
                region = scratch ? next_region : 0;
                independent = i > 0 && (plan.variant == MM_F4_V_STREAM ||
                                        (plan.variant == MM_F4_V_MX && (share || e->planes[i]))) &&
                              !(scratch && (regions_in_flight & (1u << region)));
                for (uint32_t j = first_in_flight; independent && j < i; j++)
                    if (e->ops[j].op != OP_NOP && !ops_independent(e, op, &e->ops[j]))
                        independent = 0;
            }
            if (!independent) {
                first_in_flight = i;
                regions_in_flight = 0;
            }
            if (scratch) {
                regions_in_flight |= 1u << region;
                next_region = (region + 1) % n_regions;
            }
            e->n_independent += (uint32_t)independent;
            mmb_next_op_context(independent ? MMB_PDL_INDEPENDENT : MMB_PDL_WAIT_FIRST, region,
                                e->overlap > 1, share);
        } else if (linear) {
            mmb_next_op_context(-1, 0, 0, share);
        }
        /* the first op of a group waits for the uploads of the whole group */
        if (with_copies && i % grp == 0)
            MM_CHECK(mm_event_wait(EV_OP0 + (int)(i / grp), MM_ST_COMPUTE));
        if (e->planes[i]) {
            if (e->plane_ev[i] >= 0)
                MM_CHECK(mm_event_wait(e->plane_ev[i], MM_ST_COMPUTE));
            mmb_next_op_planes(e->planes[i]);
        }
        kc.op = &e->ops[i];
        mm_status st = e->ops[i].op == MMB_OP_GATE_UP
                           ? mmb_op_mlp_gate_up(&e->ops[i], e->up[i].payload, e->up[i].scale)
                       : e->tp[i].n ? mmb_op_linear_tp(&e->ops[i], e->tp[i].y, e->tp[i].n, e->tp[i].ldy, e->tp[i].col0)
                                    : mm_kx_invoke(&kc);
        if (st != MM_OK) {
            MM_LOGE("engine: op %u (%s) failed: %s", i, e->ops[i].note, mm_status_str(st));
            return st;
        }
        if (with_copies && e->y_bound[i] && op->op != OP_NOP) {
            MM_CHECK(mm_event_record(EV_Y, MM_ST_COMPUTE));
            MM_CHECK(mm_event_wait(EV_Y, MM_ST_XFER));
            MM_CHECK(mm_d2h_async(e->y_bound[i], op->c, op_out_bytes(op), MM_ST_XFER));
        }
    }
    if (group_open)
        MM_CHECK(engine_close_group(e, group_first, e->n_ops, with_copies, grp));
    if (with_copies || n_slots) {
        MM_CHECK(mm_event_record(EV_JOIN, MM_ST_XFER));
        MM_CHECK(mm_event_wait(EV_JOIN, MM_ST_COMPUTE));
    }
    return MM_OK;
}

mm_status mm_lin_engine_capture(mm_lin_engine *e)
{
    MM_REQUIRE(e && e->n_ops > 0, MM_ERR_STATE);
    if (!e->graph)
        MM_CHECK(mm_graph_create(&e->graph));
    MM_CHECK(mm_graph_capture_begin(e->graph));
    mm_status st = run_ops(e);
    mm_status st2 = mm_graph_commit(e->graph, NULL, 0, 0);   /* always ends the capture */
    if (st != MM_OK)
        return st;
    if (st2 != MM_OK)
        return st2;
    e->captured = 1;
    e->bound_captured = e->bound;
    return MM_OK;
}

static mm_status step_status(void)
{
    unsigned flags = 0;
    MM_CHECK(mm_f4_device_status(&flags));
    if (flags) {
        MM_LOGE("engine: device status 0x%x after step", flags);
        return (flags & 1u) ? MM_ERR_TIMEOUT : MM_ERR_CUDA;
    }
    return MM_OK;
}

mm_status mm_lin_engine_step_bound(mm_lin_engine *e)
{
    MM_REQUIRE(e && e->n_ops > 0 && e->captured && e->bound_captured, MM_ERR_STATE);
    MM_REQUIRE(!mm_cuda_capturing(), MM_ERR_BUSY);
    MM_CHECK(mm_graph_launch(e->graph, MM_ST_COMPUTE));
    MM_CHECK(mm_stream_sync(MM_ST_COMPUTE));
    return step_status();
}

mm_status mm_lin_engine_launch(mm_lin_engine *e)
{
    MM_REQUIRE(e && e->n_ops > 0, MM_ERR_STATE);
    if (e->captured)
        return mm_graph_launch(e->graph, MM_ST_COMPUTE);
    return run_ops(e);
}

mm_status mm_lin_engine_launch_host(mm_lin_engine *e, const void *const *x_host,
                                    void *const *y_host)
{
    MM_REQUIRE(e && e->n_ops > 0, MM_ERR_STATE);
    MM_REQUIRE(!mm_cuda_capturing(), MM_ERR_BUSY);
    MM_REQUIRE(!(e->captured && e->bound_captured), MM_ERR_BUSY);   /* that graph already copies */
    for (uint32_t i = 0; y_host && i < e->n_ops; i++)
        if (e->tp[i].n && y_host[i])
            return MM_ERR_UNSUPPORTED;                                 /* a column slice of a wider buffer */
    for (uint32_t i = 0; x_host && i < e->n_ops; i++) {
        const mm_op_desc *op = &e->ops[i];
        if (x_host[i] && op->op != OP_NOP)
            MM_CHECK(mm_h2d_async((void *)(uintptr_t)op->a, x_host[i], op_in_bytes(op), MM_ST_COMPUTE));
    }
    if (e->captured)
        MM_CHECK(mm_graph_launch(e->graph, MM_ST_COMPUTE));
    else
        MM_CHECK(run_ops(e));
    for (uint32_t i = 0; y_host && i < e->n_ops; i++) {
        const mm_op_desc *op = &e->ops[i];
        if (y_host[i] && op->op != OP_NOP)
            MM_CHECK(mm_d2h_async(y_host[i], op->c, op_out_bytes(op), MM_ST_COMPUTE));
    }
    MM_CHECK(mm_stream_sync(MM_ST_COMPUTE));
    return step_status();
}

void mm_lin_engine_destroy(mm_lin_engine *e)
{
    if (!e)
        return;
    mm_graph_destroy(e->graph);
    free(e->ops);
    free(e->up);
    free(e->tp);
    free(e->x_bound);
    free(e->y_bound);
    free(e->planes);
    free(e->plane_ev);
    free(e);
}
