/*
 * The launcher: mimfer's operator ABI on one side, the sm_100a kernels on the
 * other.  Thin on purpose: validate, pick a plan (csrc/plan/select.c), encode
 * the TMA descriptors, launch.  No device allocation happens here
 * (reference rule: include/mimfer/alloc.h:4-29); split-K scratch is donated by
 * the caller through mm_f4_workspace_set.
 *
 * kx_op_gemm_f4 replaces src/kernels/cuda/cx.cu:358-376; its error and
 * synchronisation behaviour follows kx_sync (cx.cu:83-100): synchronise the
 * compute stream and surface errors per op, except while a graph is being
 * captured.
 */
#include "../core/core.h"
#include "../kernels/launch.h"
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int mmb_stream_init(void);
int mmb_umma_init(void);
int mmb_mx_init(void);
int mmb_mxg_init(void);

/* ------------------------------------------------------------------ state */
typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                              const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static struct {
    int        ready;
    void      *ready_stream;     /* compute stream the set-up below was made for */
    int        sm_count;
    encode_fn  encode;
    unsigned  *status_dev;
    unsigned  *status_host;      /* pinned */
    void      *ws;
    size_t     ws_bytes;
    int        forced_variant;
    int        pdl;
    int        next_pdl;         /* per-op override from the engine, -1 = none */
    int        next_region;
    int        next_shallow;     /* the next op may take the shallower K split of a run-ahead op */
    int        next_share_x;     /* the next op reads the activations the op before it sliced */
    void      *next_planes;      /* the next op's digit planes are already there (plane cache) */
    int        use_mx;           /* decode ops take the block-scaled tensor path when they can */
    uint32_t   mx_stages;        /* cap on the pipeline depth of a group launch (0 = what fits) */
    int        l2_window;        /* group launches carry a persisting L2 window over the workspace */
    int        l2_limit_set;
    int        no_tail_split;    /* prefill tiles of the last wave run whole */
    int        group_sort;       /* ops of a group launch ordered by activation rows, most first */
    int        static_units;     /* group launch: unit u on CTA u mod grid instead of handed out as CTAs ask */
    /* the digit planes made last: which activations, and where they lie */
    const void *sliced_x;
    uint32_t   sliced_M, sliced_K;
    void      *sliced_ws;
    unsigned long long launches;
    uint32_t tp_stagger;    /* mm_f4_tune key 12: spread of the first wave of a tensor-parallel prefill launch, percent of a wave's NVLink time */
    uint32_t tp_lanes;      /* mm_f4_tune key 11: copy streams per peer of mm_f4_tp_push, 0 = by the number of peers */
    /* experiment knobs (mm_f4_tune keys 2..4), all 0 in production */
    uint32_t   st_rows, st_split, st_dbg;
} G = { .forced_variant = -1, .pdl = 1, .next_pdl = -1, .use_mx = 1, .group_sort = 1, .tp_stagger = 100 };

/* The workspace is cut into WS_REGIONS equal regions, each with its own arrival
 * counters, when every region still holds WS_REGION_MIN bytes; an op uses one
 * region (0 unless the engine says otherwise). */
#define WS_REGIONS    4
#define WS_REGION_MIN ((size_t)4 << 20)

int mmb_ws_regions(void)
{
    return G.ws && G.ws_bytes / (2 * WS_REGIONS) >= WS_REGION_MIN ? WS_REGIONS : 1;
}

/* With room to divide, the lower half of the workspace holds the per-op regions
 * and the upper half is the plane cache: digit planes of activations that are
 * made once per step, ahead of the ops that read them (engine, overlap mode). */
static size_t ws_region_bytes(void)
{
    if (!G.ws)
        return 0;
    const int n = mmb_ws_regions();
    return (n > 1 ? G.ws_bytes / (size_t)(2 * n) : G.ws_bytes) & ~(size_t)1023;
}

void *mmb_plane_cache(size_t *bytes_out)
{
    const int n = mmb_ws_regions();
    if (n <= 1) {
        *bytes_out = 0;
        return NULL;
    }
    const size_t lower = (size_t)n * ws_region_bytes();
    *bytes_out = (G.ws_bytes - lower) & ~(size_t)1023;
    return (unsigned char *)G.ws + lower;
}

void mmb_next_op_context(int pdl_mode, int ws_region, int shallow_split, int share_x)
{
    G.next_pdl = pdl_mode;
    G.next_shallow = shallow_split && pdl_mode == MMB_PDL_INDEPENDENT;
    G.next_region = ws_region >= 0 && ws_region < mmb_ws_regions() ? ws_region : 0;
    G.next_share_x = share_x;
}

void mmb_next_op_planes(void *planes_ws) { G.next_planes = planes_ws; }

/* Consume the per-op context: launch mode and workspace base of this op. */
static void take_op_context(int *pdl_out, void **ws_out, int *shallow_out, int *share_out)
{
    *shallow_out = G.next_shallow;
    G.next_shallow = 0;
    *share_out = G.next_share_x;
    G.next_share_x = 0;
    int mode = G.next_pdl >= 0 ? G.next_pdl : MMB_PDL_TRIGGER_FIRST;
    *pdl_out = G.pdl ? mode : MMB_PDL_OFF;
    *ws_out = G.ws ? (unsigned char *)G.ws + (size_t)G.next_region * ws_region_bytes() : NULL;
    G.next_pdl = -1;
    G.next_region = 0;
}

/* global-scale registry: open addressing on the scale base pointer, with
 * tombstones so that an entry can be taken back (a failed staging run) */
#define GS_SLOTS 8192u                   /* more than the weights loader admits tensors (4096) */
#define GS_TOMB  ((const void *)(uintptr_t)1)
static struct { const void *key; float gs; } g_gs[GS_SLOTS];
static unsigned g_gs_used;               /* live entries + tombstones */

static unsigned gs_hash(const void *p)
{
    uint64_t v = (uint64_t)(uintptr_t)p;
    v ^= v >> 33; v *= 0xff51afd7ed558ccdull; v ^= v >> 29;
    return (unsigned)v & (GS_SLOTS - 1u);
}

mm_status mm_f4_gscale_set(const void *scale_base, float gs)
{
    MM_REQUIRE(scale_base && scale_base != GS_TOMB, MM_ERR_STATE);
    MM_REQUIRE(gs == gs && gs > 0.0f && gs < 3.0e38f, MM_ERR_RANGE);
    unsigned h = gs_hash(scale_base);
    int free_at = -1;
    for (unsigned i = 0; i < GS_SLOTS; i++, h = (h + 1u) & (GS_SLOTS - 1u)) {
        if (g_gs[h].key == scale_base) { g_gs[h].gs = gs; return MM_OK; }
        if (g_gs[h].key == GS_TOMB) { if (free_at < 0) free_at = (int)h; continue; }
        if (!g_gs[h].key) {
            if (free_at < 0) {
                if (g_gs_used + 1u >= GS_SLOTS) return MM_ERR_CAPACITY;
                free_at = (int)h;
                g_gs_used++;
            }
            break;
        }
    }
    if (free_at < 0)
        return MM_ERR_CAPACITY;
    g_gs[free_at].key = scale_base;
    g_gs[free_at].gs = gs;
    return MM_OK;
}

float mm_f4_gscale_get(const void *scale_base)
{
    unsigned h = gs_hash(scale_base);
    for (unsigned i = 0; i < GS_SLOTS; i++, h = (h + 1u) & (GS_SLOTS - 1u)) {
        if (g_gs[h].key == scale_base) return g_gs[h].gs;
        if (!g_gs[h].key) break;
    }
    return 1.0f;
}

void mm_f4_gscale_unset(const void *scale_base)
{
    if (!scale_base || scale_base == GS_TOMB)
        return;
    unsigned h = gs_hash(scale_base);
    for (unsigned i = 0; i < GS_SLOTS; i++, h = (h + 1u) & (GS_SLOTS - 1u)) {
        if (g_gs[h].key == scale_base) { g_gs[h].key = GS_TOMB; return; }
        if (!g_gs[h].key) return;
    }
}

uint32_t mm_f4_gscale_room(void)
{
    return GS_SLOTS - 1u - g_gs_used;
}

void mm_f4_gscale_clear(void)
{
    memset(g_gs, 0, sizeof g_gs);
    g_gs_used = 0;
}

void mm_f4_force_variant(int variant) { G.forced_variant = variant; }

int mm_f4_tune(int key, int value)
{
    if (key == 1) {
        int old = G.pdl;
        G.pdl = value ? 1 : 0;
        return old;
    }
    if (key == 2) { int old = (int)G.st_rows; G.st_rows = (uint32_t)value; return old; }
    if (key == 3) { int old = (int)G.st_split; G.st_split = (uint32_t)value; return old; }
#ifdef MMB_MEASURE_MODES
    if (key == 4) { int old = (int)G.st_dbg; G.st_dbg = (uint32_t)value; return old; }
#endif
    if (key == 5) { int old = G.use_mx; G.use_mx = value ? 1 : 0; return old; }
    if (key == 6) { int old = (int)G.mx_stages; G.mx_stages = (uint32_t)value; return old; }
    if (key == 7) { int old = G.l2_window; G.l2_window = value ? 1 : 0; return old; }
    if (key == 10) { int old = !G.static_units; G.static_units = value ? 0 : 1; return old; }
    if (key == 12) { int old = (int)G.tp_stagger; G.tp_stagger = value > 0 ? (uint32_t)(value > 400 ? 400 : value) : 0u; return old; }
    if (key == 11) { int old = (int)G.tp_lanes; G.tp_lanes = value > 0 ? (uint32_t)value : 0u; return old; }
    if (key == 9) { int old = G.group_sort; G.group_sort = value ? 1 : 0; return old; }
    if (key == 8) { int old = !G.no_tail_split; G.no_tail_split = value ? 0 : 1; return old; }
    return -1;
}

unsigned long long mm_f4_launch_count(int reset)
{
    unsigned long long n = G.launches;
    if (reset) G.launches = 0;
    return n;
}

/* ------------------------------------------------------------------ setup */
#define CK(call)                                                              \
    do {                                                                      \
        cudaError_t e_ = (call);                                              \
        if (e_ != cudaSuccess) {                                              \
            MM_LOGE("cuda: %s: %s", #call, cudaGetErrorString(e_));           \
            return MM_ERR_CUDA;                                               \
        }                                                                     \
    } while (0)

/* The exchange of a tensor-parallel linear by the copy engines.  A prefill-size output
 * slice is hundreds of megabytes per rank: stored from the kernel's epilogue it holds the
 * SM until NVLink has taken it; pushed by the copy engines it leaves while the next row
 * chunk is multiplied.  Side streams with an event each, up to TP_LANES per peer, made
 * on first use. */
#define TP_LANES 8u                     /* copy streams per peer at most */
static struct {
    cudaStream_t side[MMB_MAX_PEERS][TP_LANES];
    cudaEvent_t  done[MMB_MAX_PEERS][TP_LANES], ready;
    uint8_t      made[MMB_MAX_PEERS][TP_LANES], pending[MMB_MAX_PEERS][TP_LANES];
} TP;

static void tp_push_reset(void)
{
    for (uint32_t d = 0; d < MMB_MAX_PEERS; d++)
        for (uint32_t l = 0; l < TP_LANES; l++)
            if (TP.made[d][l]) {
                cudaStreamDestroy(TP.side[d][l]);
                cudaEventDestroy(TP.done[d][l]);
            }
    if (TP.ready)
        cudaEventDestroy(TP.ready);
    memset(&TP, 0, sizeof TP);
}

/* Forget everything that belongs to the device the runtime was initialised on:
 * status word, workspace, per-device kernel attributes, the side streams of the
 * tensor-parallel pushes.  Called by the runtime
 * shim's mm_cuda_shutdown, and by ensure_ready when it finds the runtime on
 * another compute stream than the one it prepared for (a shutdown followed by
 * a new mm_cuda_init, possibly on another device, in a runtime that is not the
 * shim). */
void mmb_launcher_reset(void)
{
    if (G.status_host)
        cudaFreeHost(G.status_host);
    G.status_host = NULL;
    G.status_dev = NULL;
    G.ws = NULL;
    G.ws_bytes = 0;
    G.sliced_x = NULL;
    G.sliced_ws = NULL;
    G.ready = 0;
    G.ready_stream = NULL;
    G.next_pdl = -1;
    G.next_region = 0;
    G.next_shallow = 0;
    G.l2_limit_set = 0;
    tp_push_reset();
}

static mm_status ensure_ready(void)
{
    void *cs = mm_cuda_stream_raw(MM_ST_COMPUTE);
    if (G.ready && cs == G.ready_stream)
        return MM_OK;
    if (G.ready)
        mmb_launcher_reset();
    MM_REQUIRE(cs != NULL, MM_ERR_STATE);   /* mm_cuda_init first */
    int dev = 0;
    CK(cudaGetDevice(&dev));
    CK(cudaDeviceGetAttribute(&G.sm_count, cudaDevAttrMultiProcessorCount, dev));
    int major = 0;
    CK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    MM_REQUIRE(major == 10, MM_ERR_DEVICE);
    void *fn = NULL;
    enum cudaDriverEntryPointQueryResult qr;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
    MM_REQUIRE(fn && qr == cudaDriverEntryPointSuccess, MM_ERR_CUDA);
    G.encode = (encode_fn)fn;
    CK((cudaError_t)mmb_stream_init());
    CK((cudaError_t)mmb_umma_init());
    CK((cudaError_t)mmb_mx_init());
    CK((cudaError_t)mmb_mxg_init());
    CK((cudaError_t)mmb_status_word(&G.status_dev));
    CK(cudaHostAlloc((void **)&G.status_host, 64, cudaHostAllocDefault));
    *G.status_host = 0;
    CK(cudaMemsetAsync(G.status_dev, 0, sizeof(unsigned), (cudaStream_t)cs));
    G.ready = 1;
    G.ready_stream = cs;
    return MM_OK;
}

mm_status mm_f4_workspace_set(void *dev_ptr, size_t bytes)
{
    MM_CHECK(ensure_ready());
    G.sliced_x = NULL;
    G.sliced_ws = NULL;
    if (!dev_ptr || bytes <= MMB_WS_COUNTER_B) {
        G.ws = NULL;
        G.ws_bytes = 0;
        return dev_ptr ? MM_ERR_RANGE : MM_OK;
    }
    MM_REQUIRE(((uintptr_t)dev_ptr & 255u) == 0, MM_ERR_SHAPE);
    G.ws = dev_ptr;
    G.ws_bytes = bytes;
    /* the arrival counters at the head of every region start at zero (kernels
     * leave them at zero again) */
    for (int r = 0; r < mmb_ws_regions(); r++)
        CK(cudaMemsetAsync((unsigned char *)dev_ptr + (size_t)r * ws_region_bytes(), 0, MMB_WS_COUNTER_B,
                           (cudaStream_t)mm_cuda_stream_raw(MM_ST_COMPUTE)));
    return MM_OK;
}

size_t mm_f4_workspace_bytes(void) { return G.ws_bytes; }

/* ------------------------------------------------------ TMA descriptors */
static mm_status encode_2d(unsigned char out[128], CUtensorMapDataType dt, unsigned esize,
                           const void *base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                           uint32_t box_outer, CUtensorMapSwizzle sw)
{
    CUtensorMap map;
    cuuint64_t dims[2] = { inner, outer };
    cuuint64_t strides[1] = { inner * esize };
    cuuint32_t box[2] = { box_inner, box_outer };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = G.encode(&map, dt, 2, (void *)(uintptr_t)base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        MM_LOGE("cuTensorMapEncodeTiled failed: %d (inner %llu outer %llu box %u x %u)", (int)r,
                (unsigned long long)inner, (unsigned long long)outer, box_inner, box_outer);
        return MM_ERR_CUDA;
    }
    memcpy(out, &map, 128);
    return MM_OK;
}

/* Two equal 2-D tensors `plane_stride` bytes apart as one 3-D map; a box takes
 * box_outer rows of each. */
static mm_status encode_pair(unsigned char out[128], const void *base, uint64_t inner, uint64_t outer,
                             uint64_t plane_stride, uint32_t box_inner, uint32_t box_outer,
                             CUtensorMapSwizzle sw)
{
    CUtensorMap map;
    cuuint64_t dims[3] = { inner, outer, 2 };
    cuuint64_t strides[2] = { inner, plane_stride };
    cuuint32_t box[3] = { box_inner, box_outer, 2 };
    cuuint32_t estr[3] = { 1, 1, 1 };
    CUresult r = G.encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)(uintptr_t)base, dims, strides,
                          box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        MM_LOGE("cuTensorMapEncodeTiled (pair) failed: %d (inner %llu outer %llu stride %llu)", (int)r,
                (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)plane_stride);
        return MM_ERR_CUDA;
    }
    memcpy(out, &map, 128);
    return MM_OK;
}

/* ------------------------------------------------------------------ launch */
static uint32_t min_align(const void *a, const void *b, const void *c, const void *d)
{
    uintptr_t v = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d | 256u;
    return (uint32_t)(v & (~v + 1u));
}

/* Plan of a linear op as the launcher runs it (shared with mmb_plan_for_op). */
static mm_status plan_linear(const void *x, const void *payload, const void *scale, const void *y,
                             uint32_t n_dst, uint32_t ldy, uint32_t col0, uint32_t M, uint32_t K,
                             uint32_t N, int run_ahead, mm_f4_plan *plan)
{
    mm_f4_shape sh = { M, K, N, (uint32_t)G.sm_count, min_align(x, payload, scale, y), ws_region_bytes() };
    if (sh.ptr_align < 16)
        return MM_ERR_SHAPE;               /* arena slots are >= 16-byte aligned; every kernel loads 16-byte vectors */
    if (n_dst && (col0 % 8u != 0 || ldy % 8u != 0))
        sh.ptr_align = 8;                  /* aligned operands, unaligned output slice: the row-warp kernel */
    mm_status st = G.forced_variant >= 0 ? mm_f4_select_variant(&sh, G.forced_variant, plan)
                                         : mm_f4_select(&sh, plan);
    if (st == MM_OK && plan->variant == MM_F4_V_MX && G.forced_variant < 0 && !G.use_mx)
        st = mm_f4_select_variant(&sh, MM_F4_V_STREAM, plan);     /* tuning key 5 = 0: the CUDA-core kernel */
    if (st == MM_OK && plan->variant == MM_F4_V_UMMA && G.no_tail_split) {
        plan->split_k = 1;
        plan->m_tiles = 0;
        plan->ws_needed = 0;
    }
    if (st == MM_OK && plan->variant == MM_F4_V_STREAM && (G.st_rows || G.st_split))
        return mmb_plan_stream_with(&sh, G.st_rows, G.st_split, plan);
    if (st == MM_OK && plan->variant == MM_F4_V_MX && (G.st_rows || G.st_split))
        return mmb_plan_mx_with(&sh, G.st_rows, G.st_split, plan);
    /* An op that runs ahead of its predecessors shares the GPU with them: it is
     * served best by fewer, longer K slices on about half of the SMs (less
     * exchange, the fill paid once per more steps) - the other half is busy with
     * the ops around it.  An op that has the GPU to itself keeps the deepest
     * split.  Measured on B200, us per op, run-ahead / alone: down at M = 16 with
     * 3 slices 17.0 / 31.9, with 7 slices 19.9 / 21.4; q with 3 slices 8.2 / 13.8,
     * with 5 slices 9.9 / 12.9. */
    if (st == MM_OK && run_ahead && plan->variant == MM_F4_V_STREAM && plan->split_k > 1 &&
        plan->grid_x <= 24) {              /* measured for 17 to 24 row tiles; a fused qkv (32) lost with 2 slices */
        uint32_t s = (uint32_t)(0.45 * (double)sh.sm_count / (double)plan->grid_x + 0.5);
        if (s < 1) s = 1;
        if (s < plan->split_k)
            st = mmb_plan_stream_with(&sh, plan->tile_n, s, plan);
    }
    return st;
}

/* The two launches of an op on the block-scaled tensor path: the activations'
 * digit planes into the op's scratch (skipped when the op in front sliced the
 * same activations and they are still there), then the linear kernel.  The
 * weight maps of `a` are encoded by the caller. */
static mm_status launch_mx_pair(mmb_args *a, int share_x, void *stream)
{
    const uint32_t nb = a->plan.tile_m;
    void *cached = G.next_planes;
    G.next_planes = NULL;
    const int reuse = cached != NULL ||
                      (share_x && G.sliced_ws && G.sliced_x == a->x && G.sliced_M == a->M && G.sliced_K == a->K);
    a->mx_x_ws = cached ? cached : reuse ? G.sliced_ws : (void *)((unsigned char *)a->ws + MMB_WS_COUNTER_B);
    a->mx_partial_off = MMB_WS_COUNTER_B + MMB_MX_XS_B(nb, a->K);
    unsigned char *planes = (unsigned char *)a->mx_x_ws + MMB_MX_PLANES_OFF;
    MM_CHECK(encode_2d(a->tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, planes, a->K / 2, nb, 128, nb,
                       CU_TENSOR_MAP_SWIZZLE_128B));
    MM_CHECK(encode_2d(a->tm_sfb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, planes + MMB_MX_PLANES_B(nb, a->K),
                       a->K / 16, nb, 16, nb, CU_TENSOR_MAP_SWIZZLE_NONE));
    int err;
    if (!reuse) {
        /* an op that slices its own activations waits for its predecessor (they may
         * be its output, and the scratch may still be read) */
        if (a->pdl == MMB_PDL_INDEPENDENT)
            a->pdl = MMB_PDL_WAIT_FIRST;
        if ((err = mmb_launch_xslice(a, stream)) != 0) {
            MM_LOGE("cuda: launch (activation slicing, M %u K %u): %s", a->M, a->K,
                    cudaGetErrorString((cudaError_t)err));
            return MM_ERR_CUDA;
        }
        G.launches++;
        G.sliced_x = a->x; G.sliced_M = a->M; G.sliced_K = a->K; G.sliced_ws = a->mx_x_ws;
    }
    if ((err = mmb_launch_mx(a, stream)) != 0) {
        MM_LOGE("cuda: launch (variant %d, M %u K %u N %u): %s", a->plan.variant, a->M, a->K, a->N,
                cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.launches++;
    return MM_OK;
}

static mm_status linear_impl(const void *x, const void *payload, const void *scale, float gs,
                             void *y, void *const *y_dst, uint32_t n_dst, uint32_t ldy,
                             uint32_t col0, uint32_t M, uint32_t K, uint32_t N, void *stream)
{
    MM_REQUIRE(x && payload && scale && y, MM_ERR_STATE);
    if (M == 0 || N == 0 || K == 0 || K % 16 != 0)
        return MM_ERR_SHAPE;               /* e4m3 group scale spans 16 columns */
    if (min_align(x, payload, scale, y) < 16)
        return MM_ERR_SHAPE;               /* refused before anything is launched, in every form of the op */
    MM_CHECK(ensure_ready());
    if (!stream)
        stream = mm_cuda_stream_raw(MM_ST_COMPUTE);

    mmb_args a;
    memset(&a, 0, sizeof a);
    a.x = x; a.payload = payload; a.scale = scale; a.y = y;
    a.gs = gs; a.M = M; a.K = K; a.N = N;
    int shallow = 0, share_x = 0;
    take_op_context(&a.pdl, &a.ws, &shallow, &share_x);
    for (uint32_t d = 0; d < n_dst; d++) a.y_dst[d] = y_dst[d];
    a.n_dst = n_dst; a.ldy = ldy; a.col0 = col0;


    mm_status st = plan_linear(x, payload, scale, y, n_dst, ldy, col0, M, K, N, shallow, &a.plan);
    if (st != MM_OK)
        return st;
    if (n_dst > 1 && a.plan.variant == MM_F4_V_UMMA && G.tp_stagger) {
        /* the time NVLink (about 750 bytes per ns) needs for one wave's tiles to the peers */
        const uint32_t tiles = a.plan.grid_x * a.plan.grid_y;
        const uint32_t ctas = tiles < (uint32_t)G.sm_count ? tiles : (uint32_t)G.sm_count;
        const double wave_b = (double)a.plan.tile_m * (double)a.plan.tile_n * 2.0 * (double)(n_dst - 1u) * (double)ctas;
        double ns = wave_b / 750.0 * (double)G.tp_stagger / 100.0;
        if (ns > 400000.0) ns = 400000.0;
        a.stagger_ns = tiles > ctas ? (uint32_t)ns : 0u;     /* a single wave gains nothing from it */
        a.stagger_ctas = ctas;
    }

    int err = 0;
    switch (a.plan.variant) {
    case MM_F4_V_ROWWARP:
        err = mmb_launch_rowwarp(&a, stream);
        break;
    case MM_F4_V_STREAM:
        MM_CHECK(encode_2d(a.tm_payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, payload, K / 2, N, 128,
                           a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_128B));
        MM_CHECK(encode_2d(a.tm_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, scale, K / 16, N, 16,
                           a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_NONE));
        MM_CHECK(encode_2d(a.tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, K, M, MMB_ST_KSTEP,
                           a.plan.tile_m, CU_TENSOR_MAP_SWIZZLE_NONE));
        a.dbg = G.st_dbg;
        err = mmb_launch_stream(&a, stream);
        break;
    case MM_F4_V_MX:
        MM_CHECK(encode_2d(a.tm_payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, payload, K / 2, N, 128,
                           a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_128B));
        MM_CHECK(encode_2d(a.tm_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, scale, K / 16, N, 16,
                           a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_NONE));
        MM_CHECK(launch_mx_pair(&a, share_x, stream));
        return MM_OK;
    case MM_F4_V_UMMA:
        MM_CHECK(encode_2d(a.tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, K, M, MMB_UM_KBLOCK,
                           a.plan.tile_m, CU_TENSOR_MAP_SWIZZLE_128B));
        MM_CHECK(encode_2d(a.tm_payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, payload, K / 2, N, 32,
                           a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_NONE));
        MM_CHECK(encode_2d(a.tm_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, scale, K / 16, N, 16,
                           a.plan.tile_n, CU_TENSOR_MAP_SWIZZLE_NONE));
        err = mmb_launch_umma(&a, stream);
        if (!err && a.plan.split_k > 1 && a.plan.m_tiles && a.ws)
            G.launches++;                  /* the tail kernel of the split tiles */
        break;
    default:
        return MM_ERR_UNSUPPORTED;
    }
    if (err) {
        MM_LOGE("cuda: launch (variant %d, M %u K %u N %u): %s", a.plan.variant, M, K, N,
                cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.launches++;
    return MM_OK;
}

size_t mm_f4_xslice_bytes(uint32_t M, uint32_t K)
{
    if (M == 0 || M > 32 || K == 0 || K % 256 != 0)
        return 0;
    return MMB_MX_XS_B(((M + 3u) / 4u) * 4u * MMB_MX_PLANES, K);
}

mm_status mm_f4_xslice(const void *x, uint32_t M, uint32_t K, void *scratch, size_t scratch_bytes, void *stream)
{
    MM_REQUIRE(x && scratch, MM_ERR_STATE);
    const size_t need = mm_f4_xslice_bytes(M, K);
    if (!need || ((uintptr_t)x & 15u) || ((uintptr_t)scratch & 255u))
        return MM_ERR_SHAPE;
    MM_REQUIRE(scratch_bytes >= need, MM_ERR_CAPACITY);
    MM_CHECK(ensure_ready());
    if (!stream)
        stream = mm_cuda_stream_raw(MM_ST_COMPUTE);
    mmb_args a;
    memset(&a, 0, sizeof a);
    a.x = x; a.M = M; a.K = K;
    a.plan.tile_m = ((M + 3u) / 4u) * 4u * MMB_MX_PLANES;
    a.mx_x_ws = scratch;
    a.pdl = MMB_PDL_OFF;
    int err = mmb_launch_xslice(&a, stream);
    if (err) {
        MM_LOGE("cuda: launch (activation slicing, M %u K %u): %s", M, K, cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.launches++;
    return MM_OK;
}

mm_status mm_f4_linear(const void *x, const void *payload, const void *scale, float gs, void *y,
                       uint32_t M, uint32_t K, uint32_t N, void *stream)
{
    return linear_impl(x, payload, scale, gs, y, NULL, 0, 0, 0, M, K, N, stream);
}

/* Layout rule of the gated pair: both tensors of the two projections in the
 * same address order, 16-byte-multiple distances below 2^40 (TMA strides). */
static int pair_layout(const void *gate_payload, const void *gate_scale, const void *up_payload,
                       const void *up_scale, int *gate_first, uint64_t *dpay, uint64_t *dsc)
{
    *gate_first = (uintptr_t)gate_payload < (uintptr_t)up_payload;
    if (*gate_first != ((uintptr_t)gate_scale < (uintptr_t)up_scale))
        return 0;
    *dpay = *gate_first ? (uint64_t)((uintptr_t)up_payload - (uintptr_t)gate_payload)
                        : (uint64_t)((uintptr_t)gate_payload - (uintptr_t)up_payload);
    *dsc = *gate_first ? (uint64_t)((uintptr_t)up_scale - (uintptr_t)gate_scale)
                       : (uint64_t)((uintptr_t)gate_scale - (uintptr_t)up_scale);
    return *dpay != 0 && *dsc != 0 && *dpay % 16 == 0 && *dsc % 16 == 0 && *dpay < (1ull << 40) &&
           *dsc < (1ull << 40);
}

int mmb_gate_up_fusable(const void *x, const void *gate_payload, const void *gate_scale,
                        const void *up_payload, const void *up_scale, const void *y,
                        uint32_t M, uint32_t K, uint32_t inter)
{
    int gate_first;
    uint64_t dpay, dsc;
    if (!pair_layout(gate_payload, gate_scale, up_payload, up_scale, &gate_first, &dpay, &dsc))
        return 0;
    mm_f4_plan plan;
    mm_f4_shape sh = { M, K, inter, 148u,
                       min_align(x, gate_first ? gate_payload : up_payload,
                                 gate_first ? gate_scale : up_scale, y), (size_t)1 << 40 };
    return mm_f4_select_glu(&sh, &plan) == MM_OK;
}

mm_status mm_f4_mlp_gate_up(const void *x, const void *gate_payload, const void *gate_scale,
                            float gs_gate, const void *up_payload, const void *up_scale,
                            float gs_up, void *y, uint32_t M, uint32_t K, uint32_t inter,
                            void *stream)
{
    MM_REQUIRE(x && gate_payload && gate_scale && up_payload && up_scale && y, MM_ERR_STATE);
    if (M == 0 || inter == 0 || K == 0 || K % 16 != 0)
        return MM_ERR_SHAPE;
    MM_CHECK(ensure_ready());
    if (!stream)
        stream = mm_cuda_stream_raw(MM_ST_COMPUTE);
    /* plane 0 of the 3-D maps is the lower-addressed projection, in both tensors */
    int gate_first;
    uint64_t dpay, dsc;
    if (!pair_layout(gate_payload, gate_scale, up_payload, up_scale, &gate_first, &dpay, &dsc))
        return MM_ERR_UNSUPPORTED;
    const void *pay0 = gate_first ? gate_payload : up_payload;
    const void *sc0 = gate_first ? gate_scale : up_scale;

    mmb_args a;
    memset(&a, 0, sizeof a);
    a.x = x; a.payload = pay0; a.scale = sc0; a.y = y;
    a.gs = gs_gate; a.gs_up = gs_up;
    a.glu = 1; a.gate_plane = gate_first ? 0 : 1;
    a.M = M; a.K = K; a.N = inter;
    int shallow = 0, share_x = 0;
    take_op_context(&a.pdl, &a.ws, &shallow, &share_x);
    (void)shallow;                         /* the gated pair keeps its split */
    mm_f4_shape sh = { M, K, inter, (uint32_t)G.sm_count, min_align(x, pay0, sc0, y), ws_region_bytes() };
    mm_status st = mmb_select_glu(&sh, G.use_mx, &a.plan);
    if (st != MM_OK)
        return st;
    int err = 0;
    if (a.plan.variant == MM_F4_V_MX) {
        MM_CHECK(encode_pair(a.tm_payload, pay0, K / 2, inter, dpay, 128, a.plan.tile_n / 2,
                             CU_TENSOR_MAP_SWIZZLE_128B));
        MM_CHECK(encode_pair(a.tm_scale, sc0, K / 16, inter, dsc, 16, a.plan.tile_n / 2,
                             CU_TENSOR_MAP_SWIZZLE_NONE));
        return launch_mx_pair(&a, share_x, stream);
    }
    if (a.plan.variant == MM_F4_V_STREAM) {
        MM_CHECK(encode_pair(a.tm_payload, pay0, K / 2, inter, dpay, 128, MMB_ST_ROWS / 2,
                             CU_TENSOR_MAP_SWIZZLE_128B));
        MM_CHECK(encode_pair(a.tm_scale, sc0, K / 16, inter, dsc, 16, MMB_ST_ROWS / 2,
                             CU_TENSOR_MAP_SWIZZLE_NONE));
        MM_CHECK(encode_2d(a.tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, K, M, MMB_ST_KSTEP,
                           a.plan.tile_m, CU_TENSOR_MAP_SWIZZLE_NONE));
        err = mmb_launch_stream(&a, stream);
    } else {
        MM_CHECK(encode_2d(a.tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, K, M, MMB_UM_KBLOCK,
                           a.plan.tile_m, CU_TENSOR_MAP_SWIZZLE_128B));
        MM_CHECK(encode_pair(a.tm_payload, pay0, K / 2, inter, dpay, 32, a.plan.tile_n / 2,
                             CU_TENSOR_MAP_SWIZZLE_NONE));
        MM_CHECK(encode_pair(a.tm_scale, sc0, K / 16, inter, dsc, 16, a.plan.tile_n / 2,
                             CU_TENSOR_MAP_SWIZZLE_NONE));
        err = mmb_launch_umma(&a, stream);
    }
    if (err) {
        MM_LOGE("cuda: launch (gated pair, variant %d, M %u K %u inter %u): %s", a.plan.variant, M, K,
                inter, cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.launches++;
    return MM_OK;
}

mm_status mm_silu_mul(const void *gate, const void *up, void *y, size_t n, void *stream)
{
    MM_REQUIRE(gate && up && y, MM_ERR_STATE);
    if (n == 0)
        return MM_ERR_SHAPE;
    MM_CHECK(ensure_ready());
    if (!stream)
        stream = mm_cuda_stream_raw(MM_ST_COMPUTE);
    int err = mmb_launch_silu_mul(gate, up, y, n, stream);
    if (err) {
        MM_LOGE("cuda: silu_mul launch: %s", cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.launches++;
    return MM_OK;
}

static mm_status finish_op(void);

/* ------------------------------------------------------------- group launch
 * A run of decode linears that are independent of each other, as one persistent
 * launch of the block-scaled kernel (kernels/mxg.cu).  The engine opens a group,
 * adds ops while they fit, and launches it.  Scratch: arrival counters and
 * split-K partials of every op from one workspace region, digit planes from the
 * plane cache (an activation tensor several ops read is sliced once). */
typedef struct gr_item {
    mm_op_desc  op;
    int         glu, gate_first;
    const void *pay0, *sc0;          /* the lower-addressed projection of a gated pair, else b and d */
    const void *up_scale;
    uint64_t    dpay, dsc;
    uint32_t    align;
    uint32_t    split;               /* K slices chosen at launch */
    void       *y_dst[MMB_MAX_PEERS];/* tensor parallel: every rank's copy of the full output */
    uint32_t    n_dst, ldy, col0;
} gr_item;

static struct {
    int       active;
    int       pdl;
    uint32_t  n;
    gr_item   item[MMB_MXG_MAX_OPS];
    size_t    part_bound, cache_used;    /* upper bounds kept while ops are added */
    uint32_t  counters_bound;
    unsigned char *region;
    mmb_group g;                         /* filled at launch */
} GR;

mm_status mmb_group_begin(int pdl_mode, int ws_region)
{
    MM_CHECK(ensure_ready());
    MM_REQUIRE(G.ws && mmb_ws_regions() > 1, MM_ERR_STATE);
    GR.active = 1;
    GR.n = 0;
    GR.pdl = G.pdl ? (pdl_mode >= 0 ? pdl_mode : MMB_PDL_TRIGGER_FIRST) : MMB_PDL_OFF;
    const int r = ws_region >= 0 && ws_region < mmb_ws_regions() ? ws_region : 0;
    GR.region = (unsigned char *)G.ws + (size_t)r * ws_region_bytes();
    GR.part_bound = MMB_WS_COUNTER_B;
    GR.counters_bound = 0;
    GR.cache_used = 0;
    return MM_OK;
}

uint32_t mmb_group_size(void) { return GR.active ? GR.n : 0; }

static size_t gr_partial_bytes(const mm_f4_plan *p, uint32_t K)
{
    if (p->split_k <= 1)
        return 0;
    return (p->ws_needed - MMB_WS_COUNTER_B - MMB_MX_XS_B(p->tile_m, K) + 255u) & ~(size_t)255;
}

static mm_status gr_plan(const gr_item *it, uint32_t split, mm_f4_plan *plan)
{
    mm_f4_shape sh = { it->op.n0, it->op.n1, it->op.n2, (uint32_t)G.sm_count, it->align, ws_region_bytes() };
    return mmb_plan_mx_group(&sh, it->glu, split, plan);
}

static mm_status group_add(const mm_op_desc *op, int glu, const void *up_payload, const void *up_scale,
                           void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0);

/* MM_ERR_CAPACITY: the group is full (launch it and open another);
 * MM_ERR_UNSUPPORTED: this op does not run on the block-scaled kernel. */
mm_status mmb_group_add(const mm_op_desc *op, int glu, const void *up_payload, const void *up_scale)
{
    return group_add(op, glu, up_payload, up_scale, NULL, 0, 0, 0);
}

/* The tensor-parallel form of a plain linear: op->n2 output features (this rank's
 * shard) stored at column col0 of every rank's [M][ldy] output, op->c = y_all[0]. */
mm_status mmb_group_add_tp(const mm_op_desc *op, void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0)
{
    MM_REQUIRE(op && y_all && n_ranks >= 1 && n_ranks <= MMB_MAX_PEERS, MM_ERR_RANGE);
    for (uint32_t d = 0; d < n_ranks; d++)
        MM_REQUIRE(y_all[d] && ((uintptr_t)y_all[d] & 15u) == 0, MM_ERR_STATE);
    MM_REQUIRE((uint64_t)col0 + op->n2 <= ldy, MM_ERR_SHAPE);
    return group_add(op, 0, NULL, NULL, y_all, n_ranks, ldy, col0);
}

static mm_status group_add(const mm_op_desc *op, int glu, const void *up_payload, const void *up_scale,
                           void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0)
{
    MM_REQUIRE(GR.active && op, MM_ERR_STATE);
    if (GR.n == MMB_MXG_MAX_OPS)
        return MM_ERR_CAPACITY;
    gr_item it;
    memset(&it, 0, sizeof it);
    it.op = *op;
    it.glu = glu;
    it.pay0 = op->b; it.sc0 = op->d; it.gate_first = 1;
    it.up_scale = up_scale;
    it.align = min_align(op->a, op->b, op->d, op->c);
    it.n_dst = n_ranks; it.ldy = ldy; it.col0 = col0;
    for (uint32_t d = 0; d < n_ranks; d++) it.y_dst[d] = y_all[d];
    if (it.align < 16 || op->n0 == 0 || op->n1 == 0 || op->n2 == 0 || op->n1 % 16 != 0)
        return MM_ERR_SHAPE;
    if (glu) {
        if (!pair_layout(op->b, op->d, up_payload, up_scale, &it.gate_first, &it.dpay, &it.dsc))
            return MM_ERR_UNSUPPORTED;
        it.pay0 = it.gate_first ? op->b : up_payload;
        it.sc0 = it.gate_first ? op->d : up_scale;
        it.align = min_align(op->a, it.pay0, it.sc0, op->c);
    }
    mm_f4_plan plan;
    if (gr_plan(&it, 0, &plan) != MM_OK || plan.variant != MM_F4_V_MX)
        return MM_ERR_UNSUPPORTED;
    const size_t pb = gr_partial_bytes(&plan, op->n1);
    if (GR.part_bound + pb > ws_region_bytes() || GR.counters_bound + plan.grid_x > MMB_WS_MAX_TILES - 2u)
        return MM_ERR_CAPACITY;
    int shared = 0;
    for (uint32_t i = 0; i < GR.n; i++)
        if (GR.item[i].op.a == op->a && GR.item[i].op.n0 == op->n0 && GR.item[i].op.n1 == op->n1)
            shared = 1;
    if (!shared) {
        size_t cap = 0;
        const size_t need = (MMB_MX_XS_B(plan.tile_m, op->n1) + 1023u) & ~(size_t)1023u;
        if (!mmb_plane_cache(&cap) || GR.cache_used + need > cap)
            return MM_ERR_CAPACITY;
        GR.cache_used += need;
    }
    GR.part_bound += pb;
    GR.counters_bound += plan.grid_x;
    GR.item[GR.n++] = it;
    return MM_OK;
}

/* Bytes of weights the busiest CTA streams when the units are dealt in turn over
 * `ctas` CTAs, given every op's plan: the planner's model of a launch.  (The kernel
 * hands units out as CTAs ask, which only evens things out further; a model that
 * did the same and counted the digit planes' bytes chose far too many K slices for
 * short launches, 58 us instead of 37 for the two-op down launch, because it does
 * not see what a slice costs in the split-K exchange: a split unit keeps its CTA's
 * epilogue warps for about 4 us of stores, fence and ticket, and the last to arrive
 * for 5 more.  Setting every op's split together from a common unit size ran the
 * five-op launch of a layer in 51 us instead of 38 for the same reason.) */
static double gr_makespan(const mm_f4_plan *plans, uint32_t n, uint32_t ctas)
{
    static double load[1024];
    if (ctas > 1024u) ctas = 1024u;
    for (uint32_t c = 0; c < ctas; c++) load[c] = 0.0;
    uint32_t g = 0;
    for (uint32_t i = 0; i < n; i++) {
        const double unit = (double)plans[i].tile_n * 144.0 * (double)plans[i].k_steps / (double)plans[i].split_k;
        const uint32_t units = plans[i].grid_x * plans[i].split_k;
        for (uint32_t u = 0; u < units; u++, g++)
            load[g % ctas] += unit + 40000.0;      /* a unit costs about a microsecond beside its bytes */
    }
    double worst = 0.0;
    for (uint32_t c = 0; c < ctas; c++)
        if (load[c] > worst) worst = load[c];
    return worst;
}

mm_status mmb_group_launch(void)
{
    MM_REQUIRE(GR.active, MM_ERR_STATE);
    GR.active = 0;
    if (GR.n == 0)
        return MM_OK;
    /* plans: units of up to about 768 KiB; then, from the last op backwards, a
     * finer K split is kept wherever it shortens the busiest CTA's share */
    static mm_f4_plan plans[MMB_MXG_MAX_OPS];
    /* the ops of a group are independent: the ones with many activation rows (whose units
     * take longest per byte, and whose split-K exchange is largest) go first, so that the
     * launch ends on short units (insertion sort, stable).  Measured on the ten-op decode
     * sweep: 137.8 us per step against 148.0 in list order; ordering equal-M ops by size as
     * well changed nothing. */
    if (G.group_sort)
        for (uint32_t i = 1; i < GR.n; i++) {
            const gr_item it = GR.item[i];
            uint32_t j = i;
            while (j > 0 && GR.item[j - 1].op.n0 < it.op.n0) {
                GR.item[j] = GR.item[j - 1];
                j--;
            }
            GR.item[j] = it;
        }
    for (uint32_t i = 0; i < GR.n; i++)
        MM_CHECK(gr_plan(&GR.item[i], 0, &plans[i]));
    double best = gr_makespan(plans, GR.n, (uint32_t)G.sm_count);
    /* a short launch (fewer than three units per SM) has no long run of units to even
     * things out: every op's K split is searched outright, twice over the ops, for the
     * shortest share of the busiest CTA (down alone: 20 tiles x 7 slices on 148 SMs
     * instead of 20 x 4) */
    uint32_t units = 0;
    for (uint32_t i = 0; i < GR.n; i++)
        units += plans[i].grid_x * plans[i].split_k;
    if (units < 3u * (uint32_t)G.sm_count)
        for (int pass = 0; pass < 2; pass++)
            for (uint32_t k = 0; k < GR.n; k++)
                for (uint32_t sk = 1; sk <= 16u; sk++) {
                    mm_f4_plan trial;
                    if (gr_plan(&GR.item[k], sk, &trial) != MM_OK || trial.split_k != sk ||
                        trial.split_k == plans[k].split_k || trial.grid_x != plans[k].grid_x)
                        continue;
                    const mm_f4_plan keep = plans[k];
                    const size_t was = gr_partial_bytes(&keep, GR.item[k].op.n1),
                                 now = gr_partial_bytes(&trial, GR.item[k].op.n1);
                    if (now > was && GR.part_bound + (now - was) > ws_region_bytes())
                        continue;
                    plans[k] = trial;
                    const double t = gr_makespan(plans, GR.n, (uint32_t)G.sm_count);
                    if (t < best * 0.985) {
                        best = t;
                        GR.part_bound = GR.part_bound + now - was;
                    } else {
                        plans[k] = keep;
                    }
                }
    for (uint32_t k = GR.n; k-- > 0;)
        for (uint32_t extra = 1; extra <= 2u; extra++) {
            mm_f4_plan trial;
            if (gr_plan(&GR.item[k], plans[k].split_k + extra, &trial) != MM_OK ||
                trial.split_k <= plans[k].split_k)
                continue;
            const mm_f4_plan keep = plans[k];
            const size_t grow = gr_partial_bytes(&trial, GR.item[k].op.n1) - gr_partial_bytes(&keep, GR.item[k].op.n1);
            if (GR.part_bound + grow > ws_region_bytes() || trial.grid_x != keep.grid_x)
                continue;                        /* every op's tile counters are already reserved */
            plans[k] = trial;
            const double t = gr_makespan(plans, GR.n, (uint32_t)G.sm_count);
            if (t < best * 0.985) {
                best = t;
                GR.part_bound += grow;
            } else {
                plans[k] = keep;
            }
        }

#ifdef MMB_MEASURE_MODES
    if (getenv("MMB_PRINT_PLANS"))
        for (uint32_t i = 0; i < GR.n; i++)
            fprintf(stderr, "group op %u: M=%u K=%u N=%u glu=%d rows=%u tiles=%u split=%u k_steps=%u\n", i,
                    GR.item[i].op.n0, GR.item[i].op.n1, GR.item[i].op.n2, GR.item[i].glu, plans[i].tile_n,
                    plans[i].grid_x, plans[i].split_k, plans[i].k_steps);
#endif
    mmb_group *gg = &GR.g;
    memset(gg, 0, sizeof *gg);
    gg->pdl = GR.pdl;
    gg->acc_bufs = 2;
    size_t part_used = MMB_WS_COUNTER_B, cache_used = 0, cap = 0;
    uint32_t counters_used = 0, sliced = 0;
    unsigned char *cache = (unsigned char *)mmb_plane_cache(&cap);
    for (uint32_t i = 0; i < GR.n; i++) {
        const gr_item *it = &GR.item[i];
        const mm_f4_plan *plan = &plans[i];
        const uint32_t M = it->op.n0, K = it->op.n1, N = it->op.n2, nb = plan->tile_m;
        mmb_gop *g = &gg->op[i];
        for (uint32_t j = 0; j < i; j++)
            if (gg->op[j].x == it->op.a && gg->op[j].M == M && gg->op[j].K == K)
                g->x_ws = gg->op[j].x_ws;
        if (!g->x_ws) {
            g->x_ws = cache + cache_used;
            g->slice_here = 1;
            cache_used += (MMB_MX_XS_B(nb, K) + 1023u) & ~(size_t)1023u;
            sliced++;
        }
        g->x = it->op.a; g->y = it->op.c;
        g->n_dst = it->n_dst; g->ldy = it->ldy; g->col0 = it->col0;
        for (uint32_t d = 0; d < it->n_dst; d++) g->y_dst[d] = it->y_dst[d];
        g->gs = mm_f4_gscale_get(it->op.d);
        g->gs_up = it->glu ? mm_f4_gscale_get(it->up_scale) : 0.0f;
        g->glu = it->glu; g->gate_plane = it->glu ? (it->gate_first ? 0 : 1) : 0;
        g->M = M; g->K = K; g->N = N;
        g->rows = plan->tile_n; g->nb = nb; g->k_steps = plan->k_steps; g->split_k = plan->split_k;
        g->tiles = plan->grid_x; g->unit0 = gg->n_units;
        if (plan->split_k > 1) {
            const size_t pb = gr_partial_bytes(plan, K);
            MM_REQUIRE(part_used + pb <= ws_region_bytes() && counters_used + plan->grid_x <= MMB_WS_MAX_TILES - 2u &&
                       cache_used <= cap, MM_ERR_CAPACITY);
            g->counters_idx = counters_used;
            g->partial = GR.region + part_used;
            counters_used += plan->grid_x;
            part_used += pb;
        }
        if (it->glu) {
            MM_CHECK(encode_pair(g->tm_payload, it->pay0, K / 2, N, it->dpay, 128, plan->tile_n / 2,
                                 CU_TENSOR_MAP_SWIZZLE_128B));
            MM_CHECK(encode_pair(g->tm_scale, it->sc0, K / 16, N, it->dsc, 16, plan->tile_n / 2,
                                 CU_TENSOR_MAP_SWIZZLE_NONE));
        } else {
            MM_CHECK(encode_2d(g->tm_payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, it->pay0, K / 2, N, 128,
                               plan->tile_n, CU_TENSOR_MAP_SWIZZLE_128B));
            MM_CHECK(encode_2d(g->tm_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, it->sc0, K / 16, N, 16,
                               plan->tile_n, CU_TENSOR_MAP_SWIZZLE_NONE));
        }
        unsigned char *planes = (unsigned char *)g->x_ws + MMB_MX_PLANES_OFF;
        MM_CHECK(encode_2d(g->tm_planes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, planes, K / 2, nb, 128, nb,
                           CU_TENSOR_MAP_SWIZZLE_128B));
        MM_CHECK(encode_2d(g->tm_sfb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, planes + MMB_MX_PLANES_B(nb, K), K / 16,
                           nb, 16, nb, CU_TENSOR_MAP_SWIZZLE_NONE));
        const uint32_t stage = MMB_MX_STAGE_B(plan->tile_n, nb, it->glu);
        if (stage > gg->stage_b) gg->stage_b = stage;
        if (nb > 96u) gg->acc_bufs = 1;
        gg->n_units += plan->grid_x * plan->split_k;
    }
    gg->n_ops = GR.n;
    uint32_t st = (MMB_SMEM_MAX - MMB_MXG_FIXED_B) / gg->stage_b;
    if (st > 6) st = 6;
    if (G.mx_stages && st > G.mx_stages) st = G.mx_stages;
    if (st < 2) st = 2;
    gg->stages = st;
    gg->smem_bytes = st * gg->stage_b + MMB_MXG_FIXED_B;
    gg->grid = gg->n_units < (uint32_t)G.sm_count ? gg->n_units : (uint32_t)G.sm_count;
    if (G.l2_window && G.ws) {
        /* window over the plane cache half of the workspace + this group's region */
        int dev = 0, max_win = 0, max_persist = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&max_win, cudaDevAttrMaxAccessPolicyWindowSize, dev);
        cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, dev);
        size_t want = cache_used + 4096u;
        if (want > (size_t)max_win) want = (size_t)max_win;
        if (!G.l2_limit_set && max_persist > 0) {
            size_t lim = (size_t)max_persist < ((size_t)32 << 20) ? (size_t)max_persist : ((size_t)32 << 20);
            if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, lim) == cudaSuccess)
                G.l2_limit_set = 1;
            else
                (void)cudaGetLastError();
        }
        if (G.l2_limit_set && want) {
            gg->l2_base = cache;
            gg->l2_bytes = want;
        }
    }
    /* the last two words of the region's counter block: the units handed out, the CTAs done */
    gg->counters = GR.region;
    gg->sched = G.static_units ? NULL : (void *)(GR.region + (size_t)(MMB_WS_MAX_TILES - 2u) * 4u);
    uint32_t kernels = 0;
    int err = mmb_launch_mxg(gg, mm_cuda_stream_raw(MM_ST_COMPUTE), &kernels);
    if (err) {
        MM_LOGE("cuda: group launch (%u ops, %u units): %s", gg->n_ops, gg->n_units,
                cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.launches += kernels;
    G.sliced_x = NULL;
    return finish_op();
}

mm_status mm_f4_linear_tp(const void *x, const void *payload, const void *scale, float gs,
                          void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0,
                          uint32_t M, uint32_t K, uint32_t N_local, void *stream)
{
    MM_REQUIRE(y_all && n_ranks >= 1 && n_ranks <= MMB_MAX_PEERS, MM_ERR_RANGE);
    for (uint32_t d = 0; d < n_ranks; d++)
        MM_REQUIRE(y_all[d] && ((uintptr_t)y_all[d] & 15u) == 0, MM_ERR_STATE);
    MM_REQUIRE((uint64_t)col0 + N_local <= ldy, MM_ERR_SHAPE);
    return linear_impl(x, payload, scale, gs, y_all[0], y_all, n_ranks, ldy, col0, M, K, N_local,
                       stream);
}

/* Synchronise the compute stream and collect launch/device errors, unless a
 * capture is in progress (then only launch errors can be seen). */
static mm_status finish_op(void)
{
    cudaStream_t cs = (cudaStream_t)mm_cuda_stream_raw(MM_ST_COMPUTE);
    if (!mm_cuda_capturing()) {
        CK(cudaMemcpyAsync(G.status_host, G.status_dev, sizeof(unsigned), cudaMemcpyDeviceToHost, cs));
        CK(cudaStreamSynchronize(cs));
        if (*G.status_host) {
            unsigned f = *G.status_host;
            *G.status_host = 0;
            CK(cudaMemsetAsync(G.status_dev, 0, sizeof(unsigned), cs));
            MM_LOGE("device status 0x%x after op", f);
            return (f & MMB_DEV_TIMEOUT) ? MM_ERR_TIMEOUT : MM_ERR_CUDA;
        }
    }
    CK(cudaGetLastError());
    return MM_OK;
}

mm_status mm_f4_device_status(unsigned *flags_out)
{
    MM_REQUIRE(flags_out, MM_ERR_STATE);
    MM_CHECK(ensure_ready());
    cudaStream_t cs = (cudaStream_t)mm_cuda_stream_raw(MM_ST_COMPUTE);
    CK(cudaMemcpyAsync(G.status_host, G.status_dev, sizeof(unsigned), cudaMemcpyDeviceToHost, cs));
    CK(cudaMemsetAsync(G.status_dev, 0, sizeof(unsigned), cs));
    CK(cudaStreamSynchronize(cs));
    *flags_out = *G.status_host;
    *G.status_host = 0;
    return MM_OK;
}

mm_status kx_op_gemm_f4(const mm_kcall *kc)
{
    MM_REQUIRE(kc && kc->op, MM_ERR_STATE);
    const mm_op_desc *op = kc->op;
    if (op->n1 % 16 != 0)
        return MM_ERR_SHAPE;
    MM_REQUIRE(op->a && op->b && op->c && op->d, MM_ERR_STATE);
    MM_REQUIRE(mm_cuda_stream_raw(MM_ST_COMPUTE) != NULL, MM_ERR_STATE);
    mm_status st = mm_f4_linear(op->a, op->b, op->d, mm_f4_gscale_get(op->d), op->c, op->n0,
                                op->n1, op->n2, mm_cuda_stream_raw(MM_ST_COMPUTE));
    if (st != MM_OK)
        return st;
    return finish_op();
}

mm_status kx_op_qkv(const mm_kcall *kc)
{
    MM_REQUIRE(kc && kc->op, MM_ERR_STATE);
    if (!kc->op->d)
        return MM_ERR_UNSUPPORTED;     /* bf16 fused qkv: not this library's op */
    return kx_op_gemm_f4(kc);
}

mm_status mmb_plan_for_op(const mm_op_desc *op, int glu, mm_f4_plan *out)
{
    MM_REQUIRE(op && out, MM_ERR_STATE);
    MM_CHECK(ensure_ready());
    if (glu) {
        /* the lower-addressed projection decides the alignment; both are placed alike */
        mm_f4_shape sh = { op->n0, op->n1, op->n2, (uint32_t)G.sm_count,
                           min_align(op->a, op->b, op->d, op->c), ws_region_bytes() };
        return mmb_select_glu(&sh, G.use_mx, out);
    }
    return plan_linear(op->a, op->b, op->d, op->c, 0, 0, 0, op->n0, op->n1, op->n2, 0, out);
}

/* a tensor-parallel linear of an op list that runs on its own (not in a group launch) */
mm_status mmb_op_linear_tp(const mm_op_desc *op, void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0)
{
    MM_REQUIRE(op && op->a && op->b && op->c && op->d, MM_ERR_STATE);
    MM_REQUIRE(mm_cuda_stream_raw(MM_ST_COMPUTE) != NULL, MM_ERR_STATE);
    mm_status st = mm_f4_linear_tp(op->a, op->b, op->d, mm_f4_gscale_get(op->d), y_all, n_ranks, ldy, col0,
                                   op->n0, op->n1, op->n2, mm_cuda_stream_raw(MM_ST_COMPUTE));
    if (st != MM_OK)
        return st;
    return finish_op();
}

mm_status mmb_op_mlp_gate_up(const mm_op_desc *op, const void *up_payload, const void *up_scale)
{
    MM_REQUIRE(op && op->a && op->b && op->c && op->d && up_payload && up_scale, MM_ERR_STATE);
    MM_REQUIRE(mm_cuda_stream_raw(MM_ST_COMPUTE) != NULL, MM_ERR_STATE);
    mm_status st = mm_f4_mlp_gate_up(op->a, op->b, op->d, mm_f4_gscale_get(op->d), up_payload, up_scale,
                                     mm_f4_gscale_get(up_scale), op->c, op->n0, op->n1, op->n2,
                                     mm_cuda_stream_raw(MM_ST_COMPUTE));
    if (st != MM_OK)
        return st;
    return finish_op();
}

/* OP_LMHEAD carries the same operands as a GEMM (src/kernels/cpu/cx.c:187-190
 * forwards it to the bf16 GEMM); with a scale tensor in `d` it is the NVFP4 op. */
mm_status kx_op_lmhead(const mm_kcall *kc)
{
    MM_REQUIRE(kc && kc->op, MM_ERR_STATE);
    if (!kc->op->d)
        return MM_ERR_UNSUPPORTED;     /* bf16 head: not this library's op */
    return kx_op_gemm_f4(kc);
}

/* OP_SILU_MUL: a = gate, b = up, c = y, n0 x n1 elements (include/mimfer/kernels.h:87). */
mm_status kx_op_silu_mul(const mm_kcall *kc)
{
    MM_REQUIRE(kc && kc->op, MM_ERR_STATE);
    const mm_op_desc *op = kc->op;
    MM_REQUIRE(op->a && op->b && op->c, MM_ERR_STATE);
    MM_REQUIRE(mm_cuda_stream_raw(MM_ST_COMPUTE) != NULL, MM_ERR_STATE);
    mm_status st = mm_silu_mul(op->a, op->b, op->c, (size_t)op->n0 * op->n1,
                               mm_cuda_stream_raw(MM_ST_COMPUTE));
    if (st != MM_OK)
        return st;
    return finish_op();
}

/* Epsilon of the RMSNorm.  The reference reads it from the engine's model
 * configuration (kc->e->mc.norm_eps, src/kernels/cpu/cx.c:143); the engine is
 * opaque to this library, so its owner registers the value once. */
static float g_norm_eps = 1.0e-6f;

mm_status mm_norm_eps_set(float eps)
{
    MM_REQUIRE(eps == eps && eps >= 0.0f && eps < 1.0f, MM_ERR_RANGE);
    g_norm_eps = eps;
    return MM_OK;
}

float mm_norm_eps_get(void) { return g_norm_eps; }

mm_status mm_add_rmsnorm(void *res, const void *delta, void *y, const void *gain, uint32_t M, uint32_t H,
                         void *stream)
{
    MM_REQUIRE(res && delta && y && gain, MM_ERR_STATE);
    if (M == 0 || H == 0)
        return MM_ERR_SHAPE;
    MM_CHECK(ensure_ready());
    if (!stream)
        stream = mm_cuda_stream_raw(MM_ST_COMPUTE);
    int pdl = 0, shallow = 0, share = 0;
    void *ws = NULL;
    take_op_context(&pdl, &ws, &shallow, &share);
    int err = mmb_launch_add_rmsnorm(res, delta, y, gain, M, H, g_norm_eps, pdl != MMB_PDL_OFF, stream);
    if (err) {
        MM_LOGE("cuda: add_rmsnorm launch: %s", cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.sliced_x = NULL;                 /* activations change under the planes made last */
    G.launches++;
    return MM_OK;
}

/* OP_ADD_RMSNORM: a = residual (updated in place), b = delta, c = normalised
 * output, d = gain, n0 = M rows of n1 values (include/mimfer/kernels.h:87-88). */
mm_status kx_op_add_rmsnorm(const mm_kcall *kc)
{
    MM_REQUIRE(kc && kc->op, MM_ERR_STATE);
    const mm_op_desc *op = kc->op;
    MM_REQUIRE(op->a && op->b && op->c && op->d, MM_ERR_STATE);
    MM_REQUIRE(mm_cuda_stream_raw(MM_ST_COMPUTE) != NULL, MM_ERR_STATE);
    mm_status st = mm_add_rmsnorm((void *)(uintptr_t)op->a, op->b, op->c, op->d, op->n0, op->n1,
                                  mm_cuda_stream_raw(MM_ST_COMPUTE));
    if (st != MM_OK)
        return st;
    return finish_op();
}

/* Inside the mimfer tree the dispatcher (src/kernels/kx.c) and the op preference
 * table (src/kernels/cuda/cx.cu) are mimfer's own: build with -DMMB_NO_DISPATCHER. */
#ifndef MMB_NO_DISPATCHER
int kx_cuda_oppref(int op)
{
    return op == OP_GEMM_F4 || op == OP_QKV || op == OP_LMHEAD || op == OP_SILU_MUL ||
           op == OP_ADD_RMSNORM || op == OP_NOP;
}

mm_status mm_kx_invoke(const mm_kcall *kc)
{
    if (!kc || !kc->op || !kc->e)
        return MM_ERR_STATE;
    switch (kc->op->op) {
    case OP_GEMM_F4: return kx_op_gemm_f4(kc);
    case OP_QKV:     return kx_op_qkv(kc);
    case OP_LMHEAD:  return kx_op_lmhead(kc);
    case OP_SILU_MUL: return kx_op_silu_mul(kc);
    case OP_ADD_RMSNORM: return kx_op_add_rmsnorm(kc);
    case OP_NOP:     return MM_OK;
    default:
        MM_LOGE("kx: opcode %d is not served by the NVFP4 linear library", kc->op->op);
        return MM_ERR_UNSUPPORTED;
    }
}
#endif /* MMB_NO_DISPATCHER */

mm_status mm_f4_linear_host(const void *x_host, void *x_dev, const void *payload_dev,
                            const void *scale_dev, float gs, void *y_dev, void *y_host,
                            uint32_t M, uint32_t K, uint32_t N)
{
    MM_REQUIRE(x_host && x_dev && y_dev && y_host, MM_ERR_STATE);
    MM_REQUIRE(!mm_cuda_capturing(), MM_ERR_BUSY);
    MM_CHECK(mm_h2d_async(x_dev, x_host, (size_t)M * K * 2u, MM_ST_COMPUTE));
    mm_status st = mm_f4_linear(x_dev, payload_dev, scale_dev, gs, y_dev, M, K, N, NULL);
    if (st != MM_OK)
        return st;
    MM_CHECK(mm_d2h_async(y_host, y_dev, (size_t)M * N * 2u, MM_ST_COMPUTE));
    return finish_op();
}

mm_status mm_f4_tp_barrier(void *const *flags_all, uint32_t n_ranks, uint32_t rank, void *stream)
{
    MM_REQUIRE(flags_all && n_ranks >= 1 && n_ranks <= MMB_MAX_PEERS && rank < n_ranks, MM_ERR_RANGE);
    for (uint32_t r = 0; r < n_ranks; r++)
        MM_REQUIRE(flags_all[r] && ((uintptr_t)flags_all[r] & 3u) == 0, MM_ERR_STATE);
    MM_CHECK(ensure_ready());
    if (!stream)
        stream = mm_cuda_stream_raw(MM_ST_COMPUTE);
    int err = mmb_launch_tp_barrier((unsigned *const *)flags_all, n_ranks, rank, stream);
    if (err) {
        MM_LOGE("cuda: tensor-parallel barrier launch: %s", cudaGetErrorString((cudaError_t)err));
        return MM_ERR_CUDA;
    }
    G.launches++;
    return MM_OK;
}

mm_status mm_f4_tp_push(void *const *y_all, uint32_t n_ranks, uint32_t ldy, uint32_t col0, uint32_t cols,
                        uint32_t row0, uint32_t rows)
{
    MM_REQUIRE(y_all && n_ranks >= 1 && n_ranks <= MMB_MAX_PEERS, MM_ERR_RANGE);
    MM_REQUIRE(cols && rows && (uint64_t)col0 + cols <= ldy, MM_ERR_SHAPE);
    MM_REQUIRE(ldy % 8u == 0 && col0 % 8u == 0 && cols % 8u == 0, MM_ERR_SHAPE);
    for (uint32_t d = 0; d < n_ranks; d++)
        MM_REQUIRE(y_all[d] && ((uintptr_t)y_all[d] & 15u) == 0, MM_ERR_STATE);
    MM_CHECK(ensure_ready());
    if (n_ranks == 1)
        return MM_OK;
    cudaStream_t cs = (cudaStream_t)mm_cuda_stream_raw(MM_ST_COMPUTE);
    if (!TP.ready)
        CK(cudaEventCreateWithFlags(&TP.ready, cudaEventDisableTiming));
    CK(cudaEventRecord(TP.ready, cs));                       /* the slice is complete in the own copy */
    /* One stream's copy reaches 757 GB/s to a single peer, but four ranks that push to
     * three peers each got 360 GB/s per GPU out of one stream per peer and 425 out of
     * three: every peer gets several streams, about eight over all peers, and a push is
     * cut into as many runs of rows. */
    uint32_t lanes = G.tp_lanes ? G.tp_lanes : (TP_LANES + n_ranks - 2u) / (n_ranks - 1u);
    if (lanes > TP_LANES) lanes = TP_LANES;
    if (lanes > rows / 64u) lanes = rows / 64u ? rows / 64u : 1u;
    const size_t pitch = (size_t)ldy * 2u;
    for (uint32_t d = 1; d < n_ranks; d++)
        for (uint32_t l = 0; l < lanes; l++) {
            const uint32_t r0 = (uint32_t)((uint64_t)rows * l / lanes), r1 = (uint32_t)((uint64_t)rows * (l + 1u) / lanes);
            const size_t off = (size_t)(row0 + r0) * pitch + (size_t)col0 * 2u;
            if (!TP.made[d][l]) {
                CK(cudaStreamCreateWithFlags(&TP.side[d][l], cudaStreamNonBlocking));
                CK(cudaEventCreateWithFlags(&TP.done[d][l], cudaEventDisableTiming));
                TP.made[d][l] = 1;
            }
            CK(cudaStreamWaitEvent(TP.side[d][l], TP.ready, 0));
            CK(cudaMemcpy2DAsync((unsigned char *)y_all[d] + off, pitch, (const unsigned char *)y_all[0] + off, pitch,
                                 (size_t)cols * 2u, r1 - r0, cudaMemcpyDefault, TP.side[d][l]));
            TP.pending[d][l] = 1;
        }
    return MM_OK;
}

mm_status mm_f4_tp_push_join(void)
{
    MM_CHECK(ensure_ready());
    cudaStream_t cs = (cudaStream_t)mm_cuda_stream_raw(MM_ST_COMPUTE);
    for (uint32_t d = 1; d < MMB_MAX_PEERS; d++)
        for (uint32_t l = 0; l < TP_LANES; l++) {
            if (!TP.pending[d][l])
                continue;
            CK(cudaEventRecord(TP.done[d][l], TP.side[d][l]));
            CK(cudaStreamWaitEvent(cs, TP.done[d][l], 0));
            TP.pending[d][l] = 0;
        }
    return MM_OK;
}

mm_status mm_f4_wait_selftest(unsigned *done_dev)
{
    MM_REQUIRE(done_dev, MM_ERR_STATE);
    MM_CHECK(ensure_ready());
    MM_REQUIRE(!mm_cuda_capturing(), MM_ERR_BUSY);
    cudaStream_t cs = (cudaStream_t)mm_cuda_stream_raw(MM_ST_COMPUTE);
    CK((cudaError_t)mmb_launch_wait_selftest(G.status_dev, done_dev, cs));
    G.launches++;
    return finish_op();                /* MM_ERR_TIMEOUT when the wait gave up as designed */
}

mm_status mm_f4_decode_probe(uint32_t *out_mma_dev, uint32_t *out_f32_dev, uint32_t *out_f16_dev)
{
    MM_REQUIRE(out_mma_dev && out_f32_dev && out_f16_dev, MM_ERR_STATE);
    MM_CHECK(ensure_ready());
    cudaStream_t cs = (cudaStream_t)mm_cuda_stream_raw(MM_ST_COMPUTE);
    CK((cudaError_t)mmb_launch_decode_probe(out_mma_dev, out_f32_dev, out_f16_dev, cs));
    G.launches++;
    CK(cudaStreamSynchronize(cs));
    return MM_OK;
}
