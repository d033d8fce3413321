/*
 * MXG: a group of independent NVFP4 decode linears in ONE persistent launch on
 * the block-scaled tensor path (the kernel of mx.cu turned into a work loop).
 *
 * A decode step is hundreds of short linears (3 to 100 MB of weights each).
 * Launched one by one, each pays its own launch, pipeline fill, tail and split-K
 * exchange, and the weight stream stops between them.  Here the ops the
 * engine has shown to be independent of each other (q, k and v of a layer; gate
 * and up; in a benchmark of stand-alone linears, all of them) are cut into work
 * units (op, row tile, K slice) that the CTAs, one per SM, take one after the
 * other from a shared counter, each when it is ready for one.  The TMA producer of a CTA runs ahead across unit and op borders, so
 * the weight stream never stops; the accumulators are double-buffered in tensor
 * memory (M <= 16), so a unit's epilogue overlaps the next unit's MMAs.
 *
 * The op list travels in the kernel's parameter space (up to 48 ops, 30 KB):
 * tensor maps there are usable by TMA as they are, nothing is uploaded.
 *
 * Per-op arithmetic, scale clean-up, epilogue and split-K exchange are those of
 * mx.cu; results are bit-identical to the single-op launches.
 *
 * Warp roles (15 warps): 0 = TMA producer; 1 and 10 = MMA issue (first / second
 * 128-row half); 2..9 = scale-factor copies into tensor memory (lane quadrant x
 * parity of the K step); 11..14 = epilogue (one per lane quadrant).
 *
 * It replaces a run of launches of the reference's one-thread-per-output kernel
 * (src/kernels/cuda/cx.cu:345-376), one per linear of the op walk
 * (src/plan/plan.c:119-138).
 */
#include "fp4.cuh"
#include "ptx.cuh"
#include <cooperative_groups.h>
#include "mx.cuh"

namespace mmb {

/* Time stamps of a launch, measurement builds only (-DMMB_MEASURE_MODES): per launch a
 * row of sixteen globaltimer values, minima and maxima over the CTAs.  [0]/[5] first/last
 * CTA entered, [1]/[2] first/last CTA past its grid-dependency wait, [3]/[6] first unit's
 * MMAs done in the first/last CTA, [7] last MMAs of all, [8]/[4] first/last epilogue warp
 * done, [9] last producer done, [10] first stage landed.  Slicing kernel: [3]/[6] loads
 * done, [7]/[9] last CTA past the first/second cluster barrier, [11] last thread 0 has sliced
 * its block, [10]/[4] first/last CTA done.  [15]: 1 = group kernel, 2 = slicing kernel. */
#ifdef MMB_MEASURE_MODES
#define MMB_TRACE_SLOTS 1024u
__device__ unsigned long long g_trace[MMB_TRACE_SLOTS][16];
__device__ __forceinline__ void trace_min(uint32_t slot1, uint32_t k)
{
    if (slot1) atomicMin(&g_trace[slot1 - 1u][k], static_cast<unsigned long long>(globaltimer_ns()));
}
__device__ __forceinline__ void trace_max(uint32_t slot1, uint32_t k)
{
    if (slot1) atomicMax(&g_trace[slot1 - 1u][k], static_cast<unsigned long long>(globaltimer_ns()));
}
#define MMB_TRACE_MIN(slot1, k) trace_min(slot1, k)
#define MMB_TRACE_MAX(slot1, k) trace_max(slot1, k)
#define MMB_TRACE_KIND(slot1, v) do { if (slot1) g_trace[(slot1) - 1u][15] = (v); } while (0)
#else
#define MMB_TRACE_MIN(slot1, k) ((void)0)
#define MMB_TRACE_MAX(slot1, k) ((void)0)
#define MMB_TRACE_KIND(slot1, v) ((void)0)
#endif

struct __align__(128) MxgOp {
    TmaDesc         tm_payload, tm_scale, tm_planes, tm_sfb;
    uint16_t       *y[MMB_MAX_PEERS];    /* destinations: own output, then the peers' (tensor parallel) */
    const float    *row_scale;
    float          *partial;
    float           gs, gs_up;
    uint32_t        M, N;                /* N: output features of this op (its shard's) */
    uint32_t        k_steps, tiles, unit0;
    uint32_t        counters_idx;        /* first arrival counter of the op in MxgGroup::counters */
    uint32_t        ldy, col0;           /* row pitch and column offset inside every destination */
    uint16_t        rows, nb, split_k;
    uint8_t         flags;               /* 1: gated pair, 2: the second plane of a tile is the gate */
    uint8_t         n_dst;
};
static_assert(sizeof(MxgOp) == 640, "MxgOp layout");

struct __align__(128) MxgGroup {
    uint32_t  n_ops, n_units, stages, acc_bufs;
    uint32_t  stage_b, pdl;
    unsigned *status;
    unsigned *sched;         /* [0] units handed out beyond the first of every CTA, [1] CTAs that took
                              * their last; both zero between launches.  NULL: unit u goes to CTA u mod grid */
    unsigned *counters;      /* arrival counters of the split tiles, zero between launches */
    uint32_t  trace_slot;    /* measurement builds: 1 + the launch's row of time stamps, 0 = none */
    uint32_t  pad[19];
};
static_assert(sizeof(MxgGroup) == 128, "MxgGroup layout");

/* The kernel's parameter block: the header and as many op descriptors as the launch
 * needs, in four sizes (0.8, 2.6, 7.8 and 30.8 KB).  A launch costs with the size of
 * its parameters: a one-op launch with the 48-op block took 8 to 13 us longer than the
 * single-op kernel on the same op. */
template <int NOPS>
struct __align__(128) MxgParams {
    MxgGroup grp;
    MxgOp    ops[NOPS];
};
static_assert(sizeof(MxgParams<MMB_MXG_MAX_OPS>) <= 32764, "kernel parameter space");

/* The units of one CTA, in order.  The producer thread decides them (the first is
 * blockIdx.x, the following ones come from a counter all CTAs share, so a CTA takes a
 * new unit whenever it is ready for one) and hands the numbers to the other warps
 * through a small queue in shared memory: slot j mod 8 holds the CTA's j-th unit, a
 * number >= n_units ends the walk.  Fourteen readers per slot: two MMA threads, eight
 * scale-copy warps, four epilogue warps. */
#define MMB_MXG_QUEUE   8u
#define MMB_MXG_READERS 14u
struct UnitWalk {
    uint32_t g, op, j;
    uint32_t q_ids, q_full, q_empty;
    unsigned *status;
    __device__ __forceinline__ void start(uint32_t ids, uint32_t full, uint32_t empty, unsigned *st)
    {
        q_ids = ids; q_full = full; q_empty = empty; status = st;
        g = 0; op = 0; j = 0;
    }
    /* by one thread (WARP = false) or by every lane of a warp */
    template <bool WARP>
    __device__ __forceinline__ bool valid(const MxgGroup &grp, const MxgOp *ops)
    {
        const uint32_t slot = j % MMB_MXG_QUEUE;
        bool ok = mbar_wait(q_full + 8u * slot, (j / MMB_MXG_QUEUE) & 1u, status);
        g = lds32(q_ids + 4u * slot);
        if (WARP) {
            ok = __all_sync(0xffffffffu, ok);
            if ((threadIdx.x & 31u) == 0)
                mbar_arrive(q_empty + 8u * slot);
        } else {
            mbar_arrive(q_empty + 8u * slot);
        }
        if (!ok || g >= grp.n_units)
            return false;
        while (op + 1u < grp.n_ops && g >= ops[op + 1u].unit0) op++;
        return true;
    }
    __device__ __forceinline__ void next() { j++; }
};

struct UnitGeom {
    uint32_t tile, slice, ks_begin, nsteps;
    uint32_t rows, nb, halves, h1, cnt0, cnt1, row0;
    uint32_t o_pl, o_sc, o_sfb, tx;
    bool glu;
};

__device__ __forceinline__ UnitGeom unit_geom(const MxgOp &o, uint32_t g)
{
    UnitGeom u;
    const uint32_t v = g - o.unit0;
    u.tile = v / o.split_k;
    u.slice = v - u.tile * o.split_k;
    u.ks_begin = static_cast<uint32_t>(static_cast<uint64_t>(o.k_steps) * u.slice / o.split_k);
    u.nsteps = static_cast<uint32_t>(static_cast<uint64_t>(o.k_steps) * (u.slice + 1u) / o.split_k) - u.ks_begin;
    u.glu = (o.flags & 1u) != 0u;
    u.rows = o.rows; u.nb = o.nb;
    u.halves = u.glu ? 2u : (u.rows > 128u ? 2u : 1u);
    u.h1 = u.glu ? u.rows >> 1 : 128u;
    u.cnt0 = u.glu ? u.rows >> 1 : (u.rows < 128u ? u.rows : 128u);
    u.cnt1 = u.rows - u.cnt0;
    u.row0 = u.tile * (u.glu ? u.rows >> 1 : u.rows);
    u.o_pl = (u.glu || u.rows > 128u) ? 32768u : 16384u;
    u.o_sc = u.o_pl + u.nb * 128u;
    u.o_sfb = u.o_sc + ((u.rows * 16u + 127u) & ~127u);
    u.tx = u.rows * 144u + u.nb * 144u;
    return u;
}

/* one bf16 to every destination of the op */
__device__ __forceinline__ void mxg_store(const MxgOp &o, size_t off, uint16_t v)
{
    o.y[0][off] = v;
    for (uint32_t d = 1; d < o.n_dst; d++)
        o.y[d][off] = v;
}

__device__ __forceinline__ void mxg_load_weights(const MxgOp &o, const UnitGeom &u, uint32_t st, uint32_t ks,
                                                 uint32_t bar)
{
    if (u.glu) {
        tma_load_3d(st, &o.tm_payload, static_cast<int>(ks * 128u), static_cast<int>(u.row0), 0, bar);
        tma_load_3d(st + u.o_sc, &o.tm_scale, static_cast<int>(ks * 16u), static_cast<int>(u.row0), 0, bar);
    } else {
        tma_load_2d(st, &o.tm_payload, static_cast<int>(ks * 128u), static_cast<int>(u.row0), bar);
        tma_load_2d(st + u.o_sc, &o.tm_scale, static_cast<int>(ks * 16u), static_cast<int>(u.row0), bar);
    }
}
__device__ __forceinline__ void mxg_load_planes(const MxgOp &o, const UnitGeom &u, uint32_t st, uint32_t ks,
                                                uint32_t bar)
{
    tma_load_2d(st + u.o_pl, &o.tm_planes, static_cast<int>(ks * 128u), 0, bar);
    tma_load_2d(st + u.o_sfb, &o.tm_sfb, static_cast<int>(ks * 16u), 0, bar);
}

template <int NOPS>
__global__ void __maxnreg__(128)
f4_mxg_kernel(const __grid_constant__ MxgParams<NOPS> prm)
{
    const MxgGroup &grp = prm.grp;
    const MxgOp *ops = prm.ops;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ST = grp.stages, stage_b = grp.stage_b, AB = grp.acc_bufs;
    const uint32_t bars = base + ST * stage_b;
    const uint32_t bar_full = bars;                       /* [ST] TMA landed                       */
    const uint32_t bar_empty = bar_full + 8u * ST;        /* [ST] both MMA threads past the stage  */
    const uint32_t bar_sf_full = bar_empty + 8u * ST;     /* [2]  scale factors in tensor memory   */
    const uint32_t bar_acc_full = bar_sf_full + 16u;      /* [2]  a unit's MMAs done               */
    const uint32_t bar_acc_empty = bar_acc_full + 16u;    /* [2]  its accumulators read            */
    const uint32_t tmem_slot = bar_acc_empty + 16u;
    const uint32_t last_flag = tmem_slot + 4u;
    const uint32_t q_full = tmem_slot + 8u;                /* [8] a unit number is in the slot      */
    const uint32_t q_empty = q_full + 8u * MMB_MXG_QUEUE;  /* [8] all its readers have taken it     */
    const uint32_t q_ids = q_empty + 8u * MMB_MXG_QUEUE;   /* [8] unit numbers                      */
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    if (tid == 0) {
        MMB_TRACE_MIN(grp.trace_slot, 0);
        MMB_TRACE_MAX(grp.trace_slot, 5);
        MMB_TRACE_KIND(grp.trace_slot, 1ull);
        for (uint32_t s = 0; s < ST; s++) {
            mbar_init(bar_full + 8u * s, 1u);
            mbar_init(bar_empty + 8u * s, 2u);
        }
        for (uint32_t t = 0; t < 2u; t++) {
            mbar_init(bar_sf_full + 8u * t, 4u);
            mbar_init(bar_acc_full + 8u * t, 2u);
            mbar_init(bar_acc_empty + 8u * t, 4u);
        }
        for (uint32_t q = 0; q < MMB_MXG_QUEUE; q++) {
            mbar_init(q_full + 8u * q, 1u);
            mbar_init(q_empty + 8u * q, MMB_MXG_READERS);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512u);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds32(tmem_slot);

    if (warp == 0) {
        /* ------------------------------ TMA producer -------------------------- *
         * The weights of the first ring go out before the grid-dependency wait, the
         * digit planes (made by the kernel in front) after it; from then on a step's
         * four boxes go out together as soon as its stage is free. */
        if (lane == 0) {
            uint32_t pushed = 0;
            auto push = [&](uint32_t id) {
                const uint32_t slot = pushed % MMB_MXG_QUEUE;
                if (pushed >= MMB_MXG_QUEUE)
                    mbar_wait(q_empty + 8u * slot, ((pushed / MMB_MXG_QUEUE) - 1u) & 1u, grp.status);
                sts32(q_ids + 4u * slot, id);
                mbar_arrive(q_full + 8u * slot);
                pushed++;
            };
            uint32_t g = blockIdx.x, op = 0;                /* the grid never exceeds the units */
            push(g);
            while (op + 1u < grp.n_ops && g >= ops[op + 1u].unit0) op++;
            UnitGeom u = unit_geom(ops[op], g);
            const uint32_t first = u.nsteps < ST ? u.nsteps : ST;
            for (uint32_t it = 0; it < first; it++) {
                mbar_expect_tx(bar_full + 8u * it, u.tx);
                mxg_load_weights(ops[op], u, base + it * stage_b, u.ks_begin + it, bar_full + 8u * it);
            }
            if (grp.pdl != MMB_PDL_OFF)
                grid_dep_launch();
            grid_dep_wait();                                /* also: the launch in front has reset the counter */
            MMB_TRACE_MIN(grp.trace_slot, 1);
            MMB_TRACE_MAX(grp.trace_slot, 2);
            uint32_t s = 0, round = 0, gstep = 0;
            for (;;) {
                /* the number of the unit after this one, asked for now and needed at its end */
                const uint32_t next = grp.sched ? gridDim.x + atomicAdd(grp.sched, 1u) : g + gridDim.x;
                const MxgOp &o = ops[op];
                for (uint32_t it = 0; it < u.nsteps; it++, gstep++, s = (s + 1u == ST) ? 0u : s + 1u, round += (s == 0u)) {
                    const uint32_t st = base + s * stage_b, bar = bar_full + 8u * s;
                    if (gstep >= first) {
                        if (round > 0u)
                            mbar_wait(bar_empty + 8u * s, (round - 1u) & 1u, grp.status);
                        mbar_expect_tx(bar, u.tx);
                        mxg_load_weights(o, u, st, u.ks_begin + it, bar);
                    }
                    mxg_load_planes(o, u, st, u.ks_begin + it, bar);
                }
                push(next);
                if (next >= grp.n_units)
                    break;
                g = next;
                while (op + 1u < grp.n_ops && g >= ops[op + 1u].unit0) op++;
                u = unit_geom(ops[op], g);
            }
            MMB_TRACE_MAX(grp.trace_slot, 9);
            if (grp.sched) {
                /* the CTA that is last to have taken its last number puts the counters back */
                __threadfence();
                if (atomicAdd(grp.sched + 1, 1u) == gridDim.x - 1u) {
                    grp.sched[0] = 0u;
                    grp.sched[1] = 0u;
                    __threadfence();
                }
            }
        }
    } else if (warp == 1 || warp == 10) {
        /* ------------------------------ MMA issue ------------------------------ */
        const uint32_t h = warp == 1 ? 0u : 1u;
        if (lane == 0) {
            UnitWalk w;
            uint32_t s = 0, round = 0, gstep = 0, j = 0;
            for (w.start(q_ids, q_full, q_empty, grp.status); w.valid<false>(grp, ops); w.next(), j++) {
                const MxgOp &o = ops[w.op];
                const UnitGeom u = unit_geom(o, w.g);
                const uint32_t buf = AB == 2u ? (j & 1u) : 0u, use = j / AB;
                if (use >= 1u)                       /* the epilogue has drained this buffer's previous unit */
                    mbar_wait(bar_acc_empty + 8u * buf, (use - 1u) & 1u, grp.status);
                tc_fence_after();
                const uint32_t idesc = umma_idesc_mxf4(u.nb);
                const uint32_t d = tmem + buf * MMB_MXG_ACC_STRIDE + h * u.nb;
                for (uint32_t it = 0; it < u.nsteps; it++, gstep++, s = (s + 1u == ST) ? 0u : s + 1u, round += (s == 0u)) {
                    const uint32_t t = gstep & 1u, st = base + s * stage_b;
                    mbar_wait(bar_full + 8u * s, round & 1u, grp.status);
                    if (gstep == 0u && h == 0u)
                        MMB_TRACE_MIN(grp.trace_slot, 10);
                    if (h < u.halves) {
                        mbar_wait(bar_sf_full + 8u * t, (gstep >> 1) & 1u, grp.status);
                        tc_fence_after();
                        const uint32_t sf = tmem + MMB_MX_SF_COL + t * MMB_MX_SF_SLOT;
                        const uint64_t ad = umma_desc_sw128(st + h * u.h1 * 128u), bd = umma_desc_sw128(st + u.o_pl);
#pragma unroll
                        for (uint32_t q = 0; q < 4u; q++)
                            umma_mxf4(d, ad + 2u * q, bd + 2u * q, idesc, (it | q) ? 1u : 0u,
                                      sf + h * 16u + 4u * q, sf + MMB_MX_SFB_OFF + 8u * q);
                    }
                    umma_commit(bar_empty + 8u * s);
                }
                umma_commit(bar_acc_full + 8u * buf);
            }
        }
    } else if (warp < 10) {
        /* ------------------------------ scale factors --------------------------- */
        const uint32_t quad = warp & 3u;
        const uint32_t mine_t = (warp - 2u) >> 2;
        const uint32_t tq = tmem + ((quad * 32u) << 16);
        UnitWalk w;
        uint32_t s = 0, round = 0, gstep = 0;
        uint32_t s1 = 0, round1 = 0, s2 = 0, round2 = 0;
        for (w.start(q_ids, q_full, q_empty, grp.status); w.valid<true>(grp, ops); w.next()) {
            const MxgOp &o = ops[w.op];
            const UnitGeom u = unit_geom(o, w.g);
            const uint32_t ncol = (u.nb + 31u) >> 5;
            for (uint32_t it = 0; it < u.nsteps; it++, gstep++, s2 = s1, round2 = round1, s1 = s, round1 = round,
                                                s = (s + 1u == ST) ? 0u : s + 1u, round += (s == 0u)) {
                const uint32_t t = gstep & 1u, st = base + s * stage_b;
                if (t != mine_t)
                    continue;
                mbar_wait_warp(bar_full + 8u * s, round & 1u, grp.status);
                if (gstep >= 2u)
                    mbar_wait_warp(bar_empty + 8u * s2, round2 & 1u, grp.status);
                tc_fence_after();
                const uint32_t sf = tq + MMB_MX_SF_COL + t * MMB_MX_SF_SLOT;
                bool patched = false;
                uint32_t v[64];
                uint4 qa[8];
#pragma unroll
                for (uint32_t i = 0; i < 8u; i++) {
                    const uint32_t in_half = 32u * (i & 3u) + lane;
                    qa[i] = make_uint4(0u, 0u, 0u, 0u);
                    if (in_half < ((i >> 2) ? u.cnt1 : u.cnt0))
                        qa[i] = lds128(st + u.o_sc + ((i >> 2) * u.h1 + in_half) * 16u);
                }
                uint32_t negs = 0u;
#pragma unroll
                for (uint32_t i = 0; i < 8u; i++) {
                    const uint32_t wv[4] = { qa[i].x, qa[i].y, qa[i].z, qa[i].w };
#pragma unroll
                    for (uint32_t q = 0; q < 4u; q++) {
                        const uint32_t nan = (((wv[q] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) >> 7;
                        const uint32_t clean = wv[q] & ~(nan * 0xffu);
                        negs |= clean & 0x80808080u;
                        v[(i >> 2) * 16u + 4u * q + (i & 3u)] = clean & 0x7f7f7f7fu;
                    }
                }
                if (__any_sync(0xffffffffu, negs != 0u)) {
                    if (quad == 2u && negs) {
#pragma unroll
                        for (uint32_t i = 0; i < 8u; i++) {
                            const uint32_t r = (i >> 2) * u.h1 + 32u * (i & 3u) + lane;
                            const uint32_t wv[4] = { qa[i].x, qa[i].y, qa[i].z, qa[i].w };
#pragma unroll
                            for (uint32_t q = 0; q < 4u; q++) {
                                const uint32_t nan = (((wv[q] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) >> 7;
                                const uint32_t neg = wv[q] & ~(nan * 0xffu) & 0x80808080u;
                                for (uint32_t b = 0; neg && b < 4u; b++)
                                    if (neg & (0x80u << (8u * b))) {
                                        const uint32_t off = (4u * q + b) * 8u;
                                        const uint32_t a = st + r * 128u + ((((off >> 4) ^ (r & 7u)) << 4) | (off & 15u));
                                        sts32(a, lds32(a) ^ 0x88888888u);
                                        sts32(a + 4u, lds32(a + 4u) ^ 0x88888888u);
                                    }
                            }
                        }
                    }
                    patched = true;
                }
#pragma unroll
                for (uint32_t c = 0; c < 8u; c++) {
                    const uint32_t r = 32u * c + lane;
                    uint4 q = make_uint4(0u, 0u, 0u, 0u);
                    if (c < ncol && r < u.nb)
                        q = lds128(st + u.o_sfb + r * 16u);
                    v[MMB_MX_SFB_OFF + c] = q.x;
                    v[MMB_MX_SFB_OFF + 8u + c] = q.y;
                    v[MMB_MX_SFB_OFF + 16u + c] = q.z;
                    v[MMB_MX_SFB_OFF + 24u + c] = q.w;
                }
                tmem_st_x64(sf, v);
                tmem_st_wait();
                if (patched)
                    fence_proxy_async_smem();
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(bar_sf_full + 8u * t);
            }
        }
    } else {
        /* ------------------------------ epilogue -------------------------------- *
         * Thread = weight row; a unit's accumulators are read while the MMA threads
         * fill the other buffer with the next unit. */
        const uint32_t quad = warp & 3u;
        const uint32_t tq = tmem + ((quad * 32u) << 16);
        const uint32_t lr = quad * 32u + lane;
        const uint32_t etid = tid - 11u * 32u;             /* 0..127 */
        grid_dep_wait();                                    /* row factors come from the kernel in front */
        UnitWalk w;
        uint32_t j = 0;
        for (w.start(q_ids, q_full, q_empty, grp.status); w.valid<true>(grp, ops); w.next(), j++) {
            const MxgOp &o = ops[w.op];
            const UnitGeom u = unit_geom(o, w.g);
            const uint32_t buf = AB == 2u ? (j & 1u) : 0u, use = j / AB;
            const uint32_t groups = u.nb / 24u;
            const bool direct = o.split_k == 1u;
            const bool gate_second = (o.flags & 2u) != 0u;
            const uint32_t pitch = u.glu ? o.tiles * 256u : o.N;
            /* row factors: lane l holds entries l and l + 32 of the [32][2] table */
            const float ra = lane < 2u * o.M ? __ldcg(o.row_scale + lane) : 0.0f;
            const float rb = lane + 32u < 2u * o.M ? __ldcg(o.row_scale + lane + 32u) : 0.0f;
            mbar_wait_warp(bar_acc_full + 8u * buf, use & 1u, grp.status);
            tc_fence_after();
            if (etid == 0u) {
                if (j == 0u) {
                    MMB_TRACE_MIN(grp.trace_slot, 3);
                    MMB_TRACE_MAX(grp.trace_slot, 6);
                }
                MMB_TRACE_MAX(grp.trace_slot, 7);
            }
            const uint32_t d0 = tq + buf * MMB_MXG_ACC_STRIDE;
            float *mine = o.partial + static_cast<size_t>(u.slice) * (groups * 4u) * pitch;
            for (uint32_t g4 = 0; g4 < groups; g4++) {
                uint32_t c0[24], c1[24];
                tmem_ld_x8(d0 + g4 * 24u, *reinterpret_cast<uint32_t (*)[8]>(&c0[0]));
                tmem_ld_x8(d0 + g4 * 24u + 8u, *reinterpret_cast<uint32_t (*)[8]>(&c0[8]));
                tmem_ld_x8(d0 + g4 * 24u + 16u, *reinterpret_cast<uint32_t (*)[8]>(&c0[16]));
                if (u.halves == 2u) {
                    tmem_ld_x8(d0 + u.nb + g4 * 24u, *reinterpret_cast<uint32_t (*)[8]>(&c1[0]));
                    tmem_ld_x8(d0 + u.nb + g4 * 24u + 8u, *reinterpret_cast<uint32_t (*)[8]>(&c1[8]));
                    tmem_ld_x8(d0 + u.nb + g4 * 24u + 16u, *reinterpret_cast<uint32_t (*)[8]>(&c1[16]));
                }
                tmem_ld_wait();
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const uint32_t m = g4 * 4u + r;            /* warp-uniform */
                    if (m >= o.M)
                        break;
                    const uint32_t e = 2u * m;
                    const float f1 = e < 32u ? __shfl_sync(0xffffffffu, ra, e) : __shfl_sync(0xffffffffu, rb, e - 32u);
                    const float f2 = e + 1u < 32u ? __shfl_sync(0xffffffffu, ra, e + 1u)
                                                  : __shfl_sync(0xffffffffu, rb, e - 31u);
                    const float a0 = mx_row_sum(c0, r) * f1 * f2;
                    const float a1 = u.halves == 2u ? mx_row_sum(c1, r) * f1 * f2 : 0.0f;
                    if (u.glu) {
                        const uint32_t n = u.row0 + lr;
                        const bool ok = lr < u.cnt0 && n < o.N;
                        if (direct) {
                            if (ok)
                                mxg_store(o, static_cast<size_t>(m) * o.ldy + o.col0 + n,
                                    glu_out_bf16(gate_second ? a1 : a0, gate_second ? a0 : a1, o.gs, o.gs_up));
                        } else if (ok) {
                            __stcg(mine + static_cast<size_t>(m) * pitch + u.tile * 256u + lr, a0);
                            __stcg(mine + static_cast<size_t>(m) * pitch + u.tile * 256u + 128u + lr, a1);
                        }
                    } else {
#pragma unroll
                        for (uint32_t hh = 0; hh < 2u; hh++) {
                            if (hh >= u.halves)
                                break;
                            const uint32_t n = u.row0 + hh * 128u + lr;
                            const float a = hh ? a1 : a0;
                            if (lr >= (hh ? u.cnt1 : u.cnt0) || n >= o.N)
                                continue;
                            if (direct) {
                                __nv_bfloat16 hv = __float2bfloat16_rn(a * o.gs);
                                mxg_store(o, static_cast<size_t>(m) * o.ldy + o.col0 + n, *reinterpret_cast<uint16_t *>(&hv));
                            } else {
                                __stcg(mine + static_cast<size_t>(m) * pitch + n, a);
                            }
                        }
                    }
                }
            }
            /* the accumulators are in registers or stored: the buffer may be refilled */
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(bar_acc_empty + 8u * buf);
            if (!direct) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid == 0u) {
                    /* release: the partial sums of all 128 threads (ordered before by the barrier);
                     * acquire: the other slices' sums, for the one that arrives last */
                    unsigned ticket;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                                 : "=r"(ticket) : "l"(grp.counters + o.counters_idx + u.tile) : "memory");
                    sts32(last_flag, (ticket == o.split_k - 1u) ? 1u : 0u);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (lds32(last_flag)) {
                    const size_t slice = static_cast<size_t>(groups * 4u) * pitch;
                    /* The last slice to arrive adds the tile's partial sums, slice by slice in
                     * ascending order (the same sums from run to run, and the single-op kernel's).
                     * Four columns per thread and up to sixteen 16-byte loads in flight: with one
                     * column per thread the sums of a 16-row tile in eight slices were eight
                     * dependent round trips to L2, 13 us at the end of every short launch. */
                    bool vec = ((pitch | o.N | o.ldy | o.col0 | u.row0 | u.cnt0 | u.cnt1) & 3u) == 0u;
                    for (uint32_t d = 0; d < o.n_dst; d++)
                        vec = vec && (reinterpret_cast<uintptr_t>(o.y[d]) & 7u) == 0u;
                    if (vec && !u.glu) {
                        const uint32_t cq = etid & 63u, rg = etid >> 6;
                        const uint32_t col = u.row0 + 4u * cq;
                        const bool ok = 4u * cq < u.rows && col < o.N;
                        for (uint32_t m = rg; ok && m < o.M; m += 4u) {
                            float4 sum[2] = { make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f) };
                            const bool two = m + 2u < o.M;
                            for (uint32_t sl0 = 0; sl0 < o.split_k; sl0 += 8u) {
                                float4 v[2][8];
#pragma unroll
                                for (uint32_t q = 0; q < 8u; q++) {
                                    const float *src = o.partial + (sl0 + q) * slice + static_cast<size_t>(m) * pitch + col;
                                    const bool live = sl0 + q < o.split_k;
                                    v[0][q] = live ? __ldcg(reinterpret_cast<const float4 *>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                    v[1][q] = live && two ? __ldcg(reinterpret_cast<const float4 *>(src + 2u * pitch))
                                                          : make_float4(0.f, 0.f, 0.f, 0.f);
                                }
#pragma unroll
                                for (uint32_t q = 0; q < 8u; q++)
#pragma unroll
                                    for (uint32_t r = 0; r < 2u; r++) {
                                        sum[r].x += v[r][q].x; sum[r].y += v[r][q].y;
                                        sum[r].z += v[r][q].z; sum[r].w += v[r][q].w;
                                    }
                            }
                            for (uint32_t r = 0; r < (two ? 2u : 1u); r++) {
                                const uint2 out = make_uint2(pack_bf16x2(sum[r].x * o.gs, sum[r].y * o.gs),
                                                             pack_bf16x2(sum[r].z * o.gs, sum[r].w * o.gs));
                                const size_t off = static_cast<size_t>(m + 2u * r) * o.ldy + o.col0 + col;
                                for (uint32_t d = 0; d < o.n_dst; d++)
                                    *reinterpret_cast<uint2 *>(o.y[d] + off) = out;
                            }
                        }
                    } else if (vec) {
                        /* gated pair: columns [0, 128) of the tile's partial sums are one projection,
                         * [128, 256) the other; 32 column groups x 4 row groups */
                        const uint32_t cq = etid & 31u, rg = etid >> 5;
                        const uint32_t lc = 4u * cq;
                        const bool ok = lc < u.cnt0 && u.row0 + lc < o.N;
                        for (uint32_t m = rg; ok && m < o.M; m += 4u) {
                            float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
                            for (uint32_t sl0 = 0; sl0 < o.split_k; sl0 += 8u) {
                                float4 v0[8], v1[8];
#pragma unroll
                                for (uint32_t q = 0; q < 8u; q++) {
                                    const float *src = o.partial + (sl0 + q) * slice + static_cast<size_t>(m) * pitch +
                                                       u.tile * 256u + lc;
                                    const bool live = sl0 + q < o.split_k;
                                    v0[q] = live ? __ldcg(reinterpret_cast<const float4 *>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                    v1[q] = live ? __ldcg(reinterpret_cast<const float4 *>(src + 128u))
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                                }
#pragma unroll
                                for (uint32_t q = 0; q < 8u; q++) {
                                    s0.x += v0[q].x; s0.y += v0[q].y; s0.z += v0[q].z; s0.w += v0[q].w;
                                    s1.x += v1[q].x; s1.y += v1[q].y; s1.z += v1[q].z; s1.w += v1[q].w;
                                }
                            }
                            const float4 gt = gate_second ? s1 : s0, up = gate_second ? s0 : s1;
                            const uint2 out = make_uint2(glu_out_bf16x2(gt.x, gt.y, up.x, up.y, o.gs, o.gs_up),
                                                         glu_out_bf16x2(gt.z, gt.w, up.z, up.w, o.gs, o.gs_up));
                            const size_t off = static_cast<size_t>(m) * o.ldy + o.col0 + u.row0 + lc;
                            for (uint32_t d = 0; d < o.n_dst; d++)
                                *reinterpret_cast<uint2 *>(o.y[d] + off) = out;
                        }
                    } else {
                        const uint32_t col0 = u.glu ? u.tile * 256u + lr : u.row0 + lr, col1 = col0 + 128u;
                        const bool ok0 = lr < u.cnt0 && u.row0 + lr < o.N;
                        const bool ok1 = u.glu ? ok0 : (lr < u.cnt1 && u.row0 + 128u + lr < o.N);
                        for (uint32_t m0 = 0; m0 < o.M; m0 += 4u) {
                            float s0[4] = { 0.0f, 0.0f, 0.0f, 0.0f }, s1[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
                            for (uint32_t sl0 = 0; sl0 < o.split_k; sl0 += 4u) {
                                float v0[4][4], v1[4][4];
    #pragma unroll
                                for (uint32_t r = 0; r < 4u; r++)
    #pragma unroll
                                    for (uint32_t q = 0; q < 4u; q++) {
                                        const bool live = m0 + r < o.M && sl0 + q < o.split_k;
                                        const float *src = o.partial + (sl0 + q) * slice + static_cast<size_t>(m0 + r) * pitch;
                                        v0[r][q] = live && ok0 ? __ldcg(src + col0) : 0.0f;
                                        v1[r][q] = live && ok1 ? __ldcg(src + col1) : 0.0f;
                                    }
    #pragma unroll
                                for (uint32_t r = 0; r < 4u; r++)
    #pragma unroll
                                    for (uint32_t q = 0; q < 4u; q++) {
                                        s0[r] += v0[r][q];
                                        s1[r] += v1[r][q];
                                    }
                            }
    #pragma unroll
                            for (uint32_t r = 0; r < 4u; r++) {
                                const uint32_t m = m0 + r;
                                if (m >= o.M)
                                    break;
                                if (u.glu) {
                                    if (ok0)
                                        mxg_store(o, static_cast<size_t>(m) * o.ldy + o.col0 + u.row0 + lr,
                                                  glu_out_bf16(gate_second ? s1[r] : s0[r], gate_second ? s0[r] : s1[r],
                                                               o.gs, o.gs_up));
                                } else {
                                    if (ok0) {
                                        __nv_bfloat16 hv = __float2bfloat16_rn(s0[r] * o.gs);
                                        mxg_store(o, static_cast<size_t>(m) * o.ldy + o.col0 + u.row0 + lr,
                                                  *reinterpret_cast<uint16_t *>(&hv));
                                    }
                                    if (ok1) {
                                        __nv_bfloat16 hv = __float2bfloat16_rn(s1[r] * o.gs);
                                        mxg_store(o, static_cast<size_t>(m) * o.ldy + o.col0 + u.row0 + 128u + lr,
                                                  *reinterpret_cast<uint16_t *>(&hv));
                                    }
                                }
                            }
                        }
                    }
                    if (etid == 0u)
                        grp.counters[o.counters_idx + u.tile] = 0u;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");     /* last_flag is reused by the next unit */
            }
        }
        if (lane == 0u) {
            MMB_TRACE_MAX(grp.trace_slot, 4);
            MMB_TRACE_MIN(grp.trace_slot, 8);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512u);
    }
}

/* Digit planes of every distinct activation tensor of a group, one launch:
 * blockIdx.z picks the tensor. */
struct XsliceItem {
    const uint16_t *x;
    uint8_t        *scratch;
    uint32_t        M, K, m_pad, nb;
};
struct XsliceGroup {
    uint32_t   n, pdl;
#ifdef MMB_MEASURE_MODES
    uint32_t   trace_slot;
#endif
    XsliceItem item[MMB_MXG_MAX_OPS];
    uint32_t   row0[MMB_MXG_MAX_OPS + 1];      /* first padded row of each tensor in the launch; [n] = all rows */
};

/* Two passes, so that a row is read twice and not once per chunk: chunk maxima,
 * then the slicing with the row maximum taken from them. */
__global__ void __launch_bounds__(256)
f4_xamax_group_kernel(const __grid_constant__ XsliceGroup g)
{
    grid_dep_launch();
    if (g.pdl != MMB_PDL_OFF)
        grid_dep_wait();                     /* the activations are the previous kernel's output */
    const XsliceItem &it = g.item[blockIdx.z];
    if (blockIdx.y >= it.m_pad || blockIdx.x * 1024u >= it.K)
        return;
    xamax_cta(it.x, reinterpret_cast<uint32_t *>(it.scratch + MMB_MX_CHUNKMAX_OFF), it.M, it.K, blockIdx.y,
              blockIdx.x);
}

__global__ void __launch_bounds__(256)
f4_xslice_group_kernel(const __grid_constant__ XsliceGroup g)
{
    grid_dep_launch();
    if (g.pdl != MMB_PDL_OFF)
        grid_dep_wait();
    const XsliceItem &it = g.item[blockIdx.z];
    if (blockIdx.y >= it.m_pad || blockIdx.x * 1024u >= it.K)
        return;
    uint8_t *planes = it.scratch + MMB_MX_PLANES_OFF;
    const bool two_pass = (it.K + 1023u) / 1024u <= MMB_MX_MAX_CHUNKS;
    xslice_cta(it.x, planes, planes + MMB_MX_PLANES_B(it.nb, it.K),
               reinterpret_cast<float *>(it.scratch + MMB_MX_ROWSCALE_OFF), it.M, it.K, blockIdx.y, blockIdx.x,
               two_pass ? reinterpret_cast<const uint32_t *>(it.scratch + MMB_MX_CHUNKMAX_OFF) : nullptr);
}

__device__ __forceinline__ uint32_t xslice_trace_slot(const XsliceGroup &g)
{
#ifdef MMB_MEASURE_MODES
    return g.trace_slot;
#else
    (void)g;
    return 0u;
#endif
}

/* One launch, one pass over the activations: a cluster of eight CTAs per (padded)
 * activation row, 4096 values per CTA, one 16-wide block per thread.  Each CTA
 * leaves the largest magnitude of its part in its shared memory; after a cluster
 * barrier every CTA reads the eight values through distributed shared memory and
 * slices its blocks.  Rows up to 32768 long; longer ones take the two-pass kernels. */
#define MMB_XS_CLUSTER 8u
#define MMB_XS_CTA_VALUES 4096u

__global__ void __cluster_dims__(MMB_XS_CLUSTER, 1, 1) __launch_bounds__(256)
f4_xslice_cluster_kernel(const __grid_constant__ XsliceGroup g)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ uint32_t s_warp[8];
    __shared__ uint32_t s_part;                  /* this CTA's maximum, read by the whole cluster */
    const uint32_t slot = xslice_trace_slot(g);
    if (threadIdx.x == 0) {
        MMB_TRACE_MIN(slot, 0);
        MMB_TRACE_MAX(slot, 5);
        MMB_TRACE_KIND(slot, 2ull);
    }
    grid_dep_launch();
    if (g.pdl != MMB_PDL_OFF)
        grid_dep_wait();                         /* the activations are the previous kernel's output */
    if (threadIdx.x == 0) {
        MMB_TRACE_MIN(slot, 1);
        MMB_TRACE_MAX(slot, 2);
    }
    const uint32_t row = blockIdx.x / MMB_XS_CLUSTER, part = blockIdx.x % MMB_XS_CLUSTER;
    uint32_t i = 0;
    while (i + 1u < g.n && row >= g.row0[i + 1u]) i++;
    const XsliceItem &it = g.item[i];
    const uint32_t m = row - g.row0[i], tid = threadIdx.x;
    const uint32_t blk = part * (MMB_XS_CTA_VALUES / 16u) + tid, blocks = it.K / 16u;
    const bool in_row = blk < blocks, loaded = in_row && m < it.M;
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; j++) w[j] = 0u;
    if (loaded) {
        const uint4 *src = reinterpret_cast<const uint4 *>(it.x + static_cast<size_t>(m) * it.K) + 2u * blk;
        const uint4 a = __ldcg(src), b = __ldcg(src + 1);
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    }
    uint32_t amax = 0;
#pragma unroll
    for (int j = 0; j < 8; j++)
        amax = max(amax, max(w[j] & 0x7fffu, (w[j] >> 16) & 0x7fffu));
    amax = __reduce_max_sync(0xffffffffu, amax);
    if ((tid & 31u) == 0)
        s_warp[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int j = 1; j < 8; j++) amax = max(amax, s_warp[j]);
        s_part = amax;
        MMB_TRACE_MIN(slot, 3);
        MMB_TRACE_MAX(slot, 6);
    }
    cluster.sync();                              /* every part's maximum is in place */
    if (tid == 0)
        MMB_TRACE_MAX(slot, 7);
    uint32_t row_amax = 0;
#pragma unroll
    for (uint32_t r = 0; r < MMB_XS_CLUSTER; r++)
        row_amax = max(row_amax, *cluster.map_shared_rank(&s_part, r));
    /* nobody leaves while its shared memory is still read.  (Writing the maxima into all
     * eight CTAs' shared memory instead, with one barrier, made this kernel 1.7 us shorter
     * and the steps that run it between dependent group launches 3 to 5 % longer.) */
    cluster.sync();
    if (tid == 0)
        MMB_TRACE_MAX(slot, 9);
    const RowFrame f = row_frame(row_amax);
    uint8_t *planes = it.scratch + MMB_MX_PLANES_OFF;
    if (part == 0 && tid == 0 && m < it.M)
        row_factors(f, reinterpret_cast<float *>(it.scratch + MMB_MX_ROWSCALE_OFF), m);
    if (in_row)
        xslice_block(w, f, loaded, planes, planes + MMB_MX_PLANES_B(it.nb, it.K), it.K, m, blk);
#ifdef MMB_MEASURE_MODES
    if (tid == 0)
        MMB_TRACE_MAX(slot, 11);                 /* thread 0's own block sliced */
    __syncthreads();
    if (tid == 0) {
        MMB_TRACE_MAX(slot, 4);
        MMB_TRACE_MIN(slot, 10);
    }
#endif
}
} // namespace mmb

#ifdef MMB_MEASURE_MODES
static uint32_t g_trace_next;       /* rows handed out since the last reset */
/* All rows back to "nothing recorded": minima at the largest value, maxima at zero. */
extern "C" int mmb_trace_reset(void)
{
    static unsigned long long init[MMB_TRACE_SLOTS][16];
    for (uint32_t i = 0; i < MMB_TRACE_SLOTS; i++)
        for (uint32_t k = 0; k < 16u; k++)
            init[i][k] = (k == 0u || k == 1u || k == 3u || k == 8u || k == 10u) ? ~0ull : 0ull;
    g_trace_next = 0;
    return static_cast<int>(cudaMemcpyToSymbol(mmb::g_trace, init, sizeof init));
}
/* Minima and maxima are kept across replays of a captured launch: reset the values, keep the rows. */
extern "C" int mmb_trace_clear(void)
{
    const uint32_t keep = g_trace_next;
    const int e = mmb_trace_reset();
    g_trace_next = keep;
    return e;
}
extern "C" int mmb_trace_read(unsigned long long *out, uint32_t *rows_out)
{
    *rows_out = g_trace_next;
    return static_cast<int>(cudaMemcpyFromSymbol(out, mmb::g_trace, sizeof(unsigned long long) * 16u * MMB_TRACE_SLOTS));
}
static uint32_t trace_take(void) { return g_trace_next < MMB_TRACE_SLOTS ? ++g_trace_next : 0u; }
#endif

extern "C" int mmb_mxg_init(void)
{
    cudaError_t e = cudaFuncSetAttribute(mmb::f4_mxg_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMB_SMEM_MAX);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(mmb::f4_mxg_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMB_SMEM_MAX);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(mmb::f4_mxg_kernel<12>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMB_SMEM_MAX);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(mmb::f4_mxg_kernel<MMB_MXG_MAX_OPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 MMB_SMEM_MAX);
    return static_cast<int>(e);
}

/* Digit planes of one activation tensor with the cluster kernel; -1 when the rows
 * are too long for it (the caller then uses its own kernel). */
extern "C" int mmb_launch_xslice_rows(const void *x, void *scratch, uint32_t M, uint32_t K, uint32_t nb, int pdl,
                                      void *stream)
{
    if (K > MMB_XS_CLUSTER * MMB_XS_CTA_VALUES)
        return -1;
    static mmb::XsliceGroup xs;
    memset(&xs, 0, sizeof xs);
    xs.n = 1;
    xs.pdl = static_cast<uint32_t>(pdl);
#ifdef MMB_MEASURE_MODES
    xs.trace_slot = trace_take();
#endif
    xs.item[0].x = static_cast<const uint16_t *>(x);
    xs.item[0].scratch = static_cast<uint8_t *>(scratch);
    xs.item[0].M = M; xs.item[0].K = K; xs.item[0].nb = nb; xs.item[0].m_pad = nb / MMB_MX_PLANES;
    xs.row0[1] = xs.item[0].m_pad;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(xs.row0[1] * MMB_XS_CLUSTER);
    cfg.blockDim = dim3(256);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, mmb::f4_xslice_cluster_kernel, xs));
}

extern "C" int mmb_launch_mxg(const mmb_group *hg, void *stream, uint32_t *kernels_launched)
{
    uint32_t launched = 0;
    static mmb::MxgParams<MMB_MXG_MAX_OPS> prm;   /* built in place: 30 KB is too much for the stack of a small thread */
    mmb::MxgGroup &grp = prm.grp;
    static mmb::XsliceGroup xs;
    unsigned *status = nullptr;
    int e = mmb_status_word(&status);
    if (e) return e;
    if (hg->n_ops == 0 || hg->n_ops > MMB_MXG_MAX_OPS)
        return static_cast<int>(cudaErrorInvalidValue);
    memset(&prm, 0, sizeof prm);
    memset(&xs, 0, sizeof xs);
    grp.n_ops = hg->n_ops; grp.n_units = hg->n_units; grp.stages = hg->stages; grp.acc_bufs = hg->acc_bufs;
    grp.stage_b = hg->stage_b; grp.pdl = static_cast<uint32_t>(hg->pdl); grp.status = status;
    grp.sched = static_cast<unsigned *>(hg->sched);
    grp.counters = static_cast<unsigned *>(hg->counters);
    uint32_t max_m = 0, max_kx = 0, max_k = 0;
    for (uint32_t i = 0; i < hg->n_ops; i++) {
        const mmb_gop &s = hg->op[i];
        mmb::MxgOp &d = prm.ops[i];
        memcpy(d.tm_payload.bytes, s.tm_payload, 128);
        memcpy(d.tm_scale.bytes, s.tm_scale, 128);
        memcpy(d.tm_planes.bytes, s.tm_planes, 128);
        memcpy(d.tm_sfb.bytes, s.tm_sfb, 128);
        d.y[0] = static_cast<uint16_t *>(s.y);
        d.n_dst = 1; d.ldy = s.N; d.col0 = 0;
        if (s.n_dst) {
            for (uint32_t k = 0; k < s.n_dst && k < MMB_MAX_PEERS; k++) d.y[k] = static_cast<uint16_t *>(s.y_dst[k]);
            d.n_dst = static_cast<uint8_t>(s.n_dst); d.ldy = s.ldy; d.col0 = s.col0;
        }
        d.row_scale = reinterpret_cast<const float *>(static_cast<const unsigned char *>(s.x_ws) + MMB_MX_ROWSCALE_OFF);
        d.partial = static_cast<float *>(s.partial);
        d.counters_idx = s.counters_idx;
        d.gs = s.gs; d.gs_up = s.gs_up;
        d.M = s.M; d.N = s.N;
        d.rows = static_cast<uint16_t>(s.rows); d.nb = static_cast<uint16_t>(s.nb); d.k_steps = s.k_steps;
        d.split_k = static_cast<uint16_t>(s.split_k); d.tiles = s.tiles;
        d.unit0 = s.unit0;
        d.flags = static_cast<uint8_t>((s.glu ? 1u : 0u) | (s.gate_plane ? 2u : 0u));
        if (s.slice_here) {
            mmb::XsliceItem &it = xs.item[xs.n];
            it.x = static_cast<const uint16_t *>(s.x);
            it.scratch = static_cast<uint8_t *>(s.x_ws);
            it.M = s.M; it.K = s.K; it.nb = s.nb; it.m_pad = s.nb / MMB_MX_PLANES;
            xs.row0[xs.n + 1u] = xs.row0[xs.n] + it.m_pad;
            xs.n++;
            if (it.m_pad > max_m) max_m = it.m_pad;
            if ((s.K + 1023u) / 1024u > max_kx) max_kx = (s.K + 1023u) / 1024u;
            if (s.K > max_k) max_k = s.K;
        }
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = hg->pdl ? 1 : 0;
    if (xs.n) {
        xs.pdl = static_cast<uint32_t>(hg->pdl);
#ifdef MMB_MEASURE_MODES
        xs.trace_slot = trace_take();
#endif
        cudaLaunchConfig_t cfg = {};
        cfg.blockDim = dim3(256);
        cfg.stream = st;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t err;
        if (max_k <= MMB_XS_CLUSTER * MMB_XS_CTA_VALUES) {
            cfg.gridDim = dim3(xs.row0[xs.n] * MMB_XS_CLUSTER);
            err = cudaLaunchKernelEx(&cfg, mmb::f4_xslice_cluster_kernel, xs);
            launched = 1;
        } else {
            cfg.gridDim = dim3(max_kx, max_m, xs.n);
            err = cudaLaunchKernelEx(&cfg, mmb::f4_xamax_group_kernel, xs);
            if (err == cudaSuccess)
                err = cudaLaunchKernelEx(&cfg, mmb::f4_xslice_group_kernel, xs);
            launched = 2;
        }
        if (err != cudaSuccess)
            return static_cast<int>(err);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(hg->grid);
    cfg.blockDim = dim3(MMB_MXG_THREADS);
    cfg.dynamicSmemBytes = hg->smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute gattr[2];
    gattr[0] = attr[0];
    cfg.attrs = gattr;
    cfg.numAttrs = 1;
    if (hg->l2_base && hg->l2_bytes) {
        /* the scratch every tile re-reads (digit planes, split-K partials) is kept in L2 in
         * preference to the weights, which stream through once (the reference commits such
         * windows with its graphs, src/cuda/cuda_rt.c:163-181) */
        gattr[1].id = cudaLaunchAttributeAccessPolicyWindow;
        gattr[1].val.accessPolicyWindow.base_ptr = hg->l2_base;
        gattr[1].val.accessPolicyWindow.num_bytes = hg->l2_bytes;
        gattr[1].val.accessPolicyWindow.hitRatio = 1.0f;
        gattr[1].val.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
        gattr[1].val.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
        cfg.numAttrs = 2;
    }
#ifdef MMB_MEASURE_MODES
    grp.trace_slot = trace_take();
#endif
    if (kernels_launched)
        *kernels_launched = launched + 1u;
    /* the smallest parameter block that holds the ops (its leading bytes are the larger one's) */
    if (hg->n_ops <= 1u)
        return static_cast<int>(cudaLaunchKernelEx(&cfg, mmb::f4_mxg_kernel<1>,
                                                   *reinterpret_cast<const mmb::MxgParams<1> *>(&prm)));
    if (hg->n_ops <= 4u)
        return static_cast<int>(cudaLaunchKernelEx(&cfg, mmb::f4_mxg_kernel<4>,
                                                   *reinterpret_cast<const mmb::MxgParams<4> *>(&prm)));
    if (hg->n_ops <= 12u)
        return static_cast<int>(cudaLaunchKernelEx(&cfg, mmb::f4_mxg_kernel<12>,
                                                   *reinterpret_cast<const mmb::MxgParams<12> *>(&prm)));
    return static_cast<int>(cudaLaunchKernelEx(&cfg, mmb::f4_mxg_kernel<MMB_MXG_MAX_OPS>, prm));
}
