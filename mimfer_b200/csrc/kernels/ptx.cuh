/*
 * Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor,
 * never with cluster multicast), tcgen05 (alloc, mma, commit, ld) and the
 * warp-level bf16 MMA.  Every wait is bounded: after about one second of
 * polling it sets MMB_DEV_TIMEOUT in the device status word (passed to the kernel) and returns, so a
 * lost signal ends the kernel with an error instead of hanging the GPU.
 */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "launch.h"

namespace mmb {

struct __align__(64) TmaDesc { unsigned char bytes[128]; };

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

/* ---- mbarrier ----------------------------------------------------------- */
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
/* Bounded wait.  Returns false on timeout, after raising MMB_DEV_TIMEOUT in the
 * status word; once that bit is up every later wait in the grid gives up at
 * once, so a broken hand-off costs about one second in total, not per wait. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned *status)
{
    if (mbar_try(bar, parity))
        return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try(bar, parity))
            return true;
        if ((spin & 31u) == 0) {
            if (*reinterpret_cast<volatile unsigned *>(status) & MMB_DEV_TIMEOUT)
                return false;
            if (globaltimer_ns() - t0 > 1000000000ull) {
                atomicOr(status, MMB_DEV_TIMEOUT);
                return false;
            }
        }
    }
}

/* Wait executed by every lane of the calling warp.  (Electing one poller and
 * re-converging with __syncwarp was measured 3-4 % slower on the decode
 * kernels: the reconvergence costs more than 32 lanes polling a completed
 * barrier.) */
__device__ __forceinline__ void mbar_wait_warp(uint32_t bar, uint32_t parity, unsigned *status)
{
    mbar_wait(bar, parity, status);
}

/* ---- TMA (2-D tiled loads, completion on an mbarrier) -------------------- */
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const TmaDesc *map, int x, int y,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const TmaDesc *map, int x, int y, int z,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
/* ---- bulk copies shared -> global (no tensor map): 16-byte aligned both sides, a
 * multiple of 16 bytes; completion is tracked per thread in bulk groups ---------------- */
__device__ __forceinline__ void bulk_store(void *dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
/* all but the newest `KEEP` groups of this thread have read their shared-memory source */
template <int KEEP>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(KEEP) : "memory"); }
/* every group of this thread is complete (the data is written) */
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tma_prefetch_desc(const TmaDesc *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

/* ---- programmatic dependent launch ---------------------------------------
 * A kernel launched with the programmatic-serialization attribute may start
 * while its predecessor in the stream is still draining.  grid_dep_wait()
 * blocks until the predecessor has completed and its writes are visible; work
 * that does not depend on it (weight prefetch) goes before the wait.
 * grid_dep_launch() tells the scheduler that this CTA no longer minds the
 * successor's CTAs being placed. */
__device__ __forceinline__ void grid_dep_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dep_launch()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

/* ---- shared-memory accessors --------------------------------------------- */
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a)
{
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v)
{
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

/* ---- warp-level bf16 MMA (decode path) ------------------------------------ */
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* ---- tcgen05 / TMEM (prefill path) ---------------------------------------- */
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
/* D[tmem] (+)= A[smem] * B[smem]^T, bf16 in, fp32 accumulate, one CTA. */
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
/* Arrive on an mbarrier once all MMAs issued so far by this thread are done. */
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

/* Shared-memory matrix descriptor: K-major operand rows of 128 bytes with the
 * 128-byte swizzle; 8-row groups are 1024 bytes apart. */
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);         /* start address   */
    d |= static_cast<uint64_t>(1) << 16;                             /* LBO (unused)    */
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                     /* SBO             */
    d |= static_cast<uint64_t>(1) << 46;                             /* descriptor v1   */
    d |= static_cast<uint64_t>(2) << 61;                             /* SWIZZLE_128B    */
    return d;
}
/* Instruction descriptor for kind::f16: bf16 x bf16 -> fp32, both operands
 * K-major.  (Both operands must have the same format: fp16 weights against
 * bf16 activations raise an illegal-instruction fault on B200.) */
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t m, uint32_t n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

} // namespace mmb
