/*
 * Upload of several small host buffers with one kernel.
 *
 * A decode step brings a few hundred KB of activations up from pinned host
 * memory, as many buffers as the step has ops.  As copy nodes of a graph they
 * cost several microseconds each whatever their size, one after the other on
 * the copy engine, and the first kernel of the step waits for them.  This
 * kernel reads the pinned buffers over PCIe itself (they are mapped into the
 * device's address space) and writes the ops' device operands: one node, all
 * buffers in flight together.  It stands in for the per-buffer mm_h2d_async
 * calls of the reference engine's round (src/engine/engine.c:233-357) inside
 * the op-list engine's captured step; buffers that are not mapped or not
 * 16-byte aligned are left to the copy engine.
 */
#include <cstdint>
#include <cuda_runtime.h>
#include "launch.h"

namespace mmb {

struct GatherList {
    const uint4 *src[MMB_GATHER_MAX];    /* device-side addresses of pinned host buffers */
    uint4       *dst[MMB_GATHER_MAX];
    uint32_t     n16[MMB_GATHER_MAX];    /* 16-byte units */
    uint32_t     count;
};

__global__ void __launch_bounds__(256) host_gather_kernel(const __grid_constant__ GatherList l)
{
    const uint32_t e = blockIdx.y;
    if (e >= l.count)
        return;
    const uint4 *__restrict__ src = l.src[e];
    uint4 *__restrict__ dst = l.dst[e];
    const uint32_t n = l.n16[e], stride = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __ldcs(src + i);         /* read once: no reason to keep host lines in cache */
}

} // namespace mmb

/* Returns 0 when the kernel was enqueued for all n buffers, -1 when some buffer
 * cannot be reached by the device this way (nothing enqueued: use copies), else
 * a cudaError_t.  to_host: the host side is the destination (download). */
static int launch_copy_list(const void *const *src, void *const *dst, const size_t *bytes, uint32_t n,
                            bool to_host, void *stream)
{
    if (n == 0)
        return 0;
    if (n > MMB_GATHER_MAX)
        return -1;
    mmb::GatherList l;
    l.count = n;
    uint32_t longest = 0;
    for (uint32_t i = 0; i < n; i++) {
        void *dptr = nullptr;
        void *host = to_host ? dst[i] : const_cast<void *>(src[i]);
        if ((reinterpret_cast<uintptr_t>(src[i]) & 15u) || (reinterpret_cast<uintptr_t>(dst[i]) & 15u) ||
            (bytes[i] & 15u) || bytes[i] > (static_cast<size_t>(1) << 35))
            return -1;
        if (cudaHostGetDevicePointer(&dptr, host, 0) != cudaSuccess || !dptr) {
            (void)cudaGetLastError();
            return -1;
        }
        l.src[i] = static_cast<const uint4 *>(to_host ? src[i] : dptr);
        l.dst[i] = static_cast<uint4 *>(to_host ? dptr : dst[i]);
        l.n16[i] = static_cast<uint32_t>(bytes[i] >> 4);
        if (l.n16[i] > longest) longest = l.n16[i];
    }
    uint32_t bx = (longest + 255u) / 256u;
    if (bx > 16u) bx = 16u;                    /* 4096 transfers of 16 bytes in flight per buffer */
    if (bx < 1u) bx = 1u;
    mmb::host_gather_kernel<<<dim3(bx, n), 256, 0, static_cast<cudaStream_t>(stream)>>>(l);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int mmb_launch_host_gather(const void *const *src_host, void *const *dst_dev,
                                      const size_t *bytes, uint32_t n, void *stream)
{
    return launch_copy_list(src_host, dst_dev, bytes, n, false, stream);
}

/* The other direction: the step's outputs written into pinned host buffers by one
 * kernel (posted writes over PCIe) instead of one copy node per output. */
extern "C" int mmb_launch_host_scatter(const void *const *src_dev, void *const *dst_host,
                                       const size_t *bytes, uint32_t n, void *stream)
{
    return launch_copy_list(src_dev, dst_host, bytes, n, true, stream);
}
