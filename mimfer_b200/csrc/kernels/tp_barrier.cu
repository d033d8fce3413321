/*
 * Cross-rank barrier of the tensor-parallel linear, as one small kernel on the
 * compute stream.
 *
 * The fused tensor-parallel op (mm_f4_linear_tp) stores every output tile into
 * all ranks' copies of y; before any rank reads its copy, every rank's kernels
 * must have finished.  Each rank owns a block of flags in memory its peers can
 * write (one 32-bit slot per peer, plus its own epoch counter).  A launch takes
 * the next epoch, fences, writes that epoch into its slot of every rank's block
 * (release, system scope), then waits until every slot of its own block has
 * reached the epoch (acquire, system scope).  Epochs only grow, so a peer that
 * is already one barrier ahead does no harm, and the kernel takes no argument
 * that changes between launches: it can sit in a captured graph.
 *
 * The wait is bounded like every other wait of this library: after about two
 * seconds it raises MMB_DEV_TIMEOUT in the status word and returns, so a rank
 * that never arrives costs its peers two seconds and an error code, not a hung
 * GPU.  Ranks must therefore reach a barrier within that time of each other:
 * meet on the host first wherever set-up work (loading weights, capturing a
 * graph) can take longer on one rank than on another.  The reference is single-GPU and has no counterpart.
 */
#include "ptx.cuh"

namespace mmb {

struct TpBarrierParams {
    unsigned *flags[MMB_MAX_PEERS];   /* flags[r]: rank r's block, MMB_TPB_WORDS words */
    unsigned *status;
    uint32_t  n_ranks, rank;
};

__global__ void __launch_bounds__(32, 1) tp_barrier_kernel(const TpBarrierParams p)
{
    __shared__ unsigned epoch_s;
    const uint32_t tid = threadIdx.x;
    unsigned *mine = p.flags[p.rank];
    if (tid == 0)
        epoch_s = mine[MMB_TPB_EPOCH] + 1u;          /* only this rank's launches touch the word */
    __syncwarp();
    const unsigned epoch = epoch_s;
    if (tid < p.n_ranks) {
        __threadfence_system();                      /* this rank's earlier stores, peers' copies included */
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[tid] + p.rank), "r"(epoch) : "memory");
        const uint64_t t0 = globaltimer_ns();
        for (uint32_t spin = 1;; spin++) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + tid) : "memory");
            if (static_cast<int>(v - epoch) >= 0)
                break;
            if ((spin & 63u) == 0) {
                if (*reinterpret_cast<volatile unsigned *>(p.status) & MMB_DEV_TIMEOUT)
                    break;
                if (globaltimer_ns() - t0 > 2000000000ull) {      /* ranks drift more than pipeline stages do */
                    atomicOr(p.status, MMB_DEV_TIMEOUT);
                    break;
                }
            }
        }
        __threadfence_system();
    }
    __syncwarp();
    if (tid == 0)
        mine[MMB_TPB_EPOCH] = epoch;
}

} // namespace mmb

extern "C" int mmb_launch_tp_barrier(unsigned *const *flags, uint32_t n_ranks, uint32_t rank, void *stream)
{
    unsigned *status = nullptr;
    int e = mmb_status_word(&status);
    if (e) return e;
    mmb::TpBarrierParams p;
    for (uint32_t r = 0; r < MMB_MAX_PEERS; r++) p.flags[r] = r < n_ranks ? flags[r] : nullptr;
    p.status = status;
    p.n_ranks = n_ranks;
    p.rank = rank;
    mmb::tp_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return static_cast<int>(cudaGetLastError());
}
