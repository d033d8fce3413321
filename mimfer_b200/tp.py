"""Tensor-parallel NVFP4 linear: output features sharded across ranks.

Rank p of tp owns weight rows [p*N/tp, (p+1)*N/tp).  Payload and block scales
are row-major by output feature (include/mimfer/tensor.h:17-19 in the mimfer
tree), so a shard is a contiguous byte range of each buffer and no 16-wide
scale group is ever split.  Activations are replicated.  Each rank computes
y[:, shard] with the single-GPU op, then the slices are all-gathered (NCCL over
NVLink; gloo on CPU in the tests) into [tp][M][N/tp] and laid out as [M][N].

mode="fused" removes the separate exchange: every rank's full output lives in
symmetric memory, and the kernel's epilogue stores each finished tile into all
ranks' copies through peer-mapped pointers (stores and bulk copies over NVLink, no
multicast), so the transfer overlaps the remaining tiles; one cross-rank barrier
kernel of this library (a bounded device-side spin on flags in symmetric memory)
on the stream closes the op.  The full outputs are double-buffered: call i of a
linear writes buffer i % 2 on every rank, so a rank that runs ahead into the next
step never overwrites an output a slower rank is still reading - it cannot reach
the step after that before the slower rank has arrived at the barrier in between,
which that rank enqueues after its reads.

mode="push" is for prefill sizes, where a rank's output slice is hundreds of
megabytes: the kernel stores into the rank's own copy only, chunk of rows by chunk
of rows, and the copy engines push every finished chunk to the peers
(mm_f4_tp_push) while the SMs multiply the next one; a join and the same barrier
kernel close the op.  Measured, the copy engines carry 757 GB/s to one peer but
425 GB/s per GPU when four ranks push to three peers each, less than the epilogue's
stores (617 GB/s), so "fused" is the faster form from four ranks on and the bench
times both.  The reference has no multi-GPU path; this is new surface.
"""
import ctypes as C
import os

# The kernels write to peers with unicast stores and bulk copies: the symmetric buffers need no NVLink
# multicast binding, and a rank that dies while bound to one disturbs the other GPUs.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

from . import _lib as L
import torch
import torch.distributed as dist


def shard_bounds(N, rank, world):
    if N % world != 0:
        raise ValueError(f"N={N} is not divisible by the tensor-parallel degree {world}")
    per = N // world
    return rank * per, (rank + 1) * per


def push_chunks(M, rows):
    """(row0, rows) of the chunks of a pushed linear: `rows` at a time; a last chunk of a
    multiple of 512 rows is halved while more than 512 rows are left, so that the push
    nothing overlaps is a short one (8192 rows by 1024: ..., 1024, 512, 512)."""
    out, r0 = [], 0
    while M - r0 > rows:
        out.append((r0, rows))
        r0 += rows
    left = M - r0
    while left > 512 and left % 512 == 0:
        out.append((r0, left // 2))
        r0 += left // 2
        left -= left // 2
    out.append((r0, left))
    return out


class TpBarrier:
    """Cross-rank barrier on the runtime's compute stream (mm_f4_tp_barrier): a
    64-byte flag block per rank in symmetric memory, one small kernel per call,
    a bounded wait.  One instance per process group, shared by its linears."""

    _by_group = {}

    def __init__(self, rt, rank, world, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.rt, self.rank, self.world = rt, rank, world
        g = group if group is not None else dist.group.WORLD
        self.flags = symm_mem.empty((16,), dtype=torch.int32, device=rt.device)
        self.flags.zero_()
        self.hdl = symm_mem.rendezvous(self.flags, g)
        self.ptrs = (C.c_void_p * world)(*[self.hdl.buffer_ptrs[r] for r in range(world)])
        torch.cuda.synchronize()
        dist.barrier(group=group)             # every block is zero before anyone signals

    @classmethod
    def get(cls, rt, rank, world, group=None):
        key = id(group) if group is not None else 0
        if key not in cls._by_group:
            cls._by_group[key] = cls(rt, rank, world, group)
        return cls._by_group[key]

    def sync(self):
        L.check(self.rt.lib.mm_f4_tp_barrier(self.ptrs, self.world, self.rank, None), "mm_f4_tp_barrier")


class TpLinear:
    """`local_op(x, w_shard, y_shard)` computes the shard; by default it is the
    CUDA op enqueued on the runtime's compute stream."""

    def __init__(self, weight, rank, world, rt=None, group=None, local_op=None, mode="gather", push_rows=1024):
        if mode not in ("gather", "fused", "push"):
            raise ValueError(mode)
        if push_rows <= 0:
            raise ValueError("push_rows")
        self.rank, self.world, self.group, self.rt = rank, world, group, rt
        self.push_rows = push_rows
        self.mode = mode if world > 1 else "gather"
        self._symm = {}
        self.N, self.K = weight.N, weight.K
        n0, n1 = shard_bounds(weight.N, rank, world)
        self.shard = weight.rows(n0, n1)
        self.local_op = local_op
        if local_op is None:
            if rt is None:
                raise RuntimeError("TpLinear without a local_op needs the CUDA runtime")
            self.shard.to_device(rt.device)
            self.local_op = lambda x, w, y: rt.linear_async(x, w, y)
        self._bufs = {}

    def _buffers(self, M, like):
        if M not in self._bufs:
            ns = self.N // self.world
            kw = dict(dtype=like.dtype, device=like.device)
            if self.world == 1:
                self._bufs[M] = (torch.empty((M, ns), **kw), None, None)
            else:
                self._bufs[M] = (torch.empty((M, ns), **kw), torch.empty((self.world, M, ns), **kw),
                                 torch.empty((M, self.N), **kw))
        return self._bufs[M]

    def _symm_buffers(self, M, like):
        """Full output in symmetric memory + the pointer table (own copy first): two
        sets per M, taken in turn by successive calls (every rank makes the same calls)."""
        if M not in self._symm:
            import torch.distributed._symmetric_memory as symm_mem
            sets = []
            for _ in range(2):
                y = symm_mem.empty((M, self.N), dtype=like.dtype, device=like.device)
                hdl = symm_mem.rendezvous(y, self.group if self.group is not None else dist.group.WORLD)
                order = [self.rank] + [r for r in range(self.world) if r != self.rank]
                ptrs = (C.c_void_p * self.world)(*[hdl.buffer_ptrs[r] for r in order])
                sets.append((y, hdl, ptrs))
            self._symm[M] = [sets, 0]
        entry = self._symm[M]
        chosen = entry[0][entry[1] % 2]
        entry[1] += 1
        return chosen

    def barrier(self):
        """Cross-rank barrier on the compute stream: after it, every rank's copy of
        every output written since the previous barrier is complete.  Needed once
        per group of fused forwards issued with barrier=False."""
        if self.mode not in ("fused", "push"):
            return
        if self.mode == "push":                 # the copy engines' work joins the compute stream first
            L.check(self.rt.lib.mm_f4_tp_push_join(), "mm_f4_tp_push_join")
        TpBarrier.get(self.rt, self.rank, self.world, self.group).sync()

    def _forward_fused(self, x, barrier=True):
        M = x.shape[0]
        y, hdl, ptrs = self._symm_buffers(M, x)
        n0 = self.rank * (self.N // self.world)
        w = self.shard
        L.check(self.rt.lib.mm_f4_linear_tp(x.data_ptr(), w.dev_payload.data_ptr(),
                                            w.dev_scales.data_ptr(), w.gs, ptrs, self.world,
                                            self.N, n0, M, w.K, w.N, None), "mm_f4_linear_tp")
        if barrier:
            self.barrier()                      # every rank's stores have landed everywhere
        return y

    def _forward_push(self, x, barrier=True):
        """Row chunks of push_rows: the chunk's GEMM into the own copy, then its push to the
        peers; the compute stream never waits for a push before the closing join.  The last
        chunk is halved (push_chunks) so that little of the exchange is left when the
        multiplying ends."""
        M = x.shape[0]
        y, hdl, ptrs = self._symm_buffers(M, x)
        ns = self.N // self.world
        n0 = self.rank * ns
        w, K = self.shard, self.shard.K
        own = (C.c_void_p * 1)()
        for r0, rows in push_chunks(M, self.push_rows):
            own[0] = ptrs[0] + r0 * self.N * 2
            L.check(self.rt.lib.mm_f4_linear_tp(x.data_ptr() + r0 * K * 2, w.dev_payload.data_ptr(),
                                                w.dev_scales.data_ptr(), w.gs, own, 1, self.N, n0, rows, K, w.N,
                                                None), "mm_f4_linear_tp")
            L.check(self.rt.lib.mm_f4_tp_push(ptrs, self.world, self.N, n0, ns, r0, rows), "mm_f4_tp_push")
        if barrier:
            self.barrier()
        return y

    def forward(self, x, barrier=True):
        """x: [M][K] replicated.  Returns y [M][N], complete on every rank.
        On CUDA everything is enqueued on the runtime's compute stream.
        barrier=False (fused mode) leaves the closing cross-rank barrier to the
        caller, so several linears of one step can share a single barrier()."""
        if self.mode == "fused":
            return self._forward_fused(x, barrier)
        if self.mode == "push":
            return self._forward_push(x, barrier)
        M = x.shape[0]
        y_local, gathered, y = self._buffers(M, x)
        if self.world == 1:                       # nothing to exchange
            if self.rt is not None and x.is_cuda:
                with torch.cuda.stream(self.rt.torch_stream()):
                    self.local_op(x, self.shard, y_local)
            else:
                self.local_op(x, self.shard, y_local)
            return y_local
        if self.rt is not None and x.is_cuda:
            with torch.cuda.stream(self.rt.torch_stream()):
                self.local_op(x, self.shard, y_local)
                self._gather(y_local, gathered, y, M)
        else:
            self.local_op(x, self.shard, y_local)
            self._gather(y_local, gathered, y, M)
        return y

    def _gather(self, y_local, gathered, y, M):
        dist.all_gather_into_tensor(gathered.view(-1), y_local.view(-1), group=self.group)
        if M == 1:
            y.view(-1).copy_(gathered.view(-1))
        else:
            ns = self.N // self.world
            y.view(M, self.world, ns).copy_(gathered.permute(1, 0, 2))


class TpStep:
    """The tensor-parallel linears of one step as ONE CUDA graph per rank.

    A decode step at tp=8 is a few tens of microseconds of kernel time per
    rank; issued op by op from Python, the launches and the barrier cost more
    than that on the host.  This captures `lins[i].forward(xs[i])` for every
    i plus the closing cross-rank barrier on the runtime's compute stream and
    replays them with one launch.  Fused mode only when there is more than one
    rank (the kernels' peer stores and one barrier kernel; no NCCL call is
    captured).  Two graphs are captured, one per set of output buffers, and
    replayed in turn, so that consecutive steps never write the same buffers.
    The activations are read from the same device tensors `xs` on every replay:
    refill them in place.  Outputs: what replay() returns, complete on every
    rank once the replay has finished and valid until the replay after the next."""

    def __init__(self, lins, xs):
        if len(lins) != len(xs) or not lins:
            raise ValueError("one activation tensor per linear")
        self.lins, self.xs = list(lins), list(xs)
        self.rt = lins[0].rt
        if self.rt is None:
            raise RuntimeError("TpStep needs the CUDA runtime")
        if any(lin.world > 1 and lin.mode != "fused" for lin in lins):
            raise NotImplementedError("TpStep captures fused-mode linears; gather mode issues its "
                                      "NCCL all-gather op by op")
        self.stream = self.rt.torch_stream()
        self._issue()                         # eager once: buffers, symmetric-memory rendezvous
        self.rt.sync()
        if dist.is_initialized() and lins[0].world > 1:
            dist.barrier(group=lins[0].group)
        torch.cuda.synchronize()
        self.graphs, self.outs, self.n_replays = [], [], 0
        for _ in range(2):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream, capture_error_mode="thread_local"):
                ys = self._issue()
            self.graphs.append(g)
            self.outs.append(ys)
        self.ys = self.outs[0]
        if dist.is_initialized() and lins[0].world > 1:
            dist.barrier(group=lins[0].group)     # the barrier kernel's wait is bounded: replay together
        torch.cuda.synchronize()

    def _issue(self):
        ys = [lin.forward(x, barrier=False) for lin, x in zip(self.lins, self.xs)]
        self.lins[-1].barrier()
        return ys

    def replay(self):
        k = self.n_replays % 2
        self.n_replays += 1
        with torch.cuda.stream(self.stream):
            self.graphs[k].replay()
        self.ys = self.outs[k]
        return self.ys


class TpGroupStep:
    """Several tensor-parallel DECODE linears of one step as one group launch per rank.

    Every linear is sharded along N like TpLinear; the rank's shards go into the
    op-list engine with mm_lin_engine_add_tp, so the whole step is one slicing kernel
    and one persistent launch of the block-scaled kernel whose epilogue stores every
    output tile into all ranks' copies, followed by the library's barrier kernel.
    Outputs are double-buffered like TpLinear's: two engines, captured once each,
    replayed in turn.  The activations are read from the same device tensors `xs` on
    every replay: refill them in place."""

    def __init__(self, weights, xs, rank, world, rt, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        from .linear import LinearEngine
        if len(weights) != len(xs) or not weights:
            raise ValueError("one activation tensor per linear")
        self.rank, self.world, self.rt, self.group = rank, world, rt, group
        self.xs = list(xs)
        self.shards, self.col0 = [], []
        for w in weights:
            n0, n1 = shard_bounds(w.N, rank, world)
            self.shards.append(w.rows(n0, n1).to_device(rt.device))
            self.col0.append(n0)
        g = group if group is not None else (dist.group.WORLD if world > 1 else None)
        self.outs, self.engines, self._keep = [], [], []
        for _ in range(2):
            ys, eng = [], LinearEngine(rt, max_ops=len(weights) + 1)
            for w, x, sh, c0 in zip(weights, self.xs, self.shards, self.col0):
                M = x.shape[0]
                if world > 1:
                    y = symm_mem.empty((M, w.N), dtype=x.dtype, device=x.device)
                    hdl = symm_mem.rendezvous(y, g)
                    order = [rank] + [r for r in range(world) if r != rank]
                    ptrs = (C.c_void_p * world)(*[hdl.buffer_ptrs[r] for r in order])
                    self._keep.append(hdl)
                else:
                    y = torch.empty((M, w.N), dtype=x.dtype, device=x.device)
                    ptrs = (C.c_void_p * 1)(y.data_ptr())
                eng.add_tp(x, sh, y, ptrs, world, c0)
                ys.append(y)
            eng.launch()                          # direct dispatch once: errors surface per op
            rt.sync()
            eng.capture()
            self.outs.append(ys)
            self.engines.append(eng)
        self.barrier = TpBarrier.get(rt, rank, world, group) if world > 1 else None
        if world > 1:
            dist.barrier(group=group)             # every rank holds its buffers before anyone stores
        torch.cuda.synchronize()
        self.n_replays = 0

    def replay(self):
        k = self.n_replays % 2
        self.n_replays += 1
        self.engines[k].launch()
        if self.barrier is not None:
            self.barrier.sync()
        return self.outs[k]

    def close(self):
        for e in self.engines:
            e.close()
        self.engines, self.outs, self._keep = [], [], []
