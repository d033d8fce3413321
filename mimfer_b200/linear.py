"""Host-side mirror of the operator interface for the NVFP4 linear op.

Names follow the mimfer tree: a weight is a payload + block-scale pair
(mm_wt, include/mimfer/tensor.h:121-126), an op is an mm_op_desc dispatched
through mm_kx_invoke / kx_op_gemm_f4 (include/mimfer/kernels.h:73-113).
"""
import ctypes as C

import numpy as np

from . import _lib as L


def weight_bytes(N, K):
    """Packed bytes of one weight: payload + block scales (+ 4 for the global scale)."""
    return N * K // 2 + N * K // 16 + 4


class NvFp4Weight:
    """payload [N][K/2] u8, scales [N][K/16] u8 (e4m3), fp32 global scale."""

    def __init__(self, payload, scales, gs, N, K):
        self.payload, self.scales, self.gs, self.N, self.K = payload, scales, float(gs), N, K
        self.dev_payload = self.dev_scales = None

    def rows(self, n0, n1):
        """Contiguous shard of output features [n0, n1) (tensor parallelism)."""
        return NvFp4Weight(self.payload[n0:n1], self.scales[n0:n1], self.gs, n1 - n0, self.K)

    def to_device(self, device="cuda"):
        import torch
        self.dev_payload = torch.from_numpy(np.ascontiguousarray(self.payload)).to(device)
        self.dev_scales = torch.from_numpy(np.ascontiguousarray(self.scales)).to(device)
        L.check(L.lib().mm_f4_gscale_set(self.dev_scales.data_ptr(), self.gs), "mm_f4_gscale_set")
        return self


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def place_weights(weights, device="cuda"):
    """Stage several weights into ONE device block, in order, each tensor as
    [payload | block scales] on 256-byte boundaries - the way mimfer's weight
    arena is filled (bump allocation in load order, src/model/tensor_registry.c:532-560).
    Tensors placed together keep a fixed address order, which the fused
    gate/up kernel needs.  Returns the block (keep it alive)."""
    import torch
    offs, total = [], 0
    for w in weights:
        po = total
        so = po + (w.payload.size + 255) // 256 * 256
        total = so + (w.scales.size + 255) // 256 * 256
        offs.append((po, so))
    host = np.zeros(total, np.uint8)
    for w, (po, so) in zip(weights, offs):
        host[po:po + w.payload.size] = w.payload.reshape(-1)
        host[so:so + w.scales.size] = w.scales.reshape(-1)
    block = torch.from_numpy(host).to(device)
    for w, (po, so) in zip(weights, offs):
        w.dev_payload = block[po:po + w.payload.size].view(w.N, w.K // 2)
        w.dev_scales = block[so:so + w.scales.size].view(w.N, w.K // 16)
        L.check(L.lib().mm_f4_gscale_set(w.dev_scales.data_ptr(), w.gs), "mm_f4_gscale_set")
    return block


def pack_weight(W):
    """Quantise fp32 W [N][K] with the library's packer."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    N, K = W.shape
    payload = np.empty((N, K // 2), np.uint8)
    scales = np.empty((N, K // 16), np.uint8)
    gs = C.c_float()
    L.check(L.lib().mm_f4_pack(_ptr(W), N, K, _ptr(payload), _ptr(scales), C.byref(gs)), "mm_f4_pack")
    return NvFp4Weight(payload, scales, gs.value, N, K)


def make_weight(N, K, seed=0, std=0.02):
    """Seeded N(0, std) weight, generated and packed row by row."""
    payload = np.empty((N, K // 2), np.uint8)
    scales = np.empty((N, K // 16), np.uint8)
    gs = C.c_float()
    L.check(L.lib().mm_f4_make_weight(N, K, seed, std, _ptr(payload), _ptr(scales), C.byref(gs)),
            "mm_f4_make_weight")
    return NvFp4Weight(payload, scales, gs.value, N, K)


def fill_normal(rows, cols, seed, mean=0.0, std=1.0):
    out = np.empty((rows, cols), np.float32)
    L.lib().mm_fill_normal_f32(_ptr(out), rows, cols, seed, mean, std)
    return out


def f32_to_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, np.uint16)
    L.lib().mm_f32_to_bf16(_ptr(a), _ptr(out), a.size)
    return out


def bf16_to_f32(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, np.float32)
    L.lib().mm_bf16_to_f32(_ptr(a), _ptr(out), a.size)
    return out


def make_activations(M, K, seed=1, std=1.0):
    """Seeded N(0, std) activations rounded to bf16; returned as uint16 bit patterns [M][K]."""
    return f32_to_bf16(fill_normal(M, K, seed, 0.0, std))


def select_plan(M, K, N, sm_count=148, ptr_align=256, ws_bytes=0, variant=None, glu=False):
    """glu=True: plan of the fused gate/up kernel, N = output features."""
    shape = L.F4Shape(M, K, N, sm_count, ptr_align, ws_bytes)
    plan = L.F4Plan()
    if glu:
        st = L.lib().mm_f4_select_glu(C.byref(shape), C.byref(plan))
    elif variant is None:
        st = L.lib().mm_f4_select(C.byref(shape), C.byref(plan))
    else:
        st = L.lib().mm_f4_select_variant(C.byref(shape), variant, C.byref(plan))
    L.check(st, "mm_f4_select")
    return plan


class Runtime:
    """Process-wide runtime: device, streams, split-K workspace (donated once)."""

    _instance = None

    def __init__(self, device=0, workspace_bytes=256 << 20):
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("mimfer_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.torch = torch
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.lib = L.lib()
        L.check(self.lib.mm_cuda_init(device), "mm_cuda_init")
        self.workspace = torch.zeros(workspace_bytes, dtype=torch.uint8, device=self.device)
        torch.cuda.synchronize()
        L.check(self.lib.mm_f4_workspace_set(self.workspace.data_ptr(), workspace_bytes),
                "mm_f4_workspace_set")
        self.sync()

    @classmethod
    def get(cls, device=0):
        if cls._instance is None:
            cls._instance = cls(device)
        return cls._instance

    # -- plumbing -----------------------------------------------------------
    def sync(self):
        L.check(self.lib.mm_stream_sync(L.MM_ST_COMPUTE), "mm_stream_sync")

    def stream_ptr(self):
        return self.lib.mm_cuda_stream_raw(L.MM_ST_COMPUTE)

    def torch_stream(self):
        return self.torch.cuda.ExternalStream(self.stream_ptr(), device=self.device)

    def device_status(self):
        flags = C.c_uint()
        L.check(self.lib.mm_f4_device_status(C.byref(flags)), "mm_f4_device_status")
        return flags.value

    def to_device_bf16(self, bits):
        """uint16 bf16 bit patterns (numpy) -> torch.bfloat16 tensor on the device."""
        t = self.torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(self.device)
        return t.view(self.torch.bfloat16)

    def from_device_bf16(self, t):
        return t.view(self.torch.int16).cpu().numpy().view(np.uint16)

    # -- the op -------------------------------------------------------------
    def op_desc(self, x, w, y, M=None, op=L.OP_GEMM_F4, note=b"gemm_f4"):
        M = x.shape[0] if M is None else M
        d = L.MmOpDesc()
        d.op, d.layer = op, -1
        d.a, d.b, d.c, d.d = x.data_ptr(), w.dev_payload.data_ptr(), y.data_ptr(), w.dev_scales.data_ptr()
        d.n0, d.n1, d.n2 = M, w.K, w.N
        d.note = note
        return d

    def gemm_f4(self, x, w, y=None, variant=None):
        """Dispatch one OP_GEMM_F4 through mm_kx_invoke (synchronises, like the
        reference launcher outside capture).  x: bf16 [M][K] device tensor."""
        M = x.shape[0]
        if y is None:
            y = self.torch.empty((M, w.N), dtype=self.torch.bfloat16, device=self.device)
        d = self.op_desc(x, w, y)
        kc = L.MmKcall(C.pointer(d), C.c_void_p(1), None)
        self.lib.mm_f4_force_variant(-1 if variant is None else variant)
        try:
            L.check(self.lib.mm_kx_invoke(C.byref(kc)), "mm_kx_invoke(OP_GEMM_F4)")
        finally:
            self.lib.mm_f4_force_variant(-1)
        return y

    def linear_async(self, x, w, y, M=None):
        """Enqueue on the compute stream without synchronising."""
        M = x.shape[0] if M is None else M
        L.check(self.lib.mm_f4_linear(x.data_ptr(), w.dev_payload.data_ptr(), w.dev_scales.data_ptr(),
                                      w.gs, y.data_ptr(), M, w.K, w.N, None), "mm_f4_linear")

    def mlp_gate_up_async(self, x, w_gate, w_up, y, M=None):
        """y[M][inter] = silu(x . Wgate^T) * (x . Wup^T) in one kernel (mm_f4_mlp_gate_up);
        enqueue only."""
        M = x.shape[0] if M is None else M
        L.check(self.lib.mm_f4_mlp_gate_up(x.data_ptr(), w_gate.dev_payload.data_ptr(),
                                           w_gate.dev_scales.data_ptr(), w_gate.gs,
                                           w_up.dev_payload.data_ptr(), w_up.dev_scales.data_ptr(),
                                           w_up.gs, y.data_ptr(), M, w_gate.K, w_gate.N, None),
                "mm_f4_mlp_gate_up")

    def silu_mul_async(self, gate, up, y):
        L.check(self.lib.mm_silu_mul(gate.data_ptr(), up.data_ptr(), y.data_ptr(), gate.numel(), None),
                "mm_silu_mul")

    def linear_host(self, x_host, x_dev, w, y_dev, y_host):
        """Host buffers in, host buffers out (pinned torch tensors)."""
        M = x_host.shape[0]
        L.check(self.lib.mm_f4_linear_host(x_host.data_ptr(), x_dev.data_ptr(), w.dev_payload.data_ptr(),
                                           w.dev_scales.data_ptr(), w.gs, y_dev.data_ptr(),
                                           y_host.data_ptr(), M, w.K, w.N), "mm_f4_linear_host")

    def time_begin(self):
        L.check(self.lib.mm_time_begin(), "mm_time_begin")

    def time_end(self):
        ms = C.c_float()
        L.check(self.lib.mm_time_end(C.byref(ms)), "mm_time_end")
        return ms.value

    def decode_probe(self):
        """(bf16 operand form, fp32 form, fp16 operand form), each 4096 fp32 bit patterns."""
        out = self.torch.zeros((3, 4096), dtype=self.torch.int32, device=self.device)
        self.torch.cuda.synchronize()
        L.check(self.lib.mm_f4_decode_probe(out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr()),
                "mm_f4_decode_probe")
        a = out.cpu().numpy().view(np.uint32)
        return a[0], a[1], a[2]


class LinearEngine:
    """Sequence of linear ops, optionally captured into one CUDA graph."""

    def __init__(self, rt, max_ops=1200):
        self.rt = rt
        self.h = C.c_void_p()
        L.check(rt.lib.mm_lin_engine_create(C.byref(self.h), max_ops), "mm_lin_engine_create")
        self._keep = []

    def add(self, x, w, y, M=None, op=L.OP_GEMM_F4, note=b"gemm_f4"):
        d = self.rt.op_desc(x, w, y, M, op, note)
        self._keep.append((x, w, y))
        L.check(self.rt.lib.mm_lin_engine_add(self.h, C.byref(d)), "mm_lin_engine_add")

    def add_tp(self, x, w_shard, y_full, ptrs, n_ranks, col0):
        """A tensor-parallel linear: w_shard's output features go to columns
        [col0, col0 + w_shard.N) of every rank's copy of y_full ([M][ldy]); ptrs: ctypes array
        of the n_ranks base pointers, this rank's own (y_full) first."""
        d = self.rt.op_desc(x, w_shard, y_full, None, L.OP_GEMM_F4, b"gemm_f4_tp")
        self._keep.append((x, w_shard, y_full, ptrs))
        L.check(self.rt.lib.mm_lin_engine_add_tp(self.h, C.byref(d), ptrs, n_ranks, y_full.shape[1], col0),
                "mm_lin_engine_add_tp")

    def add_silu_mul(self, gate, up, y):
        """OP_SILU_MUL over gate/up [M][inter] (src/plan/plan.c:240-241)."""
        d = L.MmOpDesc()
        d.op, d.layer = L.OP_SILU_MUL, -1
        d.a, d.b, d.c, d.d = gate.data_ptr(), up.data_ptr(), y.data_ptr(), None
        d.n0, d.n1, d.n2 = gate.shape[0], gate.shape[1], 0
        d.note = b"silu(gate)*up"
        self._keep.append((gate, up, y))
        L.check(self.rt.lib.mm_lin_engine_add(self.h, C.byref(d)), "mm_lin_engine_add")

    def add_add_rmsnorm(self, res, delta, y, gain):
        """OP_ADD_RMSNORM: res += delta in place, y = rmsnorm(res) * gain (src/plan/plan.c:446-447)."""
        d = L.MmOpDesc()
        d.op, d.layer = L.OP_ADD_RMSNORM, -1
        d.a, d.b, d.c, d.d = res.data_ptr(), delta.data_ptr(), y.data_ptr(), gain.data_ptr()
        d.n0, d.n1, d.n2 = res.shape[0], res.shape[1], 0
        d.note = b"add_rmsnorm"
        self._keep.append((res, delta, y, gain))
        L.check(self.rt.lib.mm_lin_engine_add(self.h, C.byref(d)), "mm_lin_engine_add")

    def overlap(self, on=True):
        """Dependency-aware launch order (mm_lin_engine_overlap): 1 = bits of the serial
        order, 2 = run-ahead ops may also take a shallower K split."""
        L.check(self.rt.lib.mm_lin_engine_overlap(self.h, int(on)), "mm_lin_engine_overlap")

    def group(self, on=True):
        """Runs of independent decode linears as one persistent launch (mm_lin_engine_group)."""
        L.check(self.rt.lib.mm_lin_engine_group(self.h, int(on)), "mm_lin_engine_group")

    def n_group_launches(self):
        return self.rt.lib.mm_lin_engine_n_group_launches(self.h)

    def n_independent(self):
        return self.rt.lib.mm_lin_engine_n_independent(self.h)

    def fuse_mlp(self, on=True):
        L.check(self.rt.lib.mm_lin_engine_fuse_mlp(self.h, int(on)), "mm_lin_engine_fuse_mlp")

    def capture(self):
        L.check(self.rt.lib.mm_lin_engine_capture(self.h), "mm_lin_engine_capture")

    def launch(self):
        L.check(self.rt.lib.mm_lin_engine_launch(self.h), "mm_lin_engine_launch")

    def launch_host(self, x_host, y_host):
        """One step with pinned host tensors: x_host[i] -> op i's activations,
        op i's output -> y_host[i] (None entries are skipped); synchronises."""
        n = self.n_ops()
        xs = (C.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in x_host])
        ys = (C.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in y_host])
        L.check(self.rt.lib.mm_lin_engine_launch_host(self.h, xs, ys), "mm_lin_engine_launch_host")

    def bind_host(self, x_host, y_host):
        """Bind pinned host tensors (None entries are skipped) before capture():
        the copies become nodes of the captured graph (mm_lin_engine_bind_host)."""
        n = self.n_ops()
        xs = (C.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in x_host])
        ys = (C.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in y_host])
        self._keep.append((x_host, y_host))
        L.check(self.rt.lib.mm_lin_engine_bind_host(self.h, xs, ys), "mm_lin_engine_bind_host")

    def upload_group(self, ops_per_event):
        L.check(self.rt.lib.mm_lin_engine_upload_group(self.h, ops_per_event), "mm_lin_engine_upload_group")

    def upload_kernel(self, on=True):
        L.check(self.rt.lib.mm_lin_engine_upload_kernel(self.h, int(on)), "mm_lin_engine_upload_kernel")

    def step_bound(self):
        """Replay the graph captured with bound host buffers; synchronises."""
        L.check(self.rt.lib.mm_lin_engine_step_bound(self.h), "mm_lin_engine_step_bound")

    def n_ops(self):
        return self.rt.lib.mm_lin_engine_n_ops(self.h)

    def close(self):
        if self.h:
            self.rt.lib.mm_lin_engine_destroy(self.h)
            self.h = C.c_void_p()
