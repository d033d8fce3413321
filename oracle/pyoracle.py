"""ctypes access to the two CPU checkers (test infrastructure only).

  Oracle     oracle/liboracle.so          plain-C restatement (oracle/nvfp4_oracle.c)
  Reference  oracle/_ref/libmimfer_ref.so the reference's own kx_op_gemm_f4, compiled
                                          from its sources (oracle/build.py)
Arrays are numpy: x uint16 [M][K] (bf16 bits), payload uint8 [N][K/2],
scales uint8 [N][K/16], y uint16 [M][N].
"""
import ctypes as C
import os

import numpy as np

from . import build as _build


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class Oracle:
    def __init__(self):
        self.lib = C.CDLL(_build.build_oracle())
        self.lib.orc_gemm_f4_block.restype = C.c_int
        self.lib.orc_gemm_f4_block.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p,
                                               C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                               C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]
        self.lib.orc_decode_table.argtypes = [C.c_void_p]
        self.lib.orc_e2m1_decode.restype = C.c_float
        self.lib.orc_e2m1_decode.argtypes = [C.c_uint]
        self.lib.orc_e4m3_decode.restype = C.c_float
        self.lib.orc_e4m3_decode.argtypes = [C.c_ubyte]
        self.lib.orc_bf16_from_f32.restype = C.c_uint16
        self.lib.orc_bf16_from_f32.argtypes = [C.c_float]
        self.lib.orc_silu_mul.restype = None
        self.lib.orc_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        self.lib.orc_add_rmsnorm.restype = None
        self.lib.orc_add_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_uint32, C.c_uint32, C.c_float]

    def add_rmsnorm(self, res, delta, gain, eps):
        """bf16 bit patterns [M][H], [M][H], [H]; returns (res + delta, normalised output)."""
        res = np.array(res, np.uint16, copy=True, order="C")
        delta = np.ascontiguousarray(delta, np.uint16)
        gain = np.ascontiguousarray(gain, np.uint16)
        y = np.empty(res.shape, np.uint16)
        self.lib.orc_add_rmsnorm(_p(res), _p(delta), _p(y), _p(gain), res.shape[0], res.shape[1], eps)
        return res, y

    def silu_mul(self, gate, up):
        """bf16 bit patterns in, bf16 bit patterns out, same shape."""
        gate = np.ascontiguousarray(gate, np.uint16)
        up = np.ascontiguousarray(up, np.uint16)
        y = np.empty(gate.shape, np.uint16)
        self.lib.orc_silu_mul(_p(gate), _p(up), _p(y), gate.size)
        return y

    def mlp_gate_up(self, x, w_gate, w_up, threads=None):
        """The MLP front half as the reference planner runs it (src/plan/plan.c:223-247):
        two GEMMs stored as bf16, then SILU_MUL.  w_*: objects with payload, scales, gs."""
        g = self.gemm_f4(x, w_gate.payload, w_gate.scales, w_gate.gs, threads=threads)
        u = self.gemm_f4(x, w_up.payload, w_up.scales, w_up.gs, threads=threads)
        return self.silu_mul(g, u)

    def decode_table(self):
        t = np.empty(4096, np.uint32)
        self.lib.orc_decode_table(_p(t))
        return t

    def gemm_f4(self, x, payload, scales, gs=1.0, rows=None, n_begin=0, n_end=None,
                want_acc=False, threads=None):
        """y (and optionally the fp32 accumulators) for activation rows `rows`
        (default all) and output features [n_begin, n_end)."""
        M, K = x.shape
        N = payload.shape[0]
        n_end = N if n_end is None else n_end
        x = np.ascontiguousarray(x, np.uint16)
        payload = np.ascontiguousarray(payload, np.uint8)
        scales = np.ascontiguousarray(scales, np.uint8)
        if rows is None:
            idx, n_m, idx_p = None, M, None
        else:
            idx = np.ascontiguousarray(rows, np.uint32)
            n_m, idx_p = len(idx), _p(idx)
        y = np.empty((n_m, n_end - n_begin), np.uint16)
        acc = np.empty((n_m, n_end - n_begin), np.float32) if want_acc else None
        rc = self.lib.orc_gemm_f4_block(_p(x), _p(payload), _p(scales), gs, _p(y),
                                        _p(acc) if want_acc else None, M, K, N, idx_p, n_m,
                                        n_begin, n_end, threads or host_threads())
        if rc:
            raise ValueError(f"oracle rejected the shape (status {rc})")
        return (y, acc) if want_acc else y


class Reference:
    """The compiled reference kernel; `available` is False when neither the
    reference tree nor a prebuilt library is present."""

    def __init__(self):
        path = _build.build_ref()
        self.available = bool(path) and os.path.exists(path)
        if not self.available:
            return
        self.lib = C.CDLL(path)
        self.lib.ref_silu_mul.restype = C.c_int
        self.lib.ref_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32]
        self.lib.ref_add_rmsnorm.restype = C.c_int
        self.lib.ref_add_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_uint32, C.c_uint32, C.c_float]
        for name, extra in (("ref_gemm_f4", []), ("ref_gemm_f4_mt", [C.c_int])):
            fn = getattr(self.lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                           C.c_uint32, C.c_uint32, C.c_uint32] + extra

    def silu_mul(self, gate, up):
        gate = np.ascontiguousarray(gate, np.uint16)
        up = np.ascontiguousarray(up, np.uint16)
        y = np.empty(gate.shape, np.uint16)
        rc = self.lib.ref_silu_mul(_p(gate), _p(up), _p(y), gate.size)
        return rc, y

    def add_rmsnorm(self, res, delta, gain, eps):
        res = np.array(res, np.uint16, copy=True, order="C")
        delta = np.ascontiguousarray(delta, np.uint16)
        gain = np.ascontiguousarray(gain, np.uint16)
        y = np.empty(res.shape, np.uint16)
        rc = self.lib.ref_add_rmsnorm(_p(res), _p(delta), _p(y), _p(gain), res.shape[0], res.shape[1], eps)
        return rc, res, y

    def gemm_f4(self, x, payload, scales, threads=1):
        M, K = x.shape
        N = payload.shape[0]
        x = np.ascontiguousarray(x, np.uint16)
        payload = np.ascontiguousarray(payload, np.uint8)
        scales = np.ascontiguousarray(scales, np.uint8)
        y = np.empty((M, N), np.uint16)
        if threads <= 1:
            rc = self.lib.ref_gemm_f4(_p(x), _p(payload), _p(scales), _p(y), M, K, N)
        else:
            rc = self.lib.ref_gemm_f4_mt(_p(x), _p(payload), _p(scales), _p(y), M, K, N, threads)
        return rc, y
