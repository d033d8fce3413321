"""ctypes binding of libmimfer_b200.so.

The library must exist (python -m mimfer_b200.build): there is no Python or
CPU stand-in for the kernels, and loading fails loudly without it.
"""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MIMFER_B200_LIB", os.path.join(PKG, "libmimfer_b200.so"))

MM_OK = 0
STATUS_NAMES = ["MM_OK", "MM_ERR_NOMEM", "MM_ERR_IO", "MM_ERR_CORRUPT", "MM_ERR_SHAPE",
                "MM_ERR_CUDA", "MM_ERR_DEVICE", "MM_ERR_UNSUPPORTED", "MM_ERR_RANGE",
                "MM_ERR_STATE", "MM_ERR_BUSY", "MM_ERR_TIMEOUT", "MM_ERR_CAPACITY", "MM_ERR_EOF"]
(MM_ERR_NOMEM, MM_ERR_IO, MM_ERR_CORRUPT, MM_ERR_SHAPE, MM_ERR_CUDA, MM_ERR_DEVICE,
 MM_ERR_UNSUPPORTED, MM_ERR_RANGE, MM_ERR_STATE, MM_ERR_BUSY, MM_ERR_TIMEOUT,
 MM_ERR_CAPACITY, MM_ERR_EOF) = range(1, 14)

OP_LMHEAD, OP_ADD_RMSNORM, OP_GEMM_F4, OP_GEMM_BF16, OP_QKV, OP_SILU_MUL, OP_NOP = 1, 3, 4, 5, 6, 12, 18
MM_ST_COMPUTE, MM_ST_XFER = 0, 1
V_ROWWARP, V_STREAM, V_UMMA, V_MX = 0, 1, 2, 4


class MmOpDesc(C.Structure):
    """mm_op_desc (include/mimfer_abi.h)."""
    _fields_ = [("op", C.c_int), ("layer", C.c_int), ("a", C.c_void_p), ("b", C.c_void_p),
                ("c", C.c_void_p), ("d", C.c_void_p), ("n0", C.c_uint32), ("n1", C.c_uint32),
                ("n2", C.c_uint32), ("note", C.c_char * 24)]


class MmKcall(C.Structure):
    _fields_ = [("op", C.POINTER(MmOpDesc)), ("e", C.c_void_p), ("stream", C.c_void_p)]


class MmWt(C.Structure):
    _fields_ = [("data", C.c_void_p), ("scale", C.c_void_p), ("rows", C.c_uint32), ("cols", C.c_uint32)]


class F4Went(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("rows", C.c_uint32), ("cols", C.c_uint32),
                ("dtype", C.c_uint8), ("off", C.c_uint64), ("nbytes", C.c_uint64)]


MM_DT_BF16, MM_DT_FP4E2M1 = 4, 5


class F4Shape(C.Structure):
    _fields_ = [("M", C.c_uint32), ("K", C.c_uint32), ("N", C.c_uint32), ("sm_count", C.c_uint32),
                ("ptr_align", C.c_uint32), ("ws_bytes", C.c_size_t)]


class F4Plan(C.Structure):
    _fields_ = [("variant", C.c_int), ("m_tiles", C.c_uint32), ("tile_m", C.c_uint32),
                ("tile_n", C.c_uint32), ("split_k", C.c_uint32), ("k_steps", C.c_uint32),
                ("stages", C.c_uint32), ("grid_x", C.c_uint32), ("grid_y", C.c_uint32),
                ("grid_z", C.c_uint32), ("threads", C.c_uint32), ("smem_bytes", C.c_uint32),
                ("ws_needed", C.c_size_t)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class MimferError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{what}: {name}")


# every exported entry point declared in include/mimfer_b200.h: name -> (restype, argtypes)
_u32, _vp, _sz, _f = C.c_uint32, C.c_void_p, C.c_size_t, C.c_float
SIGNATURES = {
    "kx_op_gemm_f4": (C.c_int, [C.POINTER(MmKcall)]),
    "kx_op_qkv": (C.c_int, [C.POINTER(MmKcall)]),
    "mm_kx_invoke": (C.c_int, [C.POINTER(MmKcall)]),
    "kx_cuda_oppref": (C.c_int, [C.c_int]),
    "mm_cuda_enabled": (C.c_int, []),
    "mm_cuda_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "mm_cuda_init": (C.c_int, [C.c_int]),
    "mm_cuda_shutdown": (C.c_int, []),
    "mm_cuda_stream_raw": (_vp, [C.c_int]),
    "mm_cuda_capturing": (C.c_int, []),
    "mm_stream_sync": (C.c_int, [C.c_int]),
    "mm_h2d_async": (C.c_int, [_vp, _vp, _sz, C.c_int]),
    "mm_d2h_async": (C.c_int, [_vp, _vp, _sz, C.c_int]),
    "mm_mset_async": (C.c_int, [_vp, C.c_int, _sz, C.c_int]),
    "mm_graph_create": (C.c_int, [C.POINTER(_vp)]),
    "mm_graph_capture_begin": (C.c_int, [_vp]),
    "mm_graph_commit": (C.c_int, [_vp, _vp, _sz, C.c_int]),
    "mm_graph_launch": (C.c_int, [_vp, C.c_int]),
    "mm_graph_destroy": (None, [_vp]),
    "mm_log_set_level": (None, [C.c_int]),
    "mm_status_str": (C.c_char_p, [C.c_int]),
    "mm_f4_gscale_set": (C.c_int, [_vp, _f]),
    "mm_f4_gscale_get": (_f, [_vp]),
    "mm_f4_gscale_unset": (None, [_vp]),
    "mm_f4_gscale_room": (C.c_uint32, []),
    "mm_f4_gscale_clear": (None, []),
    "mm_f4_workspace_set": (C.c_int, [_vp, _sz]),
    "mm_f4_workspace_bytes": (_sz, []),
    "mm_f4_select": (C.c_int, [C.POINTER(F4Shape), C.POINTER(F4Plan)]),
    "mm_f4_tensor_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32]),
    "mm_f4_weights_parse": (C.c_int, [_vp, C.c_size_t, C.POINTER(F4Went), C.c_uint32,
                                      C.POINTER(C.c_uint32)]),
    "mm_f4_weights_arena_bytes": (C.c_size_t, [C.POINTER(F4Went), C.c_uint32]),
    "mm_f4_weights_stage": (C.c_int, [_vp, C.c_size_t, _vp, C.c_size_t, C.POINTER(_vp)]),
    "mm_f4_weights_count": (C.c_uint32, [_vp]),
    "mm_f4_weights_used": (C.c_size_t, [_vp]),
    "mm_f4_weights_find": (C.c_int, [_vp, C.c_char_p, C.POINTER(MmWt), C.POINTER(C.c_float)]),
    "mm_f4_weights_find_bf16": (C.c_int, [_vp, C.c_char_p, C.POINTER(_vp), C.POINTER(C.c_uint32),
                                          C.POINTER(C.c_uint32)]),
    "mm_f4_weights_free": (None, [_vp]),
    "mm_f4_select_glu": (C.c_int, [C.POINTER(F4Shape), C.POINTER(F4Plan)]),
    "mm_f4_mlp_gate_up": (C.c_int, [_vp, _vp, _vp, C.c_float, _vp, _vp, C.c_float, _vp,
                                    C.c_uint32, C.c_uint32, C.c_uint32, _vp]),
    "mm_silu_mul": (C.c_int, [_vp, _vp, _vp, C.c_size_t, _vp]),
    "kx_op_lmhead": (C.c_int, [C.POINTER(MmKcall)]),
    "kx_op_silu_mul": (C.c_int, [C.POINTER(MmKcall)]),
    "kx_op_add_rmsnorm": (C.c_int, [C.POINTER(MmKcall)]),
    "mm_add_rmsnorm": (C.c_int, [_vp, _vp, _vp, _vp, _u32, _u32, _vp]),
    "mm_norm_eps_set": (C.c_int, [_f]),
    "mm_norm_eps_get": (_f, []),
    "mm_lin_engine_fuse_mlp": (C.c_int, [_vp, C.c_int]),
    "mm_lin_engine_overlap": (C.c_int, [_vp, C.c_int]),
    "mm_lin_engine_n_independent": (C.c_uint32, [_vp]),
    "mm_lin_engine_n_sliced_ahead": (C.c_uint32, [_vp]),
    "mm_lin_engine_group": (C.c_int, [_vp, C.c_int]),
    "mm_lin_engine_n_group_launches": (C.c_uint32, [_vp]),
    "mm_f4_select_variant": (C.c_int, [C.POINTER(F4Shape), C.c_int, C.POINTER(F4Plan)]),
    "mm_f4_force_variant": (None, [C.c_int]),
    "mm_f4_linear": (C.c_int, [_vp, _vp, _vp, _f, _vp, _u32, _u32, _u32, _vp]),
    "mm_f4_tp_push": (C.c_int, [C.POINTER(C.c_void_p), _u32, _u32, _u32, _u32, _u32, _u32]),
    "mm_f4_tp_push_join": (C.c_int, []),
    "mm_lin_engine_add_tp": (C.c_int, [_vp, C.POINTER(MmOpDesc), C.POINTER(C.c_void_p), _u32, _u32, _u32]),
    "mm_f4_device_status_on": (C.c_int, [_vp, C.POINTER(C.c_uint)]),
    "mm_f4_xslice_bytes": (_sz, [_u32, _u32]),
    "mm_f4_xslice": (C.c_int, [_vp, _u32, _u32, _vp, _sz, _vp]),
    "mm_f4_linear_tp": (C.c_int, [_vp, _vp, _vp, _f, C.POINTER(_vp), _u32, _u32, _u32, _u32, _u32, _u32, _vp]),
    "mm_f4_tp_barrier": (C.c_int, [C.POINTER(_vp), _u32, _u32, _vp]),
    "mm_f4_linear_static_ws": (C.c_int, [_vp, _vp, _vp, _f, _vp, _u32, _u32, _u32, _vp]),
    "mm_f4_linear_host": (C.c_int, [_vp, _vp, _vp, _vp, _f, _vp, _vp, _u32, _u32, _u32]),
    "mm_f4_device_status": (C.c_int, [C.POINTER(C.c_uint)]),
    "mm_f4_launch_count": (C.c_ulonglong, [C.c_int]),
    "mm_f4_decode_probe": (C.c_int, [_vp, _vp, _vp]),
    "mm_f4_wait_selftest": (C.c_int, [_vp]),
    "mm_f4_tune": (C.c_int, [C.c_int, C.c_int]),
    "mm_time_begin": (C.c_int, []),
    "mm_time_end": (C.c_int, [C.POINTER(_f)]),
    "mm_f4_pack": (C.c_int, [_vp, _u32, _u32, _vp, _vp, C.POINTER(_f)]),
    "mm_fill_normal_f32": (None, [_vp, C.c_uint64, C.c_uint64, C.c_uint64, _f, _f]),
    "mm_f32_to_bf16": (None, [_vp, _vp, C.c_uint64]),
    "mm_bf16_to_f32": (None, [_vp, _vp, C.c_uint64]),
    "mm_f4_make_weight": (C.c_int, [_u32, _u32, C.c_uint64, _f, _vp, _vp, C.POINTER(_f)]),
    "mm_lin_engine_create": (C.c_int, [C.POINTER(_vp), _u32]),
    "mm_lin_engine_add": (C.c_int, [_vp, C.POINTER(MmOpDesc)]),
    "mm_lin_engine_n_ops": (_u32, [_vp]),
    "mm_lin_engine_capture": (C.c_int, [_vp]),
    "mm_lin_engine_launch": (C.c_int, [_vp]),
    "mm_lin_engine_launch_host": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "mm_lin_engine_bind_host": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "mm_lin_engine_step_bound": (C.c_int, [_vp]),
    "mm_lin_engine_upload_group": (C.c_int, [_vp, _u32]),
    "mm_lin_engine_upload_kernel": (C.c_int, [_vp, C.c_int]),
    "mm_event_record": (C.c_int, [C.c_int, C.c_int]),
    "mm_event_wait": (C.c_int, [C.c_int, C.c_int]),
    "mm_lin_engine_destroy": (None, [_vp]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m mimfer_b200.build`. "
                "mimfer_b200 has no fallback path.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)          # AttributeError if a symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status, what):
    if status != MM_OK:
        raise MimferError(status, what)
