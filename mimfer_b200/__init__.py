"""mimfer_b200: B200-native NVFP4 linear layer behind the mimfer operator ABI.

The compute lives in libmimfer_b200.so (hand-written sm_100a kernels + a C
host layer); this package is the Python mirror of that C-ABI used by the
tests and the benchmark.  PyTorch is used only to own device memory and for
torch.distributed.
"""
from ._lib import (lib, check, MimferError, MmOpDesc, MmKcall, F4Shape, F4Plan,
                   OP_GEMM_F4, OP_QKV, OP_LMHEAD, OP_SILU_MUL, OP_ADD_RMSNORM, OP_NOP, V_ROWWARP, V_STREAM, V_UMMA, V_MX)
from .linear import (NvFp4Weight, make_weight, pack_weight, make_activations, select_plan,
                     place_weights, Runtime, LinearEngine, weight_bytes)

__all__ = ["lib", "check", "MimferError", "MmOpDesc", "MmKcall", "F4Shape", "F4Plan",
           "OP_GEMM_F4", "OP_QKV", "OP_LMHEAD", "OP_SILU_MUL", "OP_ADD_RMSNORM", "OP_NOP", "V_ROWWARP", "V_STREAM", "V_UMMA", "V_MX",
           "NvFp4Weight", "make_weight", "pack_weight", "make_activations", "select_plan", "place_weights",
           "Runtime", "LinearEngine", "weight_bytes"]
