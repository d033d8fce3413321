"""The drop-in boundary: the shared library loads without a GPU and exports
every entry point the public headers declare; the restated ABI structs have
the reference's layout."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import pytest

from conftest import ROOT
from mimfer_b200 import _lib as L

INCLUDE = os.path.join(ROOT, "include")
REF = os.environ.get("MIMFER_REFERENCE", os.path.join(os.sep, "root", "reference"))   # the reference tree, where mounted


def declared_functions():
    text = ""
    for name in sorted(os.listdir(INCLUDE)):
        if name.endswith(".h"):
            text += open(os.path.join(INCLUDE, name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b((?:mm|kx)_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_loads_and_exports_all_declared_symbols(lib):
    names = declared_functions()
    assert len(names) >= 45
    handle = C.CDLL(L.LIB_PATH)
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, missing
    # and the Python binding covers the same set
    assert sorted(L.SIGNATURES) == names


def test_struct_sizes():
    assert C.sizeof(L.MmOpDesc) == 80 and C.sizeof(L.MmKcall) == 24
    assert L.MmOpDesc.a.offset == 8 and L.MmOpDesc.d.offset == 32
    assert L.MmOpDesc.n0.offset == 40 and L.MmOpDesc.note.offset == 52


def test_status_strings(lib):
    assert lib.mm_status_str(0) == b"ok"
    assert lib.mm_status_str(4) == b"bad shape or stride"
    assert lib.mm_status_str(99) == b"unknown status"


PROBE = r"""
#include <stdio.h>
#include <stddef.h>
#ifdef USE_REFERENCE
#include "mimfer/mimfer.h"
#include "mimfer/plan.h"
#include "mimfer/kernels.h"
#include "mimfer/tensor.h"
#else
#include "mimfer_abi.h"
#endif
int main(void) {
    printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu ", sizeof(mm_op_desc), offsetof(mm_op_desc, op),
           offsetof(mm_op_desc, layer), offsetof(mm_op_desc, a), offsetof(mm_op_desc, b),
           offsetof(mm_op_desc, c), offsetof(mm_op_desc, d), offsetof(mm_op_desc, n0),
           offsetof(mm_op_desc, note));
    printf("%zu %zu %zu %zu ", sizeof(mm_kcall), offsetof(mm_kcall, op), offsetof(mm_kcall, e),
           offsetof(mm_kcall, stream));
    printf("%zu %zu %zu %zu ", sizeof(mm_wt), offsetof(mm_wt, scale), offsetof(mm_wt, rows),
           offsetof(mm_wt, cols));
    printf("%d %d %d %d %d %d ", OP_LMHEAD, OP_GEMM_F4, OP_GEMM_BF16, OP_QKV, OP_NOP, OP_N);
    printf("%d %d %d %d %d %d %d %d\n", MM_OK, MM_ERR_SHAPE, MM_ERR_CUDA, MM_ERR_UNSUPPORTED,
           MM_ERR_STATE, MM_ERR_TIMEOUT, MM_ERR_LAST, MM_ST_COMPUTE);
    return 0;
}
"""


def _run_probe(flags):
    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "p.c"), os.path.join(d, "p")
        open(src, "w").write(PROBE)
        subprocess.check_call(["gcc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", *flags, src, "-o", exe])
        return subprocess.check_output([exe]).decode().split()


def test_layout_matches_reference_headers():
    ours = _run_probe(["-I" + INCLUDE])
    assert ours[0] == "80"
    if not os.path.isdir(os.path.join(REF, "include", "mimfer")):
        pytest.skip("reference headers not mounted; static asserts in mimfer_abi.h pin the layout")
    theirs = _run_probe(["-DUSE_REFERENCE", "-I" + os.path.join(REF, "include")])
    assert ours == theirs
