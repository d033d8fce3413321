"""The weights-section reader with NVFP4 entries (csrc/model/weights.c): index
layout and validation gates of the reference loader
(src/model/tensor_registry.h:86-120, tensor_registry.c:372-511), fp4 admitted."""
import ctypes as C
import struct

import numpy as np
import pytest

import mimfer_b200 as mm
from mimfer_b200 import _lib as L, weights as W


def _tensors():
    return [("model.layers.0.mlp.gate_proj.weight", mm.make_weight(96, 256, seed=1)),
            ("model.layers.0.mlp.up_proj.weight", mm.make_weight(96, 256, seed=2)),
            ("model.norm.weight", mm.make_activations(1, 256, seed=3)),
            ("lm_head.weight", mm.make_weight(40, 512, seed=4))]


def test_round_trip_and_sizes(lib):
    ts = _tensors()
    data = W.write_section(ts)
    idx = W.parse_section(data)
    assert [e["name"] for e in idx] == [n for n, _ in ts]
    g = idx[0]
    assert (g["rows"], g["cols"], g["dtype"]) == (96, 256, L.MM_DT_FP4E2M1)
    assert g["nbytes"] == 96 * 256 // 2 + 96 * 256 // 16 + 4 == lib.mm_f4_tensor_bytes(96, 256)
    assert idx[2]["dtype"] == L.MM_DT_BF16 and idx[2]["nbytes"] == 512
    for e in idx:
        assert e["off"] % 256 == 0 and e["off"] + e["nbytes"] <= len(data)
    # tensor bytes are where the index says
    w = ts[0][1]
    off = g["off"]
    assert data[off:off + w.payload.size] == w.payload.tobytes()
    assert struct.unpack("<f", data[off + g["nbytes"] - 4:off + g["nbytes"]])[0] == np.float32(w.gs)
    # arena: every tensor part on a 256-byte boundary, payload and scales in separate slots
    up = lambda v: (v + 255) // 256 * 256
    want = 2 * (up(96 * 128) + up(96 * 16)) + up(512) + up(40 * 256) + up(40 * 32)
    assert W.arena_bytes(data) == want


def _expect(lib, data, status):
    lib.mm_log_set_level(-1)
    try:
        with pytest.raises(mm.MimferError) as e:
            W.parse_section(bytes(data))
        assert e.value.status == status
    finally:
        lib.mm_log_set_level(1)


def test_validation_gates(lib):
    data = bytearray(W.write_section(_tensors()))
    first = 12                                   # first entry: u16 name_len, name, 28 bytes
    nl = struct.unpack_from("<H", data, first)[0]
    rows_at = first + 2 + nl

    _expect(lib, data[:8], L.MM_ERR_CORRUPT)                         # shorter than the header
    bad = bytearray(data); struct.pack_into("<I", bad, 0, 2)
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # version
    bad = bytearray(data); struct.pack_into("<I", bad, 4, 1)
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # flags
    bad = bytearray(data); struct.pack_into("<I", bad, 8, 5000)
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # more than 4096 tensors
    bad = bytearray(data); struct.pack_into("<I", bad, 8, 40)
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # index runs into tensor bytes / off the end
    _expect(lib, data[:first + 10], L.MM_ERR_CORRUPT)                # truncated inside an entry
    for v in (0, 49):
        bad = bytearray(data); struct.pack_into("<H", bad, first, v)
        _expect(lib, bad, L.MM_ERR_CORRUPT)                          # name_len range
    bad = bytearray(data); bad[first + 2 + nl - 1] = ord("x")
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # no NUL
    bad = bytearray(data); struct.pack_into("<Q", bad, rows_at + 20, 7)
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # nbytes != rows*cols*9/16 + 4
    bad = bytearray(data); struct.pack_into("<Q", bad, rows_at + 12, 16)
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # bytes inside the index
    bad = bytearray(data); struct.pack_into("<Q", bad, rows_at + 12, len(data) - 100)
    _expect(lib, bad, L.MM_ERR_CORRUPT)                              # bytes past the end
    bad = bytearray(data); bad[rows_at + 8] = 3                      # MM_DT_F32
    _expect(lib, bad, L.MM_ERR_UNSUPPORTED)
    bad = bytearray(data); struct.pack_into("<I", bad, rows_at + 4, 250)
    _expect(lib, bad, L.MM_ERR_SHAPE)                                # fp4 cols % 16


def test_empty_section(lib):
    data = W.write_section([])
    assert len(data) == 12 and W.parse_section(data) == [] and W.arena_bytes(data) == 0


@pytest.mark.gpu
def test_stage_and_run_from_the_store(rt, oracle):
    from conftest import REL_L2_TOL, row_rel_l2
    ts = _tensors()
    data = W.write_section(ts)
    store = W.WeightStore(rt, data)
    assert len(store) == 4 and rt.lib.mm_f4_weights_used(store.h) == W.arena_bytes(data)
    # bytes on the device are the section's bytes, global scale registered
    for name, w in (ts[0], ts[1], ts[3]):
        v = store.weight(name)
        assert np.array_equal(v.dev_payload.cpu().numpy(), w.payload)
        assert np.array_equal(v.dev_scales.cpu().numpy(), w.scales)
        assert v.gs == np.float32(w.gs)
        assert rt.lib.mm_f4_gscale_get(v.dev_scales.data_ptr()) == np.float32(w.gs)
        assert v.dev_payload.data_ptr() % 256 == 0 and v.dev_scales.data_ptr() % 256 == 0
    # a linear and the fused gate/up kernel straight from the staged tensors
    head = store.weight("lm_head.weight")
    xb = mm.make_activations(3, 512, seed=5)
    y = rt.gemm_f4(rt.to_device_bf16(xb), head)
    assert row_rel_l2(rt.from_device_bf16(y), oracle.gemm_f4(xb, head.payload, head.scales, head.gs)) <= REL_L2_TOL
    gate, up = store.weight(ts[0][0]), store.weight(ts[1][0])
    xb = mm.make_activations(5, 256, seed=6)
    y = rt.torch.zeros((5, 96), dtype=rt.torch.bfloat16, device=rt.device)
    rt.mlp_gate_up_async(rt.to_device_bf16(xb), gate, up, y)
    rt.sync()
    assert row_rel_l2(rt.from_device_bf16(y), oracle.mlp_gate_up(xb, gate, up)) <= REL_L2_TOL
    # lookups of the other kind or of unknown names
    wt, gs = L.MmWt(), C.c_float()
    rt.lib.mm_log_set_level(-1)
    assert rt.lib.mm_f4_weights_find(store.h, b"model.norm.weight", C.byref(wt), C.byref(gs)) == L.MM_ERR_UNSUPPORTED
    assert rt.lib.mm_f4_weights_find(store.h, b"nope", C.byref(wt), C.byref(gs)) == L.MM_ERR_RANGE
    ptr, r, c = C.c_void_p(), C.c_uint32(), C.c_uint32()
    assert rt.lib.mm_f4_weights_find_bf16(store.h, b"model.norm.weight", C.byref(ptr), C.byref(r), C.byref(c)) == L.MM_OK
    assert (r.value, c.value) == (1, 256) and ptr.value % 256 == 0
    rt.lib.mm_log_set_level(1)
    # a duplicate name is refused at staging
    dup = W.write_section([ts[0], ts[0]])
    with pytest.raises(mm.MimferError) as e:
        W.WeightStore(rt, dup)
    assert e.value.status == L.MM_ERR_CORRUPT
    store.close()
