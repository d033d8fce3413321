"""NVFP4 tensors in the weights section of a model artifact.

write_section builds the section payload (tensor index + tensor bytes) in the
layout of the mimfer loader (src/model/tensor_registry.h:86-120) with
MM_DT_FP4E2M1 entries, which the reference loader itself rejects
(src/model/tensor_registry.c:468-474); WeightStore stages such a payload into
one device block through the C loader (csrc/model/weights.c) and hands out
NvFp4Weight views by name.
"""
import ctypes as C
import struct

import numpy as np

from . import _lib as L
from .linear import NvFp4Weight

ALIGN = 256


def write_section(tensors, align=ALIGN):
    """tensors: list of (name, NvFp4Weight) or (name, uint16 ndarray [rows][cols] of bf16 bits).
    Returns the section payload as bytes; tensor bytes start on `align` boundaries."""
    names = [n.encode() + b"\0" for n, _ in tensors]
    for n in names:
        if not 1 <= len(n) <= 48:
            raise ValueError(f"tensor name {n!r} does not fit 48 bytes")
    index_len = 12 + sum(2 + len(n) + 28 for n in names)
    blobs, entries = [], []
    at = end = (index_len + align - 1) // align * align
    for (name, t), raw in zip(tensors, names):
        if isinstance(t, NvFp4Weight):
            blob = (np.ascontiguousarray(t.payload).tobytes() + np.ascontiguousarray(t.scales).tobytes() +
                    struct.pack("<f", t.gs))
            rows, cols, dt = t.N, t.K, L.MM_DT_FP4E2M1
        else:
            a = np.ascontiguousarray(t, np.uint16)
            blob, (rows, cols), dt = a.tobytes(), a.shape, L.MM_DT_BF16
        entries.append(struct.pack("<H", len(raw)) + raw +
                       struct.pack("<IIB3xQQ", rows, cols, dt, at, len(blob)))
        blobs.append((at, blob))
        end = at + len(blob)
        at = (end + align - 1) // align * align
    head = struct.pack("<III", 1, 0, len(tensors)) + b"".join(entries)
    assert len(head) == index_len
    out = bytearray(end if blobs else index_len)
    out[:index_len] = head
    for off, blob in blobs:
        out[off:off + len(blob)] = blob
    return bytes(out)


def parse_section(data):
    """Validated tensor index: list of dicts (name, rows, cols, dtype, off, nbytes)."""
    buf = (C.c_uint8 * len(data)).from_buffer_copy(data)
    n = C.c_uint32()
    L.check(L.lib().mm_f4_weights_parse(buf, len(data), None, 0, C.byref(n)), "mm_f4_weights_parse")
    ents = (L.F4Went * max(1, n.value))()
    L.check(L.lib().mm_f4_weights_parse(buf, len(data), ents, n.value, C.byref(n)), "mm_f4_weights_parse")
    return [dict(name=e.name.decode(), rows=e.rows, cols=e.cols, dtype=e.dtype, off=e.off, nbytes=e.nbytes)
            for e in ents[:n.value]]


def arena_bytes(data):
    buf = (C.c_uint8 * len(data)).from_buffer_copy(data)
    n = C.c_uint32()
    L.check(L.lib().mm_f4_weights_parse(buf, len(data), None, 0, C.byref(n)), "mm_f4_weights_parse")
    ents = (L.F4Went * max(1, n.value))()
    L.check(L.lib().mm_f4_weights_parse(buf, len(data), ents, n.value, C.byref(n)), "mm_f4_weights_parse")
    return L.lib().mm_f4_weights_arena_bytes(ents, n.value)


class WeightStore:
    """One device block holding every tensor of a section; views by name."""

    def __init__(self, rt, data):
        self.rt = rt
        torch = rt.torch
        need = arena_bytes(data)
        self.block = torch.empty(max(need, ALIGN), dtype=torch.uint8, device=rt.device)
        torch.cuda.synchronize()
        self._host = np.frombuffer(data, np.uint8)
        self.h = C.c_void_p()
        L.check(rt.lib.mm_f4_weights_stage(self._host.ctypes.data_as(C.c_void_p), len(data),
                                           self.block.data_ptr(), self.block.numel(), C.byref(self.h)),
                "mm_f4_weights_stage")
        self.index = {e["name"]: e for e in parse_section(data)}

    def __len__(self):
        return self.rt.lib.mm_f4_weights_count(self.h)

    def weight(self, name):
        """NvFp4Weight whose device tensors alias the block (host arrays alias the section)."""
        wt, gs = L.MmWt(), C.c_float()
        L.check(self.rt.lib.mm_f4_weights_find(self.h, name.encode(), C.byref(wt), C.byref(gs)),
                "mm_f4_weights_find")
        e = self.index[name]
        N, K = wt.rows, wt.cols
        pb, sb = N * K // 2, N * K // 16
        payload = self._host[e["off"]:e["off"] + pb].reshape(N, K // 2)
        scales = self._host[e["off"] + pb:e["off"] + pb + sb].reshape(N, K // 16)
        w = NvFp4Weight(payload, scales, gs.value, N, K)
        base = self.block.data_ptr()
        po, so = wt.data - base, wt.scale - base
        w.dev_payload = self.block[po:po + pb].view(N, K // 2)
        w.dev_scales = self.block[so:so + sb].view(N, K // 16)
        return w

    def close(self):
        if self.h:
            self.rt.lib.mm_f4_weights_free(self.h)
            self.h = C.c_void_p()
