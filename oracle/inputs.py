"""Host-only synthetic inputs for the CPU checkers (test infrastructure only).

numpy restatement of the NVFP4 packing recipe, so that a run of the CPU
reference needs nothing but numpy and the compiled reference kernel:

  gs            = max|W| / (6 * 448)            (1.0 for an all-zero tensor)
  scale(block)  = e4m3 nearest-even, saturating, of amax_block / (6 * gs)
  nibble(w)     = e2m1 nearest-even, saturating, of w / (e4m3(scale) * gs)

Layout as the reference's tensor view has it (include/mimfer/tensor.h:17-19,
121-126): payload [N][K/2], low nibble = even column; scales [N][K/16].
"""
import numpy as np

_E4M3 = np.array([(1 + (c & 7) / 8.0) * 2.0 ** ((c >> 3) - 7) if c >> 3 else (c & 7) / 8.0 * 2.0 ** -6
                  for c in range(0x7F)], np.float32)           # codes 0 .. 0x7e, ascending
_E2M1_EDGES = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
_E2M1_TIE_UP = np.array([False, True, False, True, False, True, False])   # at an edge: the even code


def e4m3_encode(f):
    """f >= 0, float32 array -> uint8 codes."""
    f = np.asarray(f, np.float32)
    hi = np.clip(np.searchsorted(_E4M3, f, side="right"), 1, 0x7E)       # value(hi - 1) <= f < value(hi)
    lo = hi - 1
    dl, dh = f - _E4M3[lo], _E4M3[hi] - f
    pick_hi = (dh < dl) | ((dh == dl) & ((lo & 1) == 1))
    code = np.where(pick_hi, hi, lo)
    code = np.where(f >= 448.0, 0x7E, code)
    return np.where(f > 0, code, 0).astype(np.uint8)


def e2m1_encode(v):
    v = np.asarray(v, np.float32)
    a = np.abs(v)
    code = np.searchsorted(_E2M1_EDGES, a, side="left")                  # edges crossed strictly
    at_edge = np.isin(a, _E2M1_EDGES)
    idx = np.clip(code, 0, 6)
    code = np.where(at_edge & _E2M1_TIE_UP[idx], code + 1, code)
    return (np.where(np.signbit(v), 8, 0) | code).astype(np.uint8)


def pack(W):
    """fp32 W [N][K] -> (payload uint8 [N][K/2], scales uint8 [N][K/16], gs)."""
    W = np.ascontiguousarray(W, np.float32)
    N, K = W.shape
    wmax = np.float32(np.abs(W).max()) if W.size else np.float32(0)
    gs = np.float32(wmax / np.float32(6.0 * 448.0)) if wmax > 0 else np.float32(1.0)
    blocks = W.reshape(N, K // 16, 16)
    amax = np.abs(blocks).max(axis=2)
    scales = e4m3_encode(amax / (np.float32(6.0) * gs))
    denom = (_E4M3[scales] * gs)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(denom > 0, blocks / denom, np.float32(0)).astype(np.float32)
    nib = e2m1_encode(q).reshape(N, K)
    nib = np.where((denom > 0).repeat(16, axis=2).reshape(N, K), nib, 0).astype(np.uint8)
    payload = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    return payload, scales, float(gs)


def bf16_bits(a):
    """float32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def make_weight(N, K, seed=0, std=0.02):
    rng = np.random.Generator(np.random.PCG64(seed))
    return pack(rng.standard_normal((N, K), dtype=np.float32) * np.float32(std))


def make_activations(M, K, seed=1):
    rng = np.random.Generator(np.random.PCG64(seed))
    return bf16_bits(rng.standard_normal((M, K), dtype=np.float32))
