"""Generate the golden fixtures from the reference's own CPU kernel.

Needs oracle/_ref/libmimfer_ref.so, i.e. the mimfer tree mounted where
oracle/build.py looks for it; the fixtures are committed so the tests do not.

  decode_products.npz   every (scale byte, nibble) product, read out of the
                        reference kx_op_gemm_f4 (src/kernels/cpu/cx.c:197-216)
                        with one-hot activations; nibble in the low and in the
                        high half of a byte; second scale block of a row.
  random_bytes.npz      payload and scale bytes drawn uniformly (all 256 scale
                        codes incl. 0x7f/0xff and negative scales), inputs stored.
  silu_mul.npz          the reference kx_op_silu_mul (src/kernels/cpu/cx.c:155-167) on
                        every bf16 bit pattern as the gate against seeded random up
                        bits (PCG64 seed 5; only the output is stored).
  add_rmsnorm.npz       the reference kx_op_add_rmsnorm (src/kernels/cpu/cx.c:132-150) on
                        seeded rows: residual N(0, 1) + a few large and tiny values, delta
                        N(0, 0.5), gain N(1, 0.1), eps 1e-6; hidden sizes 64, 1000 and 5120.
                        Inputs are regenerated from the seeds, outputs are stored.
  seeded_<M>x<K>x<N>.npz  weights from the library's packer + generator (seed 0,
                        N(0, 0.02)), activations seed 1 N(0, 1); stores the
                        reference output, the global scale the packer chose and
                        FNV-1a checksums of the generated inputs.

Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import mimfer_b200 as mm                      # noqa: E402
from oracle.pyoracle import Reference        # noqa: E402

SEEDED = [(1, 256, 64), (3, 512, 40), (5, 1024, 96), (8, 768, 33), (16, 2048, 128),
          (2, 5120, 64), (33, 256, 72)]


ADD_RMSNORM_SHAPES = [(1, 64), (3, 1000), (4, 5120)]
ADD_RMSNORM_EPS = 1.0e-6


def add_rmsnorm_inputs(M, H):
    """Seeded inputs of the add + RMSNorm fixture (bf16 bit patterns)."""
    res = mm.linear.fill_normal(M, H, 100 + H, 0.0, 1.0)
    res[0, 1] = 300.0
    res[M - 1, H // 2] = -2.0e-5
    delta = mm.linear.fill_normal(M, H, 200 + H, 0.0, 0.5)
    gain = mm.linear.fill_normal(1, H, 300 + H, 1.0, 0.1)
    return mm.linear.f32_to_bf16(res), mm.linear.f32_to_bf16(delta), mm.linear.f32_to_bf16(gain)[0]


def fnv1a64(a):
    h = 1469598103934665603
    for b in np.ascontiguousarray(a).view(np.uint8).ravel().tolist():
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return np.uint64(h)


def decode_products(ref):
    one = 0x3F80                                         # bf16 1.0
    out = {}
    for name, col in (("low_nibble_col0", 0), ("high_nibble_col1", 1), ("second_block_col17", 17)):
        K = 32
        payload = np.zeros((4096, K // 2), np.uint8)
        scales = np.zeros((4096, K // 16), np.uint8)
        s = np.repeat(np.arange(256, dtype=np.uint8), 16)
        n = np.tile(np.arange(16, dtype=np.uint8), 256)
        payload[:, col // 2] = n << 4 if col & 1 else n
        scales[:, col // 16] = s
        x = np.zeros((1, K), np.uint16)
        x[0, col] = one
        rc, y = ref.gemm_f4(x, payload, scales)
        assert rc == 0
        out[name] = y[0].copy()                          # bf16 bits, index s*16+n
    return out


def main():
    ref = Reference()
    if not ref.available:
        sys.exit("reference library not available; cannot regenerate fixtures")
    np.savez_compressed(os.path.join(HERE, "decode_products.npz"), **decode_products(ref))

    rng = np.random.Generator(np.random.PCG64(20250101))
    M, K, N = 4, 512, 96
    payload = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    scales = rng.integers(0, 256, (N, K // 16), dtype=np.uint8)
    scales[0, :4] = (0x7F, 0xFF, 0x80, 0x00)
    x = mm.make_activations(M, K, seed=7)
    rc, y = ref.gemm_f4(x, payload, scales)
    assert rc == 0
    np.savez_compressed(os.path.join(HERE, "random_bytes.npz"), x=x, payload=payload, scales=scales, y=y)

    gate = np.arange(65536, dtype=np.uint16)
    up = np.random.Generator(np.random.PCG64(5)).integers(0, 65536, 65536, dtype=np.uint16)
    rc, y = ref.silu_mul(gate, up)
    assert rc == 0
    np.savez_compressed(os.path.join(HERE, "silu_mul.npz"), y=y)

    norm = {}
    for (M, H) in ADD_RMSNORM_SHAPES:
        res, delta, gain = add_rmsnorm_inputs(M, H)
        rc, res_out, y = ref.add_rmsnorm(res, delta, gain, ADD_RMSNORM_EPS)
        assert rc == 0
        norm[f"res_{M}x{H}"] = res_out
        norm[f"y_{M}x{H}"] = y
    np.savez_compressed(os.path.join(HERE, "add_rmsnorm.npz"), **norm)

    for (M, K, N) in SEEDED:
        w = mm.make_weight(N, K, seed=0, std=0.02)
        x = mm.make_activations(M, K, seed=1)
        rc, y = ref.gemm_f4(x, w.payload, w.scales)
        assert rc == 0
        np.savez_compressed(os.path.join(HERE, f"seeded_{M}x{K}x{N}.npz"), y=y,
                            gs=np.float32(w.gs), payload_fnv=fnv1a64(w.payload),
                            scales_fnv=fnv1a64(w.scales), x_fnv=fnv1a64(x))
    # K % 16 != 0 is an error in the reference
    rc, _ = ref.gemm_f4(np.zeros((1, 24), np.uint16), np.zeros((2, 12), np.uint8), np.zeros((2, 2), np.uint8))
    np.savez_compressed(os.path.join(HERE, "status.npz"), k_not_multiple_of_16=np.int32(rc))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
