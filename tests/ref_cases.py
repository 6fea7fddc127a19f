"""Seeded inputs of the device-oracle comparison (reference GroupGEMM kernel vs this library).

Pure numpy: the child process that runs the reference's kernel (tests/ref_gg_worker.py) and the
parity tests build identical operands from the same seeds.  Operand VALUES only; each side packs
them with its own packer (the reference's host packers there, oracle/pack.py and the product's
packers here).

Scheme strings are the reference's (mxmoe/kernels/tile_config.py:40-59).  Every N is a multiple of
128 and every K a multiple of 128: the reference kernel has no N guard (mm_tile.cuh:1046-1058) and
needs K % BK == 0 (cta_gemm.cuh:471).
"""
from __future__ import annotations

import numpy as np

QPARAMS = {                      # (a_bits, w_bits, gsize, sym) as in QParams, quantize.cuh:14-25
    "fp16": (16, 16, -1, 1),
    "w8a8_g-1_sym": (8, 8, -1, 1),
    "w4a4_g-1_sym": (4, 4, -1, 1),
    "w4a16_g128_asym": (16, 4, 128, 0),
    "w4a16_g-1_asym": (16, 4, -1, 0),
    "w4a4_g128_sym": (4, 4, 128, 1),
}

# (scheme, M, N, K, variant): one full tile, a ragged tail, the two linear blocks of the Qwen1.5-MoE expert.
# variant "b8" (schemes with per-channel weight scales only): the weight scales are constant over blocks of 8
# channels, so that a kernel which picked a neighbouring channel's scale inside an 8-column MMA fragment would
# still give the same result - it separates the GEMM arithmetic from the scale indexing.
CASES = [(s, m, n, k, "")
         for s in QPARAMS
         for (m, n, k) in ((128, 256, 256), (300, 2816, 2048), (77, 2048, 1408))]
CASES += [(s, 300, 2816, 2048, "b8") for s in ("w8a8_g-1_sym", "w4a4_g-1_sym", "w4a4_g128_sym")]


def make(idx: int) -> dict:
    """Operand values of case ``idx``: dict with the scheme, the shape and the arrays of its scheme."""
    scheme, m, n, k, variant = CASES[idx]
    rng = np.random.default_rng(4242 + idx)
    a_bits, w_bits, gsize, _sym = QPARAMS[scheme]
    c = {"scheme": scheme, "m": m, "n": n, "k": k}
    if a_bits == 16:
        c["a"] = rng.standard_normal((m, k)).astype(np.float16)
    else:
        hi = 2 ** (a_bits - 1) - 1
        ga = 1 if gsize == -1 else k // gsize
        c["qa"] = rng.integers(-hi, hi + 1, (m, k), dtype=np.int32)
        c["sa"] = rng.uniform(0.01, 0.5, (m, ga)).astype(np.float16)       # [M, groups]
    if w_bits == 16:
        c["b"] = (rng.standard_normal((n, k)) * 0.05).astype(np.float16)
    elif a_bits == 16:                                                     # weight-only, asymmetric
        gw = 1 if gsize == -1 else k // gsize
        c["qb"] = rng.integers(0, 16, (n, k), dtype=np.int32)
        c["sb"] = rng.uniform(0.001, 0.01, (n, gw)).astype(np.float16)     # [N, groups]
        c["zb"] = rng.uniform(-0.08, -0.01, (n, gw)).astype(np.float16)
    else:
        hi = 2 ** (w_bits - 1) - 1
        gw = 1 if gsize == -1 else k // gsize
        c["qb"] = rng.integers(-hi, hi + 1, (n, k), dtype=np.int32)
        c["sb"] = rng.uniform(0.002, 0.02, (n, gw)).astype(np.float16)
        if variant == "b8":
            c["sb"] = np.repeat(c["sb"][::8], 8, axis=0)
    return c
