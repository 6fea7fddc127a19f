"""Grouped-GEMM oracle, one problem at a time (TEST INFRASTRUCTURE ONLY).

Restates what one branch of the reference's fused kernel computes for a problem
``C[M, N] = A[M, K] x B[N, K]^T`` (layout.cuh:26-31: A row-major, B stored
``[N, K]``, C row-major fp16):

* w8a8 / w4a4  ``cta_gemm_multistage_qab_v2`` cta_gemm.cuh:423-608, epilogue
  mm_tile.cuh:468-496 + :642-646  -> :func:`int_accumulate`, :func:`wxax_epilogue`
* w4a16 g128   ``cta_gemm_wxa16g128`` cta_gemm.cuh:291-421, dequantisation
  quantize.cuh:134-214 (exact int->fp16, then one fp16 FMA)  -> :func:`dequant_w4a16`,
  :func:`fp_gemm`
* fp16         ``cta_gemm_multistage_v2`` cta_gemm.cuh:7-107 -> :func:`fp_gemm`

The integer accumulators are exact.  Floating-point accumulations (fp32 in the
reference, order unspecified) are evaluated in fp64 and rounded once, so they
are compared with a tolerance, never bit-for-bit.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_clib = None


def c_port():
    """Load ``liboracle_c.so`` (built by ``make -C oracle port``); None if absent."""
    global _clib
    if _clib is None:
        path = os.path.join(_HERE, "liboracle_c.so")
        if os.path.exists(path):
            _clib = ctypes.CDLL(path)
    return _clib


def int_accumulate(qa: np.ndarray, qb: np.ndarray) -> np.ndarray:
    """Exact ``sum_k qa[m,k]*qb[n,k]`` as int32.

    Evaluated through an fp64 matmul: every partial sum is an integer far below
    2**53, so the result is exact.
    """
    acc = qa.astype(np.float64) @ qb.astype(np.float64).T
    assert np.abs(acc).max(initial=0) < 2 ** 31
    return acc.astype(np.int32)


def int_accumulate_c(qa: np.ndarray, qb: np.ndarray) -> np.ndarray:
    """Same sum through the plain-C loop of ``oracle_c.c`` (independent of BLAS)."""
    lib = c_port()
    assert lib is not None, "run `make -C oracle port` first"
    a = np.ascontiguousarray(qa, dtype=np.int8)
    b = np.ascontiguousarray(qb, dtype=np.int8)
    m, k = a.shape
    n = b.shape[0]
    acc = np.empty((m, n), dtype=np.int32)
    lib.oracle_int_gemm(a.ctypes.data_as(ctypes.c_void_p), b.ctypes.data_as(ctypes.c_void_p),
                        m, n, k, acc.ctypes.data_as(ctypes.c_void_p))
    return acc


def wxax_epilogue(acc: np.ndarray, sa: np.ndarray, sb: np.ndarray) -> np.ndarray:
    """``fp16_rn(float(acc) * float(fp16_rn(sa[m]*sb[n])))``; mm_tile.cuh:490-493, :642-646."""
    sa = sa.astype(np.float16).reshape(-1, 1)
    sb = sb.astype(np.float16).reshape(1, -1)
    prod = (sa.astype(np.float32) * sb.astype(np.float32)).astype(np.float16)  # exact product, one rounding
    return (acc.astype(np.float32) * prod.astype(np.float32)).astype(np.float16)


def ref_kernel_scale_b_index(n: int) -> np.ndarray:
    """Which weight scale the reference's KERNEL applies to output channel c (a defect of the reference).

    ``GlobalTileC::load_scale`` (mm_tile.cuh:461-464) fills the two per-channel scales of an 8-column MMA
    fragment from ``smem_scale_b[8j + col]`` and ``[8j + col + 1]`` with ``col = lane % 4``, while the
    thread's accumulator columns are ``8j + 2*col`` and ``8j + 2*col + 1``: channel ``c`` is scaled with
    the weight scale of channel ``8*(c//8) + (c%8)//2 + c%2``.  Measured on a B200 with the reference's
    own generated kernel: its w8a8 / w4a4 outputs are bit-identical to
    ``wxax_epilogue(acc, sa, sb[ref_kernel_scale_b_index(N)])`` and differ from the fake-quant product
    (rel-L2 0.5) unless the weight scales are constant over blocks of 8 channels.  The product kernels
    apply ``sb[c]`` to channel ``c`` (what the reference's quantiser and its torch path mean); this map
    exists so that the tests can show that nothing else differs.
    """
    c = np.arange(n)
    return 8 * (c // 8) + (c % 8) // 2 + c % 2


def wxax_epilogue_c(acc: np.ndarray, sa: np.ndarray, sb: np.ndarray) -> np.ndarray:
    lib = c_port()
    assert lib is not None
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    sa = np.ascontiguousarray(sa, dtype=np.float16)
    sb = np.ascontiguousarray(sb, dtype=np.float16)
    m, n = acc.shape
    out = np.empty((m, n), dtype=np.float16)
    vp = ctypes.c_void_p
    lib.oracle_wxax_epilogue(acc.ctypes.data_as(vp), sa.ctypes.data_as(vp), sb.ctypes.data_as(vp), m, n,
                             out.ctypes.data_as(vp))
    return out


def dequant_w4a16(q: np.ndarray, scale: np.ndarray, zero: np.ndarray, gsize: int = 128) -> np.ndarray:
    """``fp16(fma(q, s, z))`` per group; quantize.cuh:79-93 (exact u4->fp16) and :189-190 (``__hfma2``).

    ``q`` [N, K] in 0..15, ``scale``/``zero`` [N, K/g] fp16.  q*s+z is exact in
    fp64 (4-bit times 11-bit significand plus an fp16), so one rounding to fp16
    reproduces the fused multiply-add.
    """
    n, k = q.shape
    s = np.repeat(scale.astype(np.float64), gsize, axis=1)
    z = np.repeat(zero.astype(np.float64), gsize, axis=1)
    return (q.astype(np.float64) * s + z).astype(np.float16)


def fp_gemm(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    """``fp16_rn(sum_k a[m,k]*w[n,k])`` with a wide accumulator (reference: fp32, mm_tile.cuh:642-646)."""
    return (a.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32).astype(np.float16)


def rel_l2(x: np.ndarray, ref: np.ndarray) -> float:
    x = x.astype(np.float64)
    ref = ref.astype(np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(x - ref) / den) if den > 0 else float(np.linalg.norm(x))
