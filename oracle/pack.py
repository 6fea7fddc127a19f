"""Packed operand layouts of the reference, restated in numpy (TEST INFRASTRUCTURE ONLY).

The only definition of these layouts in the reference is its host-side pack
code, ``mxmoe/kernels/src/include/quantize.cuh``:

* ``pack_wxax``       (:424-475)  weight+activation schemes (w8a8, w4a4): codes
  packed along K into uint16 words, first k in the most significant field.
* ``permute_weight``  (:318-385) followed by ``pack_weightonly`` (:387-421)
  weight-only schemes (w4a16): codes packed along N, fragment-permuted.
* ``permute_scale``   (:299-315)  group scales / (scale, zero) pairs, group-major.

``tests/test_oracle_golden.py`` pins every function here against golden words
produced by the reference's own functions.
"""
from __future__ import annotations

import numpy as np


# ---------------------------------------------------------------------------
# weight + activation schemes: K-packed two's-complement fields
# ---------------------------------------------------------------------------
def pack_k(codes: np.ndarray, bits: int) -> np.ndarray:
    """``[R, K]`` integer codes -> ``[R, K*bits/16]`` uint16 (quantize.cuh:457-470).

    Field ``x`` (0 = first k of the word) lands at bit ``bits*(P-1-x)``, ``P = 16/bits``;
    each field is the two's-complement code (sign bit | low bits, :441-448).
    """
    assert bits in (4, 8)
    p = 16 // bits
    r, k = codes.shape
    assert k % p == 0
    mask = (1 << bits) - 1
    fields = (codes.astype(np.int64) & mask).reshape(r, k // p, p)
    shifts = (bits * (p - 1 - np.arange(p))).astype(np.int64)
    return (fields << shifts).sum(axis=-1).astype(np.uint16)


def unpack_k(words: np.ndarray, bits: int) -> np.ndarray:
    """Inverse of :func:`pack_k`: ``[R, W]`` uint16 -> ``[R, W*16/bits]`` int32 codes."""
    p = 16 // bits
    mask = (1 << bits) - 1
    shifts = (bits * (p - 1 - np.arange(p))).astype(np.int64)
    f = (words.astype(np.int64)[..., None] >> shifts) & mask
    f = np.where(f >= (1 << (bits - 1)), f - (1 << bits), f)
    return f.reshape(words.shape[0], -1).astype(np.int32)


def expand_k4(codes: np.ndarray) -> np.ndarray:
    """``[R, K]`` 4-bit codes -> ``[R, K]`` bytes ``16*q`` in the order the B200 kernel's own int4 -> int8
    unpacking produces from the packed row (no counterpart in the reference: an internal activation
    format of this build).  Every 16 packed bytes become 16 bytes holding their high nibbles followed
    by 16 bytes holding their low nibbles, each nibble moved to the top of its byte."""
    pb = pack_k(codes, 4).view(np.uint8).reshape(codes.shape[0], -1, 16)       # [R, K/32, 16] packed bytes
    hi = pb & 0xF0
    lo = (pb << 4) & 0xF0
    return np.concatenate((hi, lo), axis=2).reshape(codes.shape[0], -1)


# ---------------------------------------------------------------------------
# weight-only 4-bit scheme: N-packed, fragment-permuted
# ---------------------------------------------------------------------------
def pack_n4(codes: np.ndarray) -> np.ndarray:
    """``[N, K]`` unsigned 4-bit codes -> ``[N/4, K]`` uint16.

    Closed form of ``pack_weightonly(permute_weight(w, N, K, 4), N, K, 4)``
    (quantize.cuh:318-421).  With ``n = 32*nb + 8*f + r`` (f in 0..3, r in 0..7)
    and ``k = 16*kb + 8*c + d`` (c in 0..1, d in 0..7) the code sits in word
    ``(row = 8*nb + r, col = 16*kb + 8*(f >> 1) + d)`` at nibble ``2*(f & 1) + c``
    counted from the least significant nibble.
    """
    n, k = codes.shape
    assert n % 32 == 0 and k % 16 == 0
    c6 = (codes.astype(np.int64) & 0xF).reshape(n // 32, 2, 2, 8, k // 16, 2, 8)
    #        axes:                               nb  fh  fl  r   kb      c   d
    out = np.zeros((n // 32, 8, k // 16, 2, 8), dtype=np.int64)  # nb r kb fh d
    for fl in range(2):
        for c in range(2):
            v = c6[:, :, fl, :, :, c, :]            # nb fh r kb d
            out |= v.transpose(0, 2, 3, 1, 4) << (4 * (2 * fl + c))
    return out.reshape(n // 4, k).astype(np.uint16)


def unpack_n4(words: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_n4`: ``[N/4, K]`` uint16 -> ``[N, K]`` int32 codes in 0..15."""
    n4, k = words.shape
    n = n4 * 4
    w = words.astype(np.int64).reshape(n // 32, 8, k // 16, 2, 8)  # nb r kb fh d
    codes = np.zeros((n // 32, 2, 2, 8, k // 16, 2, 8), dtype=np.int64)
    for fl in range(2):
        for c in range(2):
            v = (w >> (4 * (2 * fl + c))) & 0xF     # nb r kb fh d
            codes[:, :, fl, :, :, c, :] = v.transpose(0, 3, 1, 2, 4)
    return codes.reshape(n, k).astype(np.int32)


# ---------------------------------------------------------------------------
# scales
# ---------------------------------------------------------------------------
def group_major_scales(scale: np.ndarray, zero: np.ndarray | None) -> np.ndarray:
    """``[N, G]`` per-(row, group) parameters -> group-major storage (quantize.cuh:299-315).

    Symmetric (``zero is None``): ``[G, N]``; asymmetric: ``[G, N, 2]`` with
    (scale, zero) interleaved.  For per-channel schemes G == 1 and this is the
    identity on the scale vector.
    """
    if zero is None:
        return np.ascontiguousarray(scale.T)
    return np.ascontiguousarray(np.stack((scale.T, zero.T), axis=-1))
