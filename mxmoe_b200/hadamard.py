"""Hadamard rotations for row lengths that are not powers of two.

The reference rotates the input of the down projection online with ``H_n = had_K (x) H_m`` where ``n = K * m``,
``m`` a power of two and ``had_K`` a K x K Hadamard matrix taken from a table (``get_hadK``,
mxmoe/quant/hadamard_utils.py:5-59; ``matmul_hadU_cuda`` :96-105; hook mxmoe/quant/rotation.py:403-421).
:func:`hadamard_kron` is that transform on the sm_100a kernel; the factor matrix is an argument, so a caller that
holds weights rotated with the reference's tables passes the reference's matrix.  :func:`hadamard_factor` builds
a factor where a classical construction exists (Paley I / II over a prime field, Sylvester doubling) for callers
that rotate their own weights: any Hadamard matrix of the right order gives an orthogonal rotation, and weights
and activations only have to use the same one.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from .gg import current_stream_ptr

# the factor orders the reference tries, in its order of preference (get_hadK)
_FACTOR_ORDERS = (176, 172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12)


def _is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def _is_prime(q: int) -> bool:
    return q > 1 and all(q % d for d in range(2, int(math.isqrt(q)) + 1))


def _jacobsthal(q: int) -> torch.Tensor:
    """Q[i, j] = chi(i - j) over the prime field GF(q): +1 for non-zero squares, -1 for non-squares, 0 on the diagonal."""
    squares = {(x * x) % q for x in range(1, q)}
    chi = torch.tensor([0] + [1 if v in squares else -1 for v in range(1, q)], dtype=torch.int64)
    idx = (torch.arange(q).reshape(-1, 1) - torch.arange(q).reshape(1, -1)) % q
    return chi[idx]


def paley(order: int) -> torch.Tensor | None:
    """Hadamard matrix of ``order`` by Paley's constructions over a prime field, or None.

    I:  q = order - 1 prime, q = 3 (mod 4): H = I + S with S = [[0, 1^T], [-1, Q]] skew-symmetric.
    II: q = order / 2 - 1 prime, q = 1 (mod 4): the symmetric conference matrix C = [[0, 1^T], [1, Q]] with every
        0 replaced by [[1, -1], [-1, -1]] and every +-1 by +-[[1, 1], [1, -1]]."""
    q = order - 1
    if _is_prime(q) and q % 4 == 3:
        s = torch.zeros((order, order), dtype=torch.int64)
        s[0, 1:] = 1
        s[1:, 0] = -1
        s[1:, 1:] = _jacobsthal(q)
        return s + torch.eye(order, dtype=torch.int64)
    if order % 2 == 0:
        q = order // 2 - 1
        if _is_prime(q) and q % 4 == 1:
            n = q + 1
            c = torch.zeros((n, n), dtype=torch.int64)
            c[0, 1:] = 1
            c[1:, 0] = 1
            c[1:, 1:] = _jacobsthal(q)
            zero = torch.tensor([[1, -1], [-1, -1]])
            unit = torch.tensor([[1, 1], [1, -1]])
            return torch.kron(c, unit) + torch.kron(torch.eye(n, dtype=torch.int64), zero)
    return None


def hadamard_matrix(order: int) -> torch.Tensor | None:
    """A Hadamard matrix of ``order`` (int64 +-1) by Paley's constructions and Sylvester doubling, or None."""
    if order == 1:
        return torch.ones((1, 1), dtype=torch.int64)
    h = paley(order)
    if h is not None:
        return h
    if order % 2 == 0:
        half = hadamard_matrix(order // 2)
        if half is not None:
            return torch.kron(torch.tensor([[1, 1], [1, -1]]), half)
    return None


def hadamard_factor(n: int) -> tuple[torch.Tensor, int, int]:
    """``(had_K, K, m)`` with ``n = K * m``: K chosen as the reference chooses it (get_hadK's order of preference),
    the K x K matrix built here.  Raises if n has no such factorisation or no construction is known."""
    if _is_pow2(n):
        return torch.ones((1, 1), dtype=torch.int64), 1, n
    for k in _FACTOR_ORDERS:
        if n % k == 0 and _is_pow2(n // k):
            h = hadamard_matrix(k)
            if h is None:
                raise ValueError(f"no built-in Hadamard matrix of order {k} (n = {n}): pass the matrix explicitly")
            assert torch.equal(h @ h.t(), k * torch.eye(k, dtype=torch.int64))
            return h, k, n // k
    raise ValueError(f"{n} is not K * 2^j for a supported Hadamard order K")


def rotate_rows_kron(w: torch.Tensor, had_k: torch.Tensor) -> torch.Tensor:
    """Rows of ``w`` rotated by ``had_K (x) H_m / sqrt(n)`` in fp64, returned as fp16: the offline rotation of a
    weight over its input dimension that matches :func:`hadamard_kron` on the activations
    (apply_exact_had_to_linear with had_dim = -1, hadamard_utils.py:108-139)."""
    n = w.shape[-1]
    k = had_k.shape[0]
    m = n // k
    z = w.double().reshape(-1, k, m)
    h = 1
    while h < m:                                   # natural-order Walsh-Hadamard transform over the contiguous m
        v = z.reshape(-1, k, m // (2 * h), 2, h)
        z = torch.stack((v[..., 0, :] + v[..., 1, :], v[..., 0, :] - v[..., 1, :]), dim=-2).reshape(-1, k, m)
        h *= 2
    y = torch.einsum("ab,rbt->rat", had_k.to(w.device).double(), z) / math.sqrt(n)
    return y.reshape(w.shape).half()


def hadamard_kron(x: torch.Tensor, had_k: torch.Tensor, out: torch.Tensor | None = None,
                  scratch: torch.Tensor | None = None) -> torch.Tensor:
    """``matmul_hadU_cuda(x, had_k, K)`` on the GPU: fp16 rows ``[R, n]``, ``had_k`` a fp16 ``[K, K]`` device
    tensor, ``n = K * m`` with m == 8 or a power of two >= 256 (the sizes the kernels cover: 1408 = 176 x 8,
    14336 = 28 x 512).  ``out`` may be ``x``.  For m >= 256 the groups of m are transformed by the per-token
    rotation kernel first (one extra pass through ``scratch``, an fp16 buffer of the size of x)."""
    if x.dtype != torch.float16 or not x.is_cuda or not x.is_contiguous():
        raise RuntimeError("hadamard_kron needs a contiguous fp16 CUDA tensor")
    n = x.shape[-1]
    k = had_k.shape[0]
    m = n // k
    if k * m != n or not _is_pow2(m) or not (m == 8 or m >= 256):
        raise RuntimeError(f"row length {n} = {k} x {m}: m must be 8 or a power of two >= 256")
    rows = x.numel() // n
    out = torch.empty_like(x) if out is None else out
    lib = _lib.lib()
    with torch.cuda.device(x.device):
        if m == 8:
            _lib.check(lib.mxmoe_hadamard_kron(x.data_ptr(), out.data_ptr(), had_k.data_ptr(), rows, k, m,
                                               1.0 / math.sqrt(n), 1, current_stream_ptr()))
            return out
        scratch = torch.empty_like(x) if scratch is None else scratch
        t = _lib.TokenQuantArgs()
        t.inp, t.f16, t.k, t.num_tokens, t.rotate = x.data_ptr(), scratch.data_ptr(), m, rows * k, 1
        _lib.check(lib.mxmoe_quant_tokens(C.byref(t), current_stream_ptr()))        # H_m / sqrt(m) over every group
        _lib.check(lib.mxmoe_hadamard_kron(scratch.data_ptr(), out.data_ptr(), had_k.data_ptr(), rows, k, m,
                                           1.0 / math.sqrt(k), 0, current_stream_ptr()))
    return out
