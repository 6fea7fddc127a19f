"""Hadamard rotation restatement (TEST INFRASTRUCTURE ONLY).

Power-of-two sizes (the 2048- and 4096-point rotations of the hidden dimension) and
sizes n = K * 2^j with a K x K Hadamard factor (``hadamard_kron_rows``: the online
rotation of the down-projection input, 1408 = 176 x 8, 14336 = 28 x 512).  Follows ``mxmoe/quant/hadamard_utils.py:62-83`` (``matmul_hadU``,
K == 1 branch: a radix-2 butterfly over adjacent pairs, i.e. the natural-order
Sylvester transform, divided by ``torch.tensor(n).sqrt()``, which is an *fp32*
square root) and ``:89-94`` (``random_hadamard_matrix``: the transform applied
to the rows of ``diag(+-1)``).
"""
from __future__ import annotations

import numpy as np
import torch


def _is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def fwht_rows(x: torch.Tensor) -> torch.Tensor:
    """Un-normalised natural-order Walsh-Hadamard transform over the last dim."""
    n = x.shape[-1]
    assert _is_pow2(n), "only power-of-two sizes are restated"
    y = x.reshape(-1, n).clone()
    h = 1
    while h < n:
        # butterfly on index bit log2(h): (a, b) -> (a + b, a - b)
        v = y.reshape(-1, n // (2 * h), 2, h)
        a = v[:, :, 0, :] + v[:, :, 1, :]
        b = v[:, :, 0, :] - v[:, :, 1, :]
        y = torch.stack((a, b), dim=2).reshape(-1, n)
        h *= 2
    return y.reshape(x.shape)


def hadamard_rows(x: torch.Tensor) -> torch.Tensor:
    """``matmul_hadU(x)`` for power-of-two n (hadamard_utils.py:62-83)."""
    n = x.shape[-1]
    # the reference divides by an fp32-rounded sqrt(n) (0-dim float32 tensor)
    return fwht_rows(x) / torch.tensor(n).sqrt()


def hadamard_kron_rows(x: torch.Tensor, had_k: torch.Tensor) -> torch.Tensor:
    """``matmul_hadU(x)`` for ``n = K * m``, m a power of two, with the K x K factor ``had_k`` that
    ``get_hadK(n)`` returns (hadamard_utils.py:5-59, :62-83; the CUDA form ``matmul_hadU_cuda`` :96-105 computes
    the same thing): the row is viewed as ``[K, m]``, the natural-order Walsh-Hadamard transform runs over
    the m contiguous elements, ``had_k`` mixes the K groups, and the result is divided by the fp32 ``sqrt(n)``:
    ``y[a*m + t] = sum_a' had_k[a, a'] * sum_l (-1)^popcount(t & l) * x[a'*m + l] / sqrt(n)``."""
    n = x.shape[-1]
    k = had_k.shape[0]
    m = n // k
    assert k * m == n and _is_pow2(m)
    z = fwht_rows(x.reshape(-1, k, m))                       # over the contiguous m
    y = torch.einsum("ab,rbt->rat", had_k.to(x.dtype), z)
    return (y.reshape(x.shape)) / torch.tensor(n).sqrt()


def random_hadamard(n: int, generator: torch.Generator | None = None) -> torch.Tensor:
    """``random_hadamard_matrix(n)`` (hadamard_utils.py:89-94), fp64, Q = H(diag(s)).

    The reference draws the signs from torch's global generator; passing a
    generator here draws the same stream from an explicit one.
    """
    s = torch.randint(low=0, high=2, size=(n,), generator=generator).to(torch.float64) * 2 - 1
    return hadamard_rows(torch.diag(s))


def signs_of(q: torch.Tensor) -> np.ndarray:
    """Recover the +-1 diagonal from ``Q = diag(s) H / sqrt(n)`` (first column of H is all ones)."""
    return np.sign(q[:, 0].numpy()).astype(np.int8)
