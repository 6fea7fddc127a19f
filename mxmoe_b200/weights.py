"""Offline weight preparation: quantise a ``[N, K]`` fp16 weight and pack it in the
reference's operand layouts.

The quantiser follows ``mxmoe/quant/quant.py:40-84`` (min/max, per output channel
or per group of ``gsize`` input channels, arithmetic in the weight's dtype); the
packed layouts follow the reference's host packers
(``mxmoe/kernels/src/include/quantize.cuh:299-475``): K-packed two's-complement
fields for w8a8 / w4a4, N-packed fragment-permuted nibbles plus group-major
(scale, zero) pairs for w4a16 group-128.  Everything here is torch tensor
arithmetic and runs on whichever device the weight lives on.
"""
from __future__ import annotations

import dataclasses

import torch

SCHEMES = ("fp16", "w8a8_g-1_sym", "w4a4_g-1_sym", "w4a16_g128_asym")     # the schemes of the benchmark configurations
EXTRA_SCHEMES = ("w4a16_g-1_asym",)                                        # per-channel weight-only (cta_gemm.cuh:112-286)


def parse_scheme(name: str) -> tuple[int, int, int, bool]:
    """``"w4a4_g-1_sym"`` -> ``(a_bits, w_bits, gsize, sym)`` (grammar of tile_config.py:288-294)."""
    if name in ("fp16", "w16a16", "w16a16_g-1_sym"):
        return 16, 16, -1, True
    try:
        w = int(name.split("w")[1].split("a")[0])
        a = int(name.split("a")[1].split("_g")[0])
        g = int(name.split("_g")[1].split("_")[0])
    except (IndexError, ValueError) as exc:
        raise ValueError(f"malformed scheme string {name!r}") from exc
    return a, w, g, "asym" not in name


def scheme_name(a_bits: int, w_bits: int, gsize: int, sym: bool) -> str:
    if a_bits >= 16 and w_bits >= 16:
        return "fp16"
    return f"w{w_bits}a{a_bits}_g{gsize}_{'sym' if sym else 'asym'}"


def weight_bits(name: str) -> float:
    """Effective bits per weight incl. group parameters (bits_solver.py:581-593)."""
    a, w, g, sym = parse_scheme(name)
    if w >= 16:
        return 16.0
    if g == -1:
        return float(w)
    return w + (16.0 if sym else 32.0) / g


@dataclasses.dataclass
class PackedWeight:
    """One linear block ready for the grouped GEMM."""
    scheme: str
    n: int
    k: int
    data: torch.Tensor            # fp16 [N,K] | int16 [N,K/2] | int16 [N,K/4] | int16 [N/4,K]
    scale: torch.Tensor | None    # fp16 [N] | fp16 [K/128, N, 2] | None
    codes: torch.Tensor | None = None   # integer codes [N,K] (kept for checking only)

    @property
    def qparams(self) -> tuple[int, int, int, bool]:
        return parse_scheme(self.scheme)

    def nbytes(self) -> int:
        n = self.data.numel() * self.data.element_size()
        if self.scale is not None:
            n += self.scale.numel() * self.scale.element_size()
        return n

    def to(self, device) -> "PackedWeight":
        return dataclasses.replace(
            self, data=self.data.to(device), scale=None if self.scale is None else self.scale.to(device),
            codes=None if self.codes is None else self.codes.to(device))


def quantize_minmax(t: torch.Tensor, bits: int, gsize: int, sym: bool):
    """Integer codes, scale and zero of ``t`` (quant.py:40-84, clip = (1, 1))."""
    g = t.shape[-1] if gsize == -1 else gsize
    rows = t.reshape(-1, g)
    if sym:
        qmax = (1 << (bits - 1)) - 1
        scale = rows.abs().amax(dim=-1, keepdim=True) / qmax
        zero = torch.zeros_like(scale)
        codes = (rows / scale).clamp(-qmax, qmax).round()
    else:
        qmax = (1 << bits) - 1
        lo, hi = rows.aminmax(dim=-1, keepdim=True)
        scale = (hi - lo) / qmax
        zero = lo
        codes = ((rows - zero) / scale).clamp(0, qmax).round()
    return codes.reshape(t.shape), scale, zero


def pack_along_k(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """``[R, K]`` integer codes -> int16 ``[R, K*bits/16]``; first k in the top field (quantize.cuh:457-470)."""
    p = 16 // bits
    r, k = codes.shape
    if k % p:
        raise ValueError(f"K={k} is not a multiple of {p}")
    f = (codes.to(torch.int32) & ((1 << bits) - 1)).reshape(r, k // p, p)
    shifts = torch.tensor([bits * (p - 1 - i) for i in range(p)], dtype=torch.int32, device=codes.device)
    return (f << shifts).sum(dim=-1).to(torch.int16)


def pack_along_n4(codes: torch.Tensor) -> torch.Tensor:
    """``[N, K]`` codes in 0..15 -> int16 ``[N/4, K]`` in the layout of ``permute_weight`` +
    ``pack_weightonly`` (quantize.cuh:318-421): with ``n = 32 nb + 8 f + r`` and ``k = 16 kb + 8 c + d``
    the code sits in word ``(8 nb + r, 16 kb + 8 (f >> 1) + d)`` at nibble ``2 (f & 1) + c``."""
    n, k = codes.shape
    if n % 32 or k % 16:
        raise ValueError(f"w4a16 packing needs N % 32 == 0 and K % 16 == 0 (N={n}, K={k})")
    c = (codes.to(torch.int32) & 0xF).reshape(n // 32, 2, 2, 8, k // 16, 2, 8)  # nb fh fl r kb c d
    out = torch.zeros((n // 32, 8, k // 16, 2, 8), dtype=torch.int32, device=codes.device)  # nb r kb fh d
    for fl in range(2):
        for cc in range(2):
            out |= c[:, :, fl, :, :, cc, :].permute(0, 2, 3, 1, 4) << (4 * (2 * fl + cc))
    return out.reshape(n // 4, k).to(torch.int16)


def unpack_along_k(words: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of :func:`pack_along_k`: int16 ``[R, W]`` -> int8 codes ``[R, W*16/bits]`` (two's complement fields)."""
    p = 16 // bits
    w = words.to(torch.int32) & 0xFFFF
    shifts = torch.tensor([bits * (p - 1 - i) for i in range(p)], dtype=torch.int32, device=words.device)
    f = (w.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    f = torch.where(f >= (1 << (bits - 1)), f - (1 << bits), f)
    return f.reshape(words.shape[0], -1).to(torch.int8)


def unpack_along_n4(words: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_along_n4`: int16 ``[N/4, K]`` -> int8 codes ``[N, K]`` in 0..15."""
    n4, k = words.shape
    n = n4 * 4
    w = (words.to(torch.int32) & 0xFFFF).reshape(n // 32, 8, k // 16, 2, 8)     # nb r kb fh d
    codes = torch.zeros((n // 32, 2, 2, 8, k // 16, 2, 8), dtype=torch.int32, device=words.device)  # nb fh fl r kb c d
    for fl in range(2):
        for cc in range(2):
            codes[:, :, fl, :, :, cc, :] = ((w >> (4 * (2 * fl + cc))) & 0xF).permute(0, 3, 1, 2, 4)
    return codes.reshape(n, k).to(torch.int8)


def prepare_weight(w: torch.Tensor, scheme: str, keep_codes: bool = False) -> PackedWeight:
    """Quantise and pack one ``[N, K]`` fp16 weight for ``scheme``."""
    if w.dim() != 2:
        raise ValueError("weight must be [N, K]")
    a_bits, w_bits, g, sym = parse_scheme(scheme)
    n, k = w.shape
    name = scheme_name(a_bits, w_bits, g, sym)
    if name not in SCHEMES + EXTRA_SCHEMES:
        raise ValueError(f"scheme {scheme!r} is not supported (supported: {SCHEMES + EXTRA_SCHEMES})")
    if name == "fp16":
        return PackedWeight(name, n, k, w.to(torch.float16).contiguous(), None)
    codes, scale, zero = quantize_minmax(w, w_bits, g, sym)
    if name in ("w8a8_g-1_sym", "w4a4_g-1_sym"):
        data = pack_along_k(codes, w_bits)
        sc = scale.reshape(n).to(torch.float16).contiguous()
    else:  # w4a16_g128_asym, w4a16_g-1_asym (one group = the whole row)
        gs = k if g == -1 else g
        if k % gs or k % 64:
            raise ValueError(f"scheme {name} needs K % {max(gs if g != -1 else 64, 64)} == 0 (K={k})")
        data = pack_along_n4(codes)
        ng = k // gs
        s = scale.reshape(n, ng).to(torch.float16)
        z = zero.reshape(n, ng).to(torch.float16)
        sc = torch.stack((s.t(), z.t()), dim=-1).contiguous()        # [K/g, N, 2] (quantize.cuh:299-315)
    return PackedWeight(name, n, k, data.contiguous(), sc, codes.to(torch.int8) if keep_codes else None)
