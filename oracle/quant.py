"""Min/max quantiser restatement (TEST INFRASTRUCTURE ONLY).

Follows ``mxmoe/quant/quant.py:40-84`` (``quant_minmax``) and ``:87-109``
(``Quantizer``).  All arithmetic runs in the dtype of the tensor that is passed
in, exactly like the reference: an fp16 activation is scaled, divided and
rounded in fp16 (torch's CPU kernels evaluate each fp16 op in fp32 and round the
result to fp16, which is the correctly rounded fp16 result for + - * /).
"""
from __future__ import annotations

import torch


def code_range(bits: int, sym: bool) -> tuple[int, int]:
    """Integer code interval: quant.py:66-67 (and quantize.cuh:245-246)."""
    if sym:
        hi = 2 ** (bits - 1) - 1
        return -hi, hi
    return 0, 2 ** bits - 1


def minmax_quantize(t: torch.Tensor, bits: int, gsize: int, sym: bool):
    """Return ``(codes, scale, zero)``; quant.py:40-84 with clip == (1, 1).

    ``codes`` has the shape and dtype of ``t`` (integer valued), ``scale`` and
    ``zero`` have shape ``[t.numel() // g, 1]`` (``zero`` is the python int 0 for
    the symmetric scheme, as in the reference).
    """
    g = t.shape[-1] if gsize == -1 else gsize
    lo, hi = code_range(bits, sym)
    rows = t.reshape(-1, g)
    if sym:
        scale = rows.abs().amax(dim=-1, keepdim=True) / hi
        zero = 0
        scaled = rows / scale
    else:
        gmin, gmax = rows.aminmax(dim=-1, keepdim=True)
        scale = (gmax - gmin) / hi
        zero = gmin
        scaled = (rows - zero) / scale
    # clamp first, then round half to even (quant.py:82)
    codes = scaled.clamp(lo, hi).round()
    return codes.reshape(t.shape), scale, zero


def dequantize(codes: torch.Tensor, scale, zero, gsize: int) -> torch.Tensor:
    """quant.py:99-102."""
    g = codes.shape[-1] if gsize == -1 else gsize
    return (codes.reshape(-1, g) * scale + zero).reshape(codes.shape)


def fake_quant(t: torch.Tensor, bits: int, gsize: int, sym: bool) -> torch.Tensor:
    """quant.py:104-106: quantise and immediately dequantise; 16 bits is the identity."""
    if bits >= 16:
        return t
    codes, scale, zero = minmax_quantize(t, bits, gsize, sym)
    return dequantize(codes, scale, zero, gsize)


def scheme_tuple(name: str) -> tuple[int, int, int, bool]:
    """``"w4a4_g-1_sym"`` -> ``(a_bits, w_bits, gsize, sym)``; ``"fp16"`` -> (16, 16, -1, True).

    Same string grammar as gen_workload.py:43-48 / tile_config.py:288-294.
    """
    if name in ("fp16", "w16a16"):
        return 16, 16, -1, True
    w = int(name.split("w")[1].split("a")[0])
    a = int(name.split("a")[1].split("_g")[0])
    g = int(name.split("_g")[1].split("_")[0])
    return a, w, g, "asym" not in name


def fake_quant_expert_loop(x_per_expert, w_per_expert, schemes, threads: int | None = None):
    """The reference's CPU-runnable path for one linear block of every expert.

    ``y_e = fake_quant_act(x_e) @ fake_quant_weight(W_e).T`` with the activation
    hook of quant.py:126-130 and the weight fake-quant of quant.py:460-461; the
    matmul itself is what ``nn.Linear`` does in the evaluation forward
    (evaluator.py:23-57).  Inputs are fp16-valued; the product is evaluated in
    fp32 (fp16 matmul on CPU is not what the reference runs on its GPU either).
    Activations always use per-token symmetric quantisation (qconfig.py:11-13).
    """
    if threads:
        torch.set_num_threads(threads)
    outs = []
    for x, w, name in zip(x_per_expert, w_per_expert, schemes):
        a_bits, w_bits, g, sym = scheme_tuple(name)
        xq = fake_quant(x, a_bits, -1, True) if a_bits < 16 else x
        wq = fake_quant(w, w_bits, g, sym) if w_bits < 16 else w
        outs.append((xq.float() @ wq.float().t()).half())
    return outs
