"""Shared helpers of the parity tests: build grouped-GEMM problems from numpy data
(packed with the oracle's restatement of the reference layouts) and run them
through the C ABI."""
import numpy as np
import torch

from oracle import gemm as og
from oracle import pack as op
from mxmoe_b200 import gg

Q_FP16 = (16, 16, -1, True)
Q_W8A8 = (8, 8, -1, True)
Q_W4A4 = (4, 4, -1, True)
Q_W4A16 = (16, 4, 128, False)


def t16(a, dev):
    """numpy uint16/float16/int16 array -> CUDA tensor with the same bits (int16 carrier for packed words)."""
    if a.dtype == np.float16:
        return torch.from_numpy(a.copy()).to(dev)
    return torch.from_numpy(a.view(np.int16).copy()).to(dev)


def rand_codes(rng, rows, k, bits):
    hi = 2 ** (bits - 1) - 1
    return rng.integers(-hi, hi + 1, (rows, k), dtype=np.int32)


def rand_scales(rng, n, lo=0.002, hi=0.02):
    return rng.uniform(lo, hi, n).astype(np.float16)


class WxAxCase:
    """Random w8a8 / w4a4 problem with known integer codes."""

    def __init__(self, rng, m, n, k, bits, expanded=False):
        self.m, self.n, self.k, self.bits = m, n, k, bits
        self.expanded = expanded      # 4-bit activations handed over as one byte 16*q per code
        self.qa = rand_codes(rng, m, k, bits)
        self.qb = rand_codes(rng, n, k, bits)
        self.sa = rand_scales(rng, m, 0.01, 0.5)
        self.sb = rand_scales(rng, n)
        self.acc = og.int_accumulate(self.qa, self.qb)
        self.ref = og.wxax_epilogue(self.acc, self.sa, self.sb)

    def problem(self, dev, out_mode=gg.OUT_FP16):
        if self.expanded:
            self.A = torch.from_numpy(op.expand_k4(self.qa).copy()).to(dev)
        else:
            self.A = t16(op.pack_k(self.qa, self.bits), dev)
        self.B = t16(op.pack_k(self.qb, self.bits), dev)
        self.SA = t16(self.sa, dev)
        self.SB = t16(self.sb, dev)
        if out_mode == gg.OUT_ACC:
            self.C = torch.full((self.m, self.n), -12345, dtype=torch.int32, device=dev)
        else:
            self.C = torch.full((self.m, self.n), float("nan"), dtype=torch.float16, device=dev)
        q = Q_W8A8 if self.bits == 8 else Q_W4A4
        return gg.Problem(A=self.A, B=self.B, C=self.C, M=self.m, N=self.n, K=self.k, qparams=q,
                          scale_a=self.SA, scale_b=self.SB, out_mode=out_mode, a_expanded=1 if self.expanded else 0)


class Fp16Case:
    def __init__(self, rng, m, n, k):
        self.m, self.n, self.k = m, n, k
        self.a = rng.standard_normal((m, k)).astype(np.float16)
        self.b = (rng.standard_normal((n, k)) * 0.05).astype(np.float16)
        self.ref = og.fp_gemm(self.a, self.b)

    def problem(self, dev, out_mode=gg.OUT_FP16):
        self.A, self.B = t16(self.a, dev), t16(self.b, dev)
        dt = torch.float32 if out_mode == gg.OUT_ACC else torch.float16
        self.C = torch.full((self.m, self.n), float("nan"), dtype=dt, device=dev)
        return gg.Problem(A=self.A, B=self.B, C=self.C, M=self.m, N=self.n, K=self.k, qparams=Q_FP16,
                          out_mode=out_mode)


class W4A16Case:
    def __init__(self, rng, m, n, k):
        self.m, self.n, self.k = m, n, k
        self.a = rng.standard_normal((m, k)).astype(np.float16)
        self.q = rng.integers(0, 16, (n, k), dtype=np.int32)
        g = k // 128
        self.s = rng.uniform(0.001, 0.01, (n, g)).astype(np.float16)
        self.z = rng.uniform(-0.08, -0.01, (n, g)).astype(np.float16)
        self.w = og.dequant_w4a16(self.q, self.s, self.z)
        self.ref = og.fp_gemm(self.a, self.w)

    def problem(self, dev, out_mode=gg.OUT_FP16):
        self.A = t16(self.a, dev)
        self.B = t16(op.pack_n4(self.q), dev)
        self.SB = t16(op.group_major_scales(self.s, self.z), dev)
        dt = torch.float32 if out_mode == gg.OUT_ACC else torch.float16
        self.C = torch.full((self.m, self.n), float("nan"), dtype=dt, device=dev)
        return gg.Problem(A=self.A, B=self.B, C=self.C, M=self.m, N=self.n, K=self.k, qparams=Q_W4A16,
                          scale_b=self.SB, out_mode=out_mode)


# launch geometry used when a test does not ask for one: 0 = library default, a large positive number =
# single-CTA kernel on every SM, a large negative number = CTA-pair kernel on every SM.  tests/test_gpu_gemm.py runs with both.
DEFAULT_CTAS = 0


def run(problems, num_ctas=None):
    g = gg.GroupedGemm(problems)
    g.run(DEFAULT_CTAS if num_ctas is None else num_ctas)
    g.check()
    return g
