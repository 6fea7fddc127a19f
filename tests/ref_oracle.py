"""CPU oracle result of a case of tests/ref_cases.py (shared by the CPU and the GPU parity tests)."""
import numpy as np

from oracle import gemm as og
from tests import ref_cases


def oracle_output(c: dict, ref_scale_index: bool = False) -> np.ndarray:
    """fp16 [M, N] result of case ``c`` by the CPU oracle.  ``ref_scale_index``: apply the per-channel weight
    scales through the reference kernel's channel map (oracle.gemm.ref_kernel_scale_b_index)."""
    a_bits, w_bits, gsize, _sym = ref_cases.QPARAMS[c["scheme"]]
    if a_bits < 16:
        assert gsize == -1
        sb = c["sb"][:, 0]
        if ref_scale_index:
            sb = sb[og.ref_kernel_scale_b_index(sb.size)]
        return og.wxax_epilogue(og.int_accumulate(c["qa"], c["qb"]), c["sa"][:, 0], sb)
    if w_bits == 16:
        return og.fp_gemm(c["a"], c["b"])
    w = og.dequant_w4a16(c["qb"], c["sb"], c["zb"], gsize if gsize > 0 else c["k"])
    return og.fp_gemm(c["a"], w)
