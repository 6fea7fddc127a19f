"""The CPU oracle against outputs of the reference's OWN GroupGEMM kernel.

``tests/golden/ref_gg_kernel.npz`` holds fp16 outputs of the reference's generated fused kernel
(compose_kernel.py:503-530; branches cta_gemm.cuh:7-107, :112-286, :291-421, :423-608) compiled for
sm_100a and run on a B200 by ``tests/ref_gg_worker.py`` on the seeded cases of ``tests/ref_cases.py``
(``tests/golden/make_ref_gg_golden.py`` made the fixture).  This pins the two floating-point steps of the
oracle that no host code of the reference covers: the w8a8 / w4a4 scale epilogue (bit for bit) and the
w4a16 dequantisation + fp32 accumulation (rel-L2; the accumulation order of the device differs).
"""
import os

import numpy as np
import pytest

from oracle import gemm as og
from tests import ref_cases, ref_oracle
from tests.golden.make_ref_gg_golden import rows_kept

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gg_kernel.npz"))
IDS = [i for i in range(len(ref_cases.CASES)) if f"c{i}" in GOLD.files]


@pytest.mark.parametrize("idx", IDS)
def test_oracle_matches_reference_kernel(idx):
    scheme, m, n, k, variant = ref_cases.CASES[idx]
    c = ref_cases.make(idx)
    want = GOLD[f"c{idx}"]
    rows = rows_kept(m, n)
    a_bits = ref_cases.QPARAMS[scheme][0]
    if a_bits < 16:
        # integer schemes: same bits, once the oracle applies the weight scales through the reference kernel's
        # channel map (a defect of the reference, see oracle.gemm.ref_kernel_scale_b_index); with weight scales
        # that are constant over 8 channels ("b8") the map changes nothing and the plain oracle is bit-equal too
        got = ref_oracle.oracle_output(c, ref_scale_index=True)[rows]
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
        plain = ref_oracle.oracle_output(c)[rows]
        if variant == "b8":
            assert np.array_equal(plain.view(np.uint16), want.view(np.uint16))
        else:
            assert og.rel_l2(plain, want) > 0.1      # the reference's defect is visible on general scales
    else:
        got = ref_oracle.oracle_output(c)[rows]
        assert og.rel_l2(got, want) <= 1e-4, og.rel_l2(got, want)
