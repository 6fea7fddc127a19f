"""This library's grouped GEMM against the reference's OWN GroupGEMM kernel, both run here on the GPU.

The reference's generated fused kernel (mma.sync code for sm_80/89, compose_kernel.py:503-530) is built for
sm_100a into ``oracle/_ref/libref_gg.so`` (``make -C oracle refgg``) and run by a child process
(``tests/ref_gg_worker.py``) on the seeded cases of ``tests/ref_cases.py``; this process runs the same cases
through the C ABI and compares:

* fp16, w4a16 group-128 and w4a16 per-channel: rel-L2 <= 1e-3 (the bound stated for fp16 outputs against the reference's
  GroupGEMM; the two kernels accumulate in fp32 in different orders);
* w8a8 / w4a4: the same bits.  The reference kernel scales channel c with the weight scale of channel
  ``8*(c//8) + (c%8)//2 + c%2`` (oracle.gemm.ref_kernel_scale_b_index), so the comparison is made (a) with
  weight scales constant over blocks of 8 channels, where that map is the identity, and (b) on general scales
  by handing this library the scales already gathered through the map.  Both are bit-exact; with the true
  scales this library follows the quantiser's meaning (channel c, scale c), as the fp32 dequant-then-matmul
  loop does.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import gemm as og
from oracle import pack as op
from mxmoe_b200 import gg
from tests import ref_cases, ref_oracle, util

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "_ref", "libref_gg.so")
SCHEMES = ("fp16", "w8a8_g-1_sym", "w4a4_g-1_sym", "w4a16_g128_asym", "w4a16_g-1_asym")
REL_L2 = 1e-3


@pytest.fixture(scope="module")
def ref_out(cuda_device, tmp_path_factory):
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libref_gg.so is not built (make -C oracle refgg REF_ROOT=<MxMoE checkout>)")
    out = str(tmp_path_factory.mktemp("refgg") / "ref.npz")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_gg_worker.py"), "--out", out,
                          "--schemes", ",".join(SCHEMES)], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    return np.load(out)


def run_ours(c: dict, dev, remap_sb: bool = False) -> np.ndarray:
    a_bits, w_bits, gsize, sym = ref_cases.QPARAMS[c["scheme"]]
    m, n, k = c["m"], c["n"], c["k"]
    C = torch.full((m, n), float("nan"), dtype=torch.float16, device=dev)
    keep = []
    if a_bits < 16:
        sb = c["sb"][:, 0]
        if remap_sb:
            sb = sb[og.ref_kernel_scale_b_index(n)]
        t = [util.t16(op.pack_k(c["qa"], a_bits), dev), util.t16(op.pack_k(c["qb"], w_bits), dev),
             util.t16(np.ascontiguousarray(c["sa"][:, 0]), dev), util.t16(np.ascontiguousarray(sb), dev)]
        p = gg.Problem(A=t[0], B=t[1], C=C, M=m, N=n, K=k, qparams=(a_bits, w_bits, gsize, True), scale_a=t[2],
                       scale_b=t[3])
    elif w_bits == 16:
        t = [util.t16(c["a"], dev), util.t16(c["b"], dev)]
        p = gg.Problem(A=t[0], B=t[1], C=C, M=m, N=n, K=k, qparams=util.Q_FP16)
    else:
        t = [util.t16(c["a"], dev), util.t16(op.pack_n4(c["qb"]), dev),
             util.t16(op.group_major_scales(c["sb"], c["zb"]), dev)]
        p = gg.Problem(A=t[0], B=t[1], C=C, M=m, N=n, K=k, qparams=(16, 4, gsize, False), scale_b=t[2])
    keep.append(t)
    util.run([p])
    return C.cpu().numpy()


CASE_IDS = [i for i, cs in enumerate(ref_cases.CASES) if cs[0] in SCHEMES]


@pytest.mark.parametrize("idx", CASE_IDS)
def test_matches_reference_kernel(cuda_device, ref_out, idx):
    scheme, m, n, k, variant = ref_cases.CASES[idx]
    c = ref_cases.make(idx)
    want = ref_out[f"c{idx}"]
    if ref_cases.QPARAMS[scheme][0] < 16:
        got = run_ours(c, cuda_device, remap_sb=True)
        diff = np.count_nonzero(got.view(np.uint16) != want.view(np.uint16))
        assert diff == 0, f"{diff} of {got.size} fp16 words differ from the reference kernel"
        if variant == "b8":
            got = run_ours(c, cuda_device)
            assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
        else:
            # with the true scales: this library == the oracle (channel c, scale c), the reference kernel is not
            got = run_ours(c, cuda_device)
            assert np.array_equal(got.view(np.uint16), ref_oracle.oracle_output(c).view(np.uint16))
    else:
        got = run_ours(c, cuda_device)
        err = og.rel_l2(got, want)
        print(f"{scheme} {m}x{n}x{k}: rel-L2 vs the reference kernel {err:.2e}")
        assert err <= REL_L2, err
