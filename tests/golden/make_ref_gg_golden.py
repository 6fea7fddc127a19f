"""Reduce the outputs of the reference's own GroupGEMM kernel to a small committed fixture.

The outputs come from ``tests/ref_gg_worker.py`` (the reference's generated kernel, built by
``make -C oracle refgg REF_ROOT=<MxMoE checkout>``, run on a B200):

    python tests/ref_gg_worker.py --out /tmp/ref_gg_out.npz          # on the GPU machine
    python tests/golden/make_ref_gg_golden.py /tmp/ref_gg_out.npz    # writes tests/golden/ref_gg_kernel.npz

Kept per case of ``tests/ref_cases.py``: all rows of the one-tile cases (N <= 256), otherwise the first
four and the last four rows.  The inputs are not stored; they are regenerated from the seeds.  The
w4a4_g128 cases are left out: that branch of the reference reads per-group scales from shared-memory
slots it has not filled (cta_gemm.cuh:668-689: the slot pointer is advanced with the stage index of the
PREVIOUS load), so its output is not a function of the inputs.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests import ref_cases  # noqa: E402


def rows_kept(m: int, n: int) -> np.ndarray:
    return np.arange(m) if n <= 256 else np.concatenate((np.arange(4), np.arange(m - 4, m)))


def main() -> None:
    src = np.load(sys.argv[1])
    out = {}
    for i, (scheme, m, n, _k, _v) in enumerate(ref_cases.CASES):
        if f"c{i}" in src and scheme != "w4a4_g128_sym":
            out[f"c{i}"] = src[f"c{i}"][rows_kept(m, n)]
    np.savez_compressed(os.path.join(HERE, "ref_gg_kernel.npz"), **out)
    print(sorted(out), sum(v.nbytes for v in out.values()))


if __name__ == "__main__":
    main()
