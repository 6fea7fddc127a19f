"""A device-side wait that runs out: the kernel must end by itself, report where it gave up, and leave the
workspace usable.

Every mbarrier wait of the grouped GEMM is bounded (1 s by default).  The failure is produced on the host: a test
hook of the C ABI (mxmoe_gg_debug) shortens the limit to 20 ms and tells the producer of CTA 0 to leave out one
weight load, so the barrier that load would complete is a flag that nothing sets.  Nothing traps, faults or spins
without a limit; the other CTAs finish their tiles normally.
"""
import time

import numpy as np
import pytest
import torch

from mxmoe_b200 import gg
from mxmoe_b200._lib import MxMoEError
from tests import util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,expanded", [(4, True), (8, False)])
def test_wait_runs_out_then_workspace_recovers(cuda_device, bits, expanded):
    rng = np.random.default_rng(bits)
    c = util.WxAxCase(rng, 300, 512, 512, bits, expanded=expanded)     # CTA 0 owns tile 0: four pipeline stages
    g = gg.GroupedGemm([c.problem(cuda_device)])
    g.run(kernel="swap")
    g.check()
    assert np.array_equal(c.C.cpu().numpy().view(np.uint16), c.ref.view(np.uint16))

    g.debug(timeout_ms=20, skip_stage=2)
    t0 = time.time()
    g.run(kernel="swap")
    with pytest.raises(MxMoEError) as err:
        g.check()
    elapsed = time.time() - t0
    assert err.value.status == 5                                        # MXMOE_ERR_DEVICE
    msg = str(err.value)
    # the first role whose wait ran out is named: the warp waiting for the missing weights (a converter, or the warp
    # that forwards operands to the MMA issuer), or the epilogue, which waits for the accumulator of the same tile
    assert "bounded wait ran out" in msg and "tile 0" in msg, msg
    assert any(f"role {r}" in msg for r in ("converter", "mma(operands)", "epilogue")), msg
    assert elapsed < 5.0, f"the launch took {elapsed:.1f} s to give up"

    # the report was taken and cleared: the same workspace runs again, bit-exact
    g.debug(timeout_ms=0, skip_stage=-1)
    c.C.fill_(float("nan"))
    g.run(kernel="swap")
    g.check()
    assert np.array_equal(c.C.cpu().numpy().view(np.uint16), c.ref.view(np.uint16))
