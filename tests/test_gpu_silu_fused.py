"""silu(gate) * up in the epilogue of the gate_up GEMM (out_mode 2).

The fused epilogue must produce, bit for bit, what the two-step path produces: the scaled fp16 [M, 2 I] rows of
out_mode 0 followed by the first half of the stand-alone silu-mul kernel (`silu_mul_then_quant_kernel`,
ref_bind.cu:701-716: fp16(fp16(silu(gate)) * up)).  A float32 torch evaluation of the same formula pins the
meaning (rel-L2 <= 2e-3: the device uses the fast exponential).
"""
import numpy as np
import pytest
import torch

from mxmoe_b200 import gg, verify, workload
from mxmoe_b200._lib import MxMoEError
from mxmoe_b200.layer import MoELayer
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["swap", "swap-small"])
def gg_tiles(request, monkeypatch):
    monkeypatch.setenv("MXMOE_GG_KERNEL", "swap")
    if request.param == "swap-small":
        monkeypatch.setenv("MXMOE_GG_TILES", "small")
    else:
        monkeypatch.delenv("MXMOE_GG_TILES", raising=False)
    yield request.param


# (M, I, K): one tile; one row; ragged rows; the layer's shape with ragged rows; several channel tiles
SHAPES = [(128, 64, 128), (1, 128, 128), (17, 128, 256), (300, 1408, 2048), (200, 704, 512)]


def _case(kind, rng, m, inter, k):
    if kind == "fp16":
        return util.Fp16Case(rng, m, 2 * inter, k)
    return util.WxAxCase(rng, m, 2 * inter, k, 8 if kind == "w8a8" else 4, expanded=(kind == "w4a4x"))


def _fused_problem(c, dev):
    """The case's problem once more with out_mode 2 and its own [M, I] output."""
    p = c.problem(dev)
    two_step = c.C
    p2 = c.problem(dev)
    p2.out_mode = gg.OUT_SILU
    p2.C = torch.full((c.m, c.n // 2), float("nan"), dtype=torch.float16, device=dev)
    return p, two_step, p2


@pytest.mark.parametrize("kind", ["w4a4", "w4a4x", "w8a8", "fp16"])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_epilogue_equals_two_steps(cuda_device, kind, shape):
    rng = np.random.default_rng(hash((kind,) + shape) % 2**32)
    c = _case(kind, rng, *shape)
    p, rows, p2 = _fused_problem(c, cuda_device)
    util.run([p])
    util.run([p2])
    want = verify._silu_rows(rows)
    got = p2.C
    assert not torch.isnan(got).any()
    diff = int((got.view(torch.int16) != want.view(torch.int16)).sum().item())
    assert diff == 0, f"{diff} of {got.numel()} values differ"
    g, u = rows[:, : c.n // 2].float(), rows[:, c.n // 2:].float()
    ref = (torch.nn.functional.silu(g).half().float() * u).half()
    ok = torch.isfinite(ref) & torch.isfinite(got)          # the random scales let a few products leave fp16's range
    assert ok.float().mean() > 0.5
    err = float((got[ok].float() - ref[ok].float()).norm() / ref[ok].float().norm())
    assert err <= 2e-3, err


def test_fused_and_plain_problems_in_one_launch(cuda_device):
    """Problems with and without the fused epilogue, of three schemes, share a launch (and its tile walk)."""
    rng = np.random.default_rng(5)
    cases = [_case(k, rng, m, i, kk) for k, m, i, kk in
             (("w4a4x", 190, 192, 256), ("w8a8", 33, 64, 384), ("fp16", 177, 128, 128), ("w4a4", 64, 256, 128))]
    plain, fused, rows = [], [], []
    for c in cases:
        p, r, p2 = _fused_problem(c, cuda_device)
        plain.append(p)
        rows.append(r)
        fused.append(p2)
    extra = util.W4A16Case(rng, 70, 256, 256)
    util.run(plain)
    util.run([fused[0], plain[1], extra.problem(cuda_device), fused[2], fused[3], fused[1]], num_ctas=3)
    for r, p2 in zip(rows, fused):
        assert torch.equal(verify._silu_rows(r).view(torch.int16), p2.C.view(torch.int16))


def test_fused_epilogue_argument_checks(cuda_device):
    rng = np.random.default_rng(6)
    c = util.W4A16Case(rng, 16, 256, 128)
    p = c.problem(cuda_device)
    p.out_mode = gg.OUT_SILU
    with pytest.raises(MxMoEError):
        gg.GroupedGemm([p])
    c = util.WxAxCase(rng, 16, 192, 128, 8)      # I = 96 is not a multiple of 64
    p = c.problem(cuda_device)
    p.out_mode = gg.OUT_SILU
    with pytest.raises(MxMoEError):
        gg.GroupedGemm([p])


def _layers(spec, dev, **kw):
    gate_up, down, signs, _ = workload.build_layer_weights(spec, device=dev, **{k: v for k, v in kw.items() if k == "online_had"})
    mk = lambda fuse: MoELayer(spec.num_experts, spec.topk, spec.hidden, spec.inter, gate_up, down, spec.tokens,
                               shared_inter=spec.shared_inter, signs=signs, rotate=spec.rotate, device=dev,
                               fuse_silu=fuse, **kw)
    return mk(True), mk(False)


@pytest.mark.parametrize("scheme,shared", [("w4a4_g-1_sym", False), ("w8a8_g-1_sym", True), ("fp16", False)])
def test_layer_with_fused_silu_equals_layer_without(cuda_device, scheme, shared, gg_tiles):
    if gg_tiles != "swap":
        pytest.skip("layers choose their own tile geometry")
    spec = workload.LayerSpec("tiny", 6, 2, 512, 256, 512 if shared else 0, 70, "zipf", 1.2, True,
                              scheme != "fp16", scheme)
    hidden = workload.make_hidden(spec).to(cuda_device)
    ids, wts = workload.make_routing(spec)
    ids, wts = ids.to(cuda_device), wts.to(cuda_device)
    fused, plain = _layers(spec, cuda_device)
    out_f = fused.forward(hidden, ids, wts).clone()
    out_p = plain.forward(hidden, ids, wts).clone()
    fused.check()
    plain.check()
    assert fused._core.fused_silu and not plain._core.fused_silu
    R = spec.tokens * spec.topk
    assert torch.equal(fused._core.q2.view(torch.int16), plain._core.q2.view(torch.int16))
    assert torch.equal(fused._core.s2[:R].view(torch.int16), plain._core.s2[:R].view(torch.int16))
    assert torch.equal(fused.o2.view(torch.int16), plain.o2.view(torch.int16))
    assert torch.equal(out_f.view(torch.int16), out_p.view(torch.int16))
    rep = verify.check_layer(fused)
    assert rep["ok"], rep
    assert all(p.get("silu_mismatch", 0) == 0 for p in rep["problems"])


def test_weight_only_layer_keeps_the_two_step_path(cuda_device, gg_tiles):
    if gg_tiles != "swap":
        pytest.skip("layers choose their own tile geometry")
    spec = workload.LayerSpec("tiny", 6, 2, 512, 256, 0, 40, "zipf", 1.2, True, False, "w4a16_g128_asym")
    fused, _ = _layers(spec, cuda_device)
    hidden = workload.make_hidden(spec).to(cuda_device)
    ids, wts = workload.make_routing(spec)
    fused.forward(hidden, ids.to(cuda_device), wts.to(cuda_device))
    fused.check()
    assert not fused._core.fused_silu
