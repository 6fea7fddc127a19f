"""The CPU-runnable correctness layer of the benchmark configurations on the GPU, at full size:
Qwen1.5-MoE shape (60 experts, hidden 2048, intermediate 1408, top-4), 512 tokens, w4a4 per-token /
per-channel with Hadamard-rotated activations - and the golden slice of the same configuration that the
reference's own Python produced (tests/golden/layer_w4a4_had.npz).
"""
import os

import numpy as np
import pytest
import torch

from oracle import gemm as og
from oracle import pack as op
from mxmoe_b200 import gg, ops, verify, workload
from mxmoe_b200.layer import MoELayer
from tests import util
from tests.test_gpu_layer import _oracle_layer, TOL_FAKEQUANT

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("fuse_silu", [False, True])
def test_config1_full_layer(cuda_device, fuse_silu):
    """All 60 experts, 512 tokens.  int32 accumulators and scaled outputs of the hottest, a median and the coldest
    expert bit-exact (both linear blocks); every expert's rows and the layer output within 2e-2 of the fp32
    dequant-then-matmul loop of the oracle (the reference's torch path).  With silu(gate) * up in the first GEMM's
    epilogue (the layer's default) the gate_up rows are not stored: the self-check then launches the three experts'
    problems on their own and the layer's silu rows must be the bits of the two-step path."""
    spec = workload.CONFIGS["qwen15-w4a4-512"]
    hidden = workload.make_hidden(spec)
    ids, wts = workload.make_routing(spec)
    gate_up, down, signs, (gu_s, dn_s) = workload.build_layer_weights(spec, device=cuda_device)
    lay = MoELayer(spec.num_experts, spec.topk, spec.hidden, spec.inter, gate_up, down, spec.tokens,
                   signs=signs, rotate=True, device=cuda_device, fuse_silu=fuse_silu)
    out = lay.forward(hidden.to(cuda_device), ids.to(cuda_device), wts.to(cuda_device))
    lay.check()
    assert lay._core.fused_silu == fuse_silu
    rep = verify.check_layer(lay)
    assert len(rep["problems"]) == 6, rep
    for p in rep["problems"]:
        assert p["acc_mismatch"] == 0 and p["out_mismatch"] == 0 and p.get("silu_mismatch", 0) == 0, p
    R = spec.tokens * spec.topk
    if fuse_silu:
        plain = MoELayer(spec.num_experts, spec.topk, spec.hidden, spec.inter, gate_up, down, spec.tokens,
                         signs=signs, rotate=True, device=cuda_device, fuse_silu=False)
        out_p = plain.forward(hidden.to(cuda_device), ids.to(cuda_device), wts.to(cuda_device))
        assert torch.equal(out.view(torch.int16), out_p.view(torch.int16))
        assert torch.equal(lay.o2.view(torch.int16), plain.o2.view(torch.int16))
        return
    g1 = lay.o1.view(-1, 2 * spec.inter)[:R].cpu()
    ref1, ref2, _, srt, order = _oracle_layer(spec, hidden, ids, signs, gu_s, dn_s, g1)
    assert og.rel_l2(g1.numpy(), ref1.numpy()) <= TOL_FAKEQUANT
    rows = lay.o2.view(-1, spec.hidden)[:R].cpu()
    assert og.rel_l2(rows.numpy(), ref2.numpy()) <= TOL_FAKEQUANT
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel())
    ref_out = (ref2.float()[inv].view(spec.tokens, spec.topk, -1) * wts[:, :, None]).sum(1)
    assert og.rel_l2(out.cpu().numpy(), ref_out.numpy()) <= TOL_FAKEQUANT


@pytest.mark.parametrize("tag", ["hot", "median", "cold"])
def test_config1_golden_slice(cuda_device, tag):
    """Vectors made by the reference's own code: rotation (fp64 matmul), quant_minmax codes and scales, exact int32
    accumulators, fake-quant product.  The quantiser kernel must reproduce codes and scales bit for bit from the
    rotated rows, the grouped GEMM the accumulators bit for bit, and the fused rotation + quantiser the codes up
    to the rounding of the fp16 butterfly."""
    z = np.load(os.path.join(G, "layer_w4a4_had.npz"))
    dev = cuda_device
    xr, qa, sa = z[f"{tag}_xr"], z[f"{tag}_qa"].astype(np.int32), z[f"{tag}_sa"]
    qb, sb, acc = z[f"{tag}_qb"].astype(np.int32), z[f"{tag}_sb"], z[f"{tag}_acc"]
    m, k = xr.shape
    n = qb.shape[0]
    ids = torch.zeros((m, 1), dtype=torch.int32, device=dev)
    # 1. quantiser on the reference-rotated rows (one expert, top-1: row order is token order)
    r = ops.quant_inp_act(torch.from_numpy(xr).to(dev), ids, 1, 64, 0, [(4, 4, -1, True)])
    inp, scl = r[0], r[1]
    got_q = op.unpack_k(inp[0].cpu().view(torch.int16).numpy().view(np.uint16).reshape(m, -1), 4)
    assert np.array_equal(got_q, qa)
    assert np.array_equal(scl[0].cpu().numpy().view(np.uint16), sa.view(np.uint16))
    # 2. grouped GEMM on the packed codes: exact accumulators, epilogue == oracle, close to the fake-quant product
    B = util.t16(op.pack_k(qb, 4), dev)
    SB = util.t16(sb, dev)
    C32 = torch.zeros((m, n), dtype=torch.int32, device=dev)
    C16 = torch.zeros((m, n), dtype=torch.float16, device=dev)
    util.run([gg.Problem(A=inp[0], B=B, C=C32, M=m, N=n, K=k, qparams=util.Q_W4A4, scale_a=scl[0], scale_b=SB,
                         out_mode=gg.OUT_ACC)])
    assert np.array_equal(C32.cpu().numpy(), acc)
    util.run([gg.Problem(A=inp[0], B=B, C=C16, M=m, N=n, K=k, qparams=util.Q_W4A4, scale_a=scl[0], scale_b=SB)])
    out = C16.cpu().numpy()
    assert np.array_equal(out.view(np.uint16), og.wxax_epilogue(acc, sa, sb).view(np.uint16))
    assert og.rel_l2(out, z[f"{tag}_fake"]) < 2e-3
    # 3. fused rotation + quantiser from the unrotated rows
    signs = torch.from_numpy(z["signs"]).to(dev)
    r = ops.quant_inp_act(torch.from_numpy(z[f"{tag}_x"]).to(dev), ids, 1, 64, 0, [(4, 4, -1, True)], rotate=True,
                          signs=signs)
    got_q = op.unpack_k(r[0][0].cpu().view(torch.int16).numpy().view(np.uint16).reshape(m, -1), 4)
    diff = np.abs(got_q - qa)
    assert diff.max() <= 1 and (diff != 0).mean() <= 0.01
