"""Online Hadamard rotation for row lengths n = K * m (the rotation of the down-projection input): kernel against the
oracle's restatement of the reference's matmul_hadU (pinned to the reference by tests/golden/hadamard_kron.npz, which
also holds the reference's own K x K factors), and a layer that uses it."""
import os

import numpy as np
import pytest
import torch

from oracle import gemm as og
from oracle import hadamard as oh
from oracle import quant as oq
from mxmoe_b200 import hadamard, workload
from mxmoe_b200.layer import MoELayer

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("n,rows", [(1408, 3), (1408, 77), (14336, 3), (14336, 19)])
def test_kron_rotation_matches_reference_transform(cuda_device, n, rows):
    z = np.load(os.path.join(G, "hadamard_kron.npz"))
    had = torch.from_numpy(z[f"had{n}"].astype(np.float64))
    if rows == 3:
        x = torch.from_numpy(z[f"x{n}"]).half()
    else:
        x = torch.randn(rows, n, generator=torch.Generator().manual_seed(n + rows)).half()
    want = oh.hadamard_kron_rows(x.double(), had)
    if rows == 3:      # the fp16-rounded inputs change the golden outputs by fp16 rounding only
        assert og.rel_l2(want.numpy(), z[f"y{n}"]) < 1e-3
    xd = x.to(cuda_device)
    hk = had.to(cuda_device).half()
    got = hadamard.hadamard_kron(xd, hk)
    err = og.rel_l2(got.cpu().numpy(), want.numpy())
    assert err <= 1e-3, err
    # in place, and with the factor built here instead of the reference's: still an orthogonal rotation
    own, k, m = hadamard.hadamard_factor(n)
    y2 = hadamard.hadamard_kron(xd.clone(), own.to(cuda_device).half())
    assert abs(float(y2.float().norm() / xd.float().norm()) - 1.0) < 2e-3
    x_in = xd.clone()
    hadamard.hadamard_kron(x_in, hk, out=x_in)
    assert torch.equal(x_in, got)


def test_layer_with_online_rotation_of_the_down_input(cuda_device):
    """Routed experts with the online rotation: down rows equal the fake-quant loop on rotated h and rotated W_down."""
    spec = workload.LayerSpec("tiny-had", 4, 2, 512, 1408, 0, 64, "zipf", 1.2, True, True, "w4a4_g-1_sym")
    had, k, m = hadamard.hadamard_factor(spec.inter)
    assert (k, m) == (176, 8)
    hidden = workload.make_hidden(spec)
    ids, wts = workload.make_routing(spec)
    gate_up, down, signs, (gu_s, dn_s) = workload.build_layer_weights(spec, device=cuda_device, online_had=had)
    lay = MoELayer(spec.num_experts, spec.topk, spec.hidden, spec.inter, gate_up, down, spec.tokens, signs=signs,
                   rotate=True, device=cuda_device, online_had=had, fuse_silu=False)
    lay.forward(hidden.to(cuda_device), ids.to(cuda_device), wts.to(cuda_device))
    lay.check()
    # the same layer with silu(gate) * up in the first GEMM's epilogue: the rows that are rotated are the same bits
    lay_f = MoELayer(spec.num_experts, spec.topk, spec.hidden, spec.inter, gate_up, down, spec.tokens, signs=signs,
                     rotate=True, device=cuda_device, online_had=had, fuse_silu=True)
    lay_f.forward(hidden.to(cuda_device), ids.to(cuda_device), wts.to(cuda_device))
    lay_f.check()
    assert lay_f._core.fused_silu and torch.equal(lay_f.o2.view(torch.int16), lay.o2.view(torch.int16))
    R = spec.tokens * spec.topk
    g1 = lay.o1.view(-1, 2 * spec.inter)[:R].cpu()
    rows = lay.o2.view(-1, spec.hidden)[:R].cpu()
    srt, _ = torch.sort(ids.reshape(-1).long(), stable=True)
    cnt = torch.bincount(srt, minlength=spec.num_experts).tolist()
    r0, ref = 0, []
    for e, mrows in enumerate(cnt):
        if mrows:
            _, wdn = workload.expert_weights_fp16(spec, e)
            y1 = g1[r0:r0 + mrows]
            h = torch.nn.functional.silu(y1[:, :spec.inter].float()).half() * y1[:, spec.inter:]
            h_rot = oh.hadamard_kron_rows(h.double(), had.double()).half()
            w_rot = oh.hadamard_kron_rows(wdn.double(), had.double()).half()
            ref.append(oq.fake_quant_expert_loop([h_rot], [w_rot], [dn_s[e]])[0])
        r0 += mrows
    err = og.rel_l2(rows.numpy(), torch.cat(ref).numpy())
    assert err <= 2e-2, err
