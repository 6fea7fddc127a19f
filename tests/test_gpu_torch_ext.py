"""The torch C++ extension ``mxmoe_ops`` (the reference's operator names, ref_bind.cu:759-768, compiled over the C ABI)
gives the same bits as the Python operator API on one mixed-precision layer pass."""
import pytest
import torch

from mxmoe_b200 import ops, workload

pytestmark = pytest.mark.gpu


def test_extension_matches_python_operator_api(cuda_device):
    mxmoe_ops = pytest.importorskip("mxmoe_b200.mxmoe_ops")
    spec = workload.LayerSpec("tiny", 6, 2, 512, 256, 512, 70, "zipf", 1.2, True, False, "mixed5")
    hidden = workload.make_hidden(spec).to(cuda_device)
    ids, _ = workload.make_routing(spec)
    ids = ids.to(cuda_device)
    gate_up, down, _, _ = workload.build_layer_weights(spec, device=cuda_device)
    n_all = spec.num_experts + 1
    qp1 = [gate_up[e].qparams for e in range(n_all)]
    qp2 = [down[e].qparams for e in range(n_all)]

    def empty():
        return torch.empty(0, device=cuda_device, dtype=torch.float16)

    def run(api):
        r = api.quant_inp_act(hidden, ids, spec.num_experts, spec.inter, 1, qp1)
        inp, sc, outl, _, _, out_store, recv, perm, dst = r
        outl[-1] = torch.empty((spec.tokens, 2 * spec.shared_inter), dtype=torch.float16, device=cuda_device)
        api.gg_mxmoe_share_fused(inp, [gate_up[e].data for e in range(n_all)], sc,
                                 [gate_up[e].scale if gate_up[e].scale is not None else empty() for e in range(n_all)],
                                 outl, 2 * spec.inter, spec.hidden, 2 * spec.shared_inter, spec.hidden, qp1, recv)
        return inp, sc, outl, recv, dst
    a = run(ops)
    b = run(mxmoe_ops)
    assert torch.equal(a[3], b[3]) and torch.equal(a[4], b[4])
    for x, y in zip(a[0] + a[1] + a[2], b[0] + b[1] + b[2]):
        assert x.shape == y.shape and torch.equal(x.view(torch.int16), y.view(torch.int16))

    # silu_mul_then_quant + down, routed experts only (the shared rows of this tiny layer are not 2N wide)
    spec2 = workload.LayerSpec("tiny2", 6, 2, 512, 256, 0, 70, "zipf", 1.2, True, False, "mixed5")
    gate_up, down, _, _ = workload.build_layer_weights(spec2, device=cuda_device)
    qp1 = [gate_up[e].qparams for e in range(6)]
    qp2 = [down[e].qparams for e in range(6)]

    def run2(api):
        inp, sc, outl, _, _, out_store, recv, perm, dst = api.quant_inp_act(hidden, ids, 6, spec2.inter, 0, qp1)
        api.gg_mxmoe_share_fused(inp, [gate_up[e].data for e in range(6)], sc,
                                 [gate_up[e].scale if gate_up[e].scale is not None else empty() for e in range(6)],
                                 outl, 2 * spec2.inter, spec2.hidden, 0, 0, qp1, recv)
        r2 = api.silu_mul_then_quant(out_store, len(inp), 6, spec2.hidden, spec2.inter, 0, spec2.tokens, spec2.topk, dst,
                                     recv, qp2)
        inp2, sc2, outl2 = r2[:3]
        api.gg_mxmoe_share_fused(inp2, [down[e].data for e in range(6)], sc2,
                                 [down[e].scale if down[e].scale is not None else empty() for e in range(6)],
                                 outl2, spec2.hidden, spec2.inter, 0, 0, qp2, recv)
        return inp2 + sc2 + outl2
    for x, y in zip(run2(ops), run2(mxmoe_ops)):
        assert torch.equal(x.view(torch.int16), y.view(torch.int16))

    # fp16 baselines
    experts = (torch.randn(4, 256, 128, device=cuda_device) * 0.05).half()
    x = torch.randn(33, 128, device=cuda_device).half()
    tid = torch.randint(0, 4, (33, 2), device=cuda_device, dtype=torch.int32)
    o1 = ops.gg_cutlass(x, experts, tid, torch.zeros(66, 256, device=cuda_device, dtype=torch.float16))
    o2 = mxmoe_ops.gg_cutlass(x, experts, tid, torch.zeros(66, 256, device=cuda_device, dtype=torch.float16))
    assert torch.equal(o1, o2)
