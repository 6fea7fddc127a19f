"""Worker of the multi-GPU expert-parallel test (launched by tests/test_gpu_ep.py under torchrun, or
in-process with world size 1): the expert-parallel layer must return, for this rank's tokens,
exactly the bits a single-GPU layer holding ALL experts returns for the same tokens."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def run(spec_name: str = "tiny-ep") -> None:
    from mxmoe_b200 import workload
    from mxmoe_b200.ep import EPMoELayer
    from mxmoe_b200.layer import MoELayer
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    specs = {
        "tiny-ep": workload.LayerSpec("tiny-ep", 6, 2, 512, 256, 512, 96, "zipf", 1.2, True, True, "mixed5"),
        "tiny-ep-w4a4": workload.LayerSpec("tiny-ep-w4a4", 8, 2, 512, 256, 0, 200, "zipf", 1.0, False, True,
                                           "w4a4_g-1_sym"),
        "tiny-ep-w8w4": workload.LayerSpec("tiny-ep-w8w4", 8, 2, 512, 256, 0, 160, "softmax_biased", 0.0, True, True,
                                           "mixed_w8w4"),
    }
    spec = specs[spec_name]
    hidden = workload.make_hidden(spec, seed=1 + rank).to(dev)
    ids, wts = workload.make_routing(spec, seed=2 + rank)
    ids, wts = ids.to(dev), wts.to(dev)
    outs = {}
    for transport, fmt in (("p2p", "expanded"), ("p2p", "packed"), ("nccl", "packed")):
        ep = EPMoELayer(spec, dev, capacity_factor=float(world) + 1.0, transport=transport, dispatch_format=fmt)
        out_ep = ep.forward(hidden, ids, wts).clone()
        out_ep2 = ep.forward(hidden, ids, wts).clone()          # a second step reuses every buffer
        ep.check()
        outs[transport + "/" + fmt] = (out_ep, out_ep2)
        if transport == "nccl":
            assert sum(ep.last_plan.send_rows) == spec.tokens * spec.topk
        else:
            got = ep.total_recv[:1].clone().float()
            dist.all_reduce(got)
            assert int(got.item()) == world * spec.tokens * spec.topk, "rows received over all ranks"
    gate_up, down, signs, _ = workload.build_layer_weights(spec, device=dev)
    full = MoELayer(spec.num_experts, spec.topk, spec.hidden, spec.inter, gate_up, down, spec.tokens,
                    shared_inter=spec.shared_inter, signs=signs, rotate=spec.rotate, device=dev)
    out_full = full.forward(hidden, ids, wts)
    full.check()
    torch.cuda.synchronize()
    assert torch.isfinite(out_full.float()).all()
    for transport, (out_ep, out_ep2) in outs.items():
        assert torch.equal(out_ep, out_full), f"rank {rank} ({transport}): expert-parallel output differs from the single-GPU layer"
        assert torch.equal(out_ep2, out_full), f"rank {rank} ({transport}): second step differs"


if __name__ == "__main__":
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        for name in sys.argv[1:] or ["tiny-ep"]:
            run(name)
        print(f"rank {dist.get_rank()} ok", flush=True)
    finally:
        dist.destroy_process_group()
