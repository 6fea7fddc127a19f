"""Parity of the activation prologue, routing and combine kernels against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import hadamard as oh
from oracle import pack as op
from oracle import quant as oq
from mxmoe_b200 import ops

pytestmark = pytest.mark.gpu


def _routing(rng, t, e, k):
    ids = np.stack([rng.choice(e, k, replace=False) for _ in range(t)]).astype(np.int32)
    return torch.from_numpy(ids)


def _unpack_rows(words, tag, k):
    w = words.cpu().view(torch.int16).numpy().view(np.uint16)
    if tag == 1:
        return op.unpack_k(w, 8)
    if tag == 2:
        return op.unpack_k(w, 4)
    return w.view(np.float16)


@pytest.mark.parametrize("fused", [False, True, "scatter"])
@pytest.mark.parametrize("k", [256, 1408, 2048, 4096, 5632, 14336])
def test_quant_inp_act_matches_quantiser(cuda_device, k, fused):
    """Codes and scales are bit-identical to the fp16 min/max quantiser (quant.py:40-84) for every tag."""
    rng = np.random.default_rng(k)
    t, e, topk = 37, 6, 2
    hidden = torch.from_numpy(rng.standard_normal((t, k)).astype(np.float16))
    hidden[3] = 0            # an all-zero row: scale 0, codes 0 (the reference would divide by zero)
    ids = _routing(rng, t, e, topk)
    qp = [(4, 4, -1, True), (8, 8, -1, True), (16, 16, -1, True), (16, 4, 128, False), (4, 4, -1, True),
          (8, 8, -1, True), (4, 4, -1, True)]          # last entry: shared expert
    out = ops.quant_inp_act(hidden.to(cuda_device), ids.to(cuda_device), e, 64, 1, qp, fused=fused)
    inp_list, scale_list, out_list, _, _, _, recv, perm, dst = out
    assert recv.device.type == "cpu" and recv.dtype == torch.int64
    srt, order = torch.sort(ids.reshape(-1), stable=True)
    assert torch.equal(dst.cpu(), srt) and torch.equal(perm.cpu(), order // topk)
    assert torch.equal(recv, torch.bincount(srt, minlength=e))
    tokens = recv.tolist() + [t]
    src_rows = torch.cat([order // topk, torch.arange(t)])
    pidx, row = 0, 0
    for ex in range(e + 1):
        m = tokens[ex]
        if m == 0:
            continue
        x = hidden[src_rows[row:row + m]]
        a_bits = qp[ex][0]
        tag = 0 if a_bits >= 16 else (1 if a_bits == 8 else 2)
        got = _unpack_rows(inp_list[pidx], tag, k)
        if tag == 0:
            assert np.array_equal(got.view(np.uint16), x.numpy().view(np.uint16))
            assert scale_list[pidx].numel() == 0 or True
        else:
            codes, scale, _ = oq.minmax_quantize(x, a_bits, -1, True)
            zero_rows = (x.abs().amax(dim=-1) == 0)
            codes[zero_rows] = 0
            assert np.array_equal(got, codes.numpy().astype(np.int32)), f"expert {ex}"
            s = scale_list[pidx].cpu().numpy()
            assert np.array_equal(s.view(np.uint16), scale.reshape(-1).numpy().view(np.uint16))
        assert out_list[pidx].shape == (m, 64 * 2 * (1 if ex == e else 1))
        pidx += 1
        row += m
    assert pidx == len(inp_list)


@pytest.mark.parametrize("fused", [False, True, "scatter"])
@pytest.mark.parametrize("k", [256, 2048, 4096])
def test_quant_inp_act_with_rotation(cuda_device, k, fused):
    """Rotated rows match matmul_hadU on (x * signs) to rel-L2 1e-3 after dequantisation of 8-bit codes;
    4-bit codes differ from the oracle's in at most 1 % of positions and never by more than one step."""
    rng = np.random.default_rng(k + 1)
    t, e, topk = 33, 4, 2
    hidden = torch.from_numpy(rng.standard_normal((t, k)).astype(np.float16))
    signs = torch.from_numpy(rng.choice([-1, 1], k).astype(np.int8))
    ids = _routing(rng, t, e, topk)
    qp = [(16, 16, -1, True), (8, 8, -1, True), (4, 4, -1, True), (4, 4, -1, True)]
    out = ops.quant_inp_act(hidden.to(cuda_device), ids.to(cuda_device), e, 64, 0, qp, rotate=True,
                            signs=signs.to(cuda_device), fused=fused)
    inp_list, scale_list, _, _, _, _, recv, perm, _ = out
    rot = oh.hadamard_rows(hidden.double() * signs.double())
    pidx, row = 0, 0
    for ex, m in enumerate(recv.tolist()):
        if m == 0:
            continue
        ref = rot[perm.cpu()[row:row + m]]
        a_bits = qp[ex][0]
        tag = 0 if a_bits >= 16 else (1 if a_bits == 8 else 2)
        got = _unpack_rows(inp_list[pidx], tag, k)
        if tag == 0:
            err = np.linalg.norm(got.astype(np.float64) - ref.numpy()) / np.linalg.norm(ref.numpy())
            assert err <= 1e-3, err
        else:
            codes, scale, _ = oq.minmax_quantize(ref.half(), a_bits, -1, True)
            diff = np.abs(got - codes.numpy().astype(np.int32))
            assert diff.max() <= 1
            assert (diff != 0).mean() <= 0.01
            s = scale_list[pidx].cpu().numpy().astype(np.float64)
            assert np.allclose(s, scale.reshape(-1).double().numpy(), rtol=2e-3)
        pidx += 1
        row += m


@pytest.mark.parametrize("n,ns", [(64, 0), (1408, 0), (1408, 2), (5632, 1), (14336, 0)])
def test_silu_mul_then_quant(cuda_device, n, ns):
    rng = np.random.default_rng(n + ns)
    t, e, topk, hid = 19, 5, 2, 256
    ids = _routing(rng, t, e, topk)
    srt, order = torch.sort(ids.reshape(-1), stable=True)
    recv = torch.bincount(srt, minlength=e)
    rows = t * topk
    gate_up = torch.from_numpy((rng.standard_normal((rows, 2 * n)) * 2).astype(np.float16))
    shared = torch.from_numpy((rng.standard_normal((t, 2 * n * max(ns, 1))) * 2).astype(np.float16))
    flat = torch.cat([gate_up.reshape(-1), shared.reshape(-1)]) if ns else gate_up.reshape(-1)
    qp = [(4, 4, -1, True), (8, 8, -1, True), (16, 16, -1, True), (8, 8, -1, True), (4, 4, -1, True), (8, 8, -1, True)]
    out = ops.silu_mul_then_quant(flat.to(cuda_device), int((recv != 0).sum()), e, hid, n, ns, t, topk,
                                  srt.to(cuda_device), recv, qp)
    inp_list, scale_list, out_list, _, _, out_store = out
    assert out_store.numel() == (1 + topk) * t * hid
    tokens = recv.tolist() + ([t] if ns else [])
    pidx, row = 0, 0
    for ex, m in enumerate(tokens):
        if m == 0:
            continue
        if ex == e:
            src, width = shared, n * ns
        else:
            src, width = gate_up[row:row + m], n
        g, u = src[:, :width].float(), src[:, width:2 * width]
        h = (torch.nn.functional.silu(g).half() * u)          # fp16 module semantics: silu -> fp16, product -> fp16
        a_bits = qp[ex][0]
        tag = 0 if a_bits >= 16 else (1 if a_bits == 8 else 2)
        got = _unpack_rows(inp_list[pidx], tag, width)
        if tag == 0:
            d = np.abs(got.astype(np.float32) - h.numpy().astype(np.float32))
            assert (d > 0).mean() < 0.02          # expf differs from the CPU library in the last ulp now and then
            assert np.linalg.norm(d) / np.linalg.norm(h.numpy().astype(np.float32)) < 1e-3
        else:
            codes, scale, _ = oq.minmax_quantize(h, a_bits, -1, True)
            diff = np.abs(got - codes.numpy().astype(np.int32))
            assert diff.max() <= 1 and (diff != 0).mean() <= 0.02
        assert out_list[pidx].shape == (m, hid)
        pidx += 1
        if ex < e:
            row += m


# decode batch (one block does everything), layer sizes, many experts, many pairs
@pytest.mark.parametrize("t,e,k", [(1, 8, 2), (37, 60, 4), (1000, 64, 6), (8192, 60, 4), (300, 8, 2), (600, 256, 2),
                                   (700, 300, 3), (70000, 16, 4), (513, 2, 2)])
def test_device_routing_matches_stable_sort(cuda_device, t, e, k):
    from mxmoe_b200.layer import MoELayer
    rng = np.random.default_rng(t)
    ids = _routing(rng, t, e, k)
    lay = MoELayer.__new__(MoELayer)
    # only the routing state of a layer is needed here
    dev = cuda_device
    lay.E, lay.R = e, t * k
    lay.counts = torch.zeros(e, dtype=torch.int32, device=dev)
    lay.row_start = torch.zeros(e + 1, dtype=torch.int32, device=dev)
    lay.row_expert = torch.zeros(t * k, dtype=torch.int32, device=dev)
    lay.row_token = torch.zeros(t * k, dtype=torch.int64, device=dev)
    lay.slot_row = torch.zeros(t * k, dtype=torch.int32, device=dev)
    from mxmoe_b200 import _lib
    lay.route_ws = torch.zeros(_lib.lib().mxmoe_route_workspace_bytes(t * k, 1, e) // 4 + 1, dtype=torch.int32,
                               device=dev)
    lay.route(ids.to(dev))
    torch.cuda.synchronize()
    srt, order = torch.sort(ids.reshape(-1), stable=True)
    cnt = torch.bincount(srt, minlength=e)
    assert torch.equal(lay.counts.cpu().long(), cnt)
    assert torch.equal(lay.row_start.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), cnt.cumsum(0)]))
    assert torch.equal(lay.row_expert.cpu(), srt)
    assert torch.equal(lay.row_token.cpu(), order // k)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel())
    assert torch.equal(lay.slot_row.cpu().long(), inv)


@pytest.mark.parametrize("replicated", [False, True])
def test_device_routing_renumbers_ids_as_it_reads_them(cuda_device, replicated):
    """The optional map of the routing arguments: original expert -> (a copy chosen by token index ->) new id.  The
    result must be the stable sort of the ids a host-side renumbering gives."""
    from mxmoe_b200 import _lib
    from mxmoe_b200.layer import MoELayer
    rng = np.random.default_rng(11)
    t, e0, k = 777, 12, 3
    dev = cuda_device
    ids = _routing(rng, t, e0, k)
    reps = rng.integers(1, 4, e0) if replicated else np.ones(e0, dtype=np.int64)
    base = np.concatenate([[0], np.cumsum(reps)[:-1]])
    e = int(reps.sum())
    perm = rng.permutation(e)
    tok = torch.arange(t).repeat_interleave(k)
    flat = ids.reshape(-1).long()
    virt = torch.from_numpy(base)[flat] + tok % torch.from_numpy(reps)[flat]
    new = torch.from_numpy(perm)[virt]
    lay = MoELayer.__new__(MoELayer)
    lay.E, lay.R = e, t * k
    i32 = dict(dtype=torch.int32, device=dev)
    lay.counts, lay.row_start = torch.zeros(e, **i32), torch.zeros(e + 1, **i32)
    lay.row_expert, lay.slot_row = torch.zeros(t * k, **i32), torch.zeros(t * k, **i32)
    lay.row_token = torch.zeros(t * k, dtype=torch.int64, device=dev)
    lay.route_ws = torch.zeros(_lib.lib().mxmoe_route_workspace_bytes(t * k, 1, e) // 4 + 1, **i32)
    lay.id_map, lay.num_ids = torch.from_numpy(perm.astype(np.int32)).to(dev), e0
    lay.rep_base = torch.from_numpy(base.astype(np.int32)).to(dev) if replicated else None
    lay.rep_count = torch.from_numpy(reps.astype(np.int32)).to(dev) if replicated else None
    lay.route(ids.to(dev))
    torch.cuda.synchronize()
    srt, order = torch.sort(new, stable=True)
    assert torch.equal(lay.counts.cpu().long(), torch.bincount(srt, minlength=e))
    assert torch.equal(lay.row_expert.cpu().long(), srt)
    assert torch.equal(lay.row_token.cpu(), order // k)


def test_combine(cuda_device):
    from mxmoe_b200 import _lib
    from mxmoe_b200.gg import current_stream_ptr
    rng = np.random.default_rng(9)
    t, k, h = 50, 4, 512
    y = torch.from_numpy(rng.standard_normal((t * k, h)).astype(np.float16)).to(cuda_device)
    ysh = torch.from_numpy(rng.standard_normal((t, h)).astype(np.float16)).to(cuda_device)
    slot = torch.from_numpy(rng.permutation(t * k).astype(np.int32)).to(cuda_device)
    w = torch.from_numpy(rng.uniform(0, 1, (t, k)).astype(np.float32)).to(cuda_device)
    out = torch.empty((t, h), dtype=torch.float16, device=cuda_device)
    _lib.check(_lib.lib().mxmoe_combine_topk(y.data_ptr(), slot.data_ptr(), w.data_ptr(), ysh.data_ptr(),
                                             out.data_ptr(), t, k, h, current_stream_ptr()))
    ref = (y.float()[slot.long()].view(t, k, h) * w[:, :, None]).sum(1) + ysh.float()
    assert torch.allclose(out.float(), ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("world,rank", [(1, 0), (3, 1), (4, 3)])
def test_device_exchange_plan_matches_host_plan(cuda_device, world, rank):
    """mxmoe_ep_plan on one GPU with made-up counts of `world` ranks against the numpy plan of the NCCL transport."""
    import ctypes as C
    from mxmoe_b200 import _lib
    from mxmoe_b200.ep import ExchangePlan, expert_ranges
    from mxmoe_b200.gg import current_stream_ptr
    rng = np.random.default_rng(7 + world)
    E = 13
    counts = rng.integers(0, 40, (world, E)).astype(np.int32)
    counts[:, 2] = 0
    ranges = expert_ranges(E, world)
    lo, hi = ranges[rank]
    el = hi - lo
    plan = ExchangePlan.build(counts, ranges, rank)
    i32 = dict(dtype=torch.int32, device=cuda_device)
    cap = plan.total_recv + 5
    t = {
        "counts_all": torch.tensor(counts.reshape(-1), **i32), "range_lo": torch.tensor([r[0] for r in ranges] + [E], **i32),
        "seg_m": torch.zeros(world * el, **i32), "seg_row0": torch.zeros(world * el, **i32),
        "seg_src_row0": torch.zeros(world * el, **i32), "recv_row_expert": torch.full((cap,), -1, **i32),
        "total_recv": torch.zeros(2, **i32), "dst_row0": torch.zeros(E, **i32), "exp_owner": torch.zeros(E, **i32),
    }
    a = _lib.EpPlanArgs()
    for name, ten in t.items():
        setattr(a, name, ten.data_ptr())
    a.world, a.rank, a.num_experts, a.experts_local, a.recv_capacity = world, rank, E, el, cap
    _lib.check(_lib.lib().mxmoe_ep_plan(C.byref(a), current_stream_ptr()))
    torch.cuda.synchronize()
    assert t["seg_m"].tolist() == plan.seg_m and t["seg_row0"].tolist() == plan.seg_row0
    assert t["total_recv"].tolist() == [plan.total_recv, 0]
    # first row of each segment in the source's expert-sorted order
    want_src = [int(counts[s, :lo + j].sum()) for s in range(world) for j in range(el)]
    assert t["seg_src_row0"].tolist() == want_src
    owner = [next(r for r, (a0, b0) in enumerate(ranges) if a0 <= e < b0) for e in range(E)]
    assert t["exp_owner"].tolist() == owner
    # where my rows for expert e start at their owner: behind lower ranks' rows for the owner's experts and my
    # rows for the owner's earlier experts
    want_dst = []
    for e in range(E):
        dlo, dhi = ranges[owner[e]]
        want_dst.append(int(counts[:rank, dlo:dhi].sum() + counts[rank, dlo:e].sum()))
    assert t["dst_row0"].tolist() == want_dst
    rexp = t["recv_row_expert"].cpu().numpy()
    want_rexp = np.concatenate([np.full(m, lo + (i % el)) for i, m in enumerate(plan.seg_m)] + [np.full(5, -1)])
    assert np.array_equal(rexp, want_rexp)
    # a store that is too small: segments are clipped and the overflow word reports the rows wanted
    a.recv_capacity = max(plan.total_recv - 7, 0)
    _lib.check(_lib.lib().mxmoe_ep_plan(C.byref(a), current_stream_ptr()))
    torch.cuda.synchronize()
    if plan.total_recv > 7:
        assert t["total_recv"].tolist() == [plan.total_recv - 7, plan.total_recv]
        ends = (t["seg_row0"] + t["seg_m"]).max().item()
        assert ends <= plan.total_recv - 7


@pytest.mark.parametrize("t,e,k,dtype,renorm", [(70, 60, 4, torch.float32, True), (33, 64, 6, torch.float16, False),
                                                 (5, 8, 2, torch.float32, True), (129, 300, 8, torch.float32, True)])
def test_gate_topk_matches_torch(cuda_device, t, e, k, dtype, renorm):
    from mxmoe_b200 import ops
    g = torch.Generator().manual_seed(e * 7 + k)
    logits = (torch.randn(t, e, generator=g) * 2).to(dtype)
    if dtype == torch.float16:   # distinct, exactly representable values: no ties to break
        logits = torch.stack([torch.randperm(e, generator=g) for _ in range(t)]).to(torch.float16) / 8 - 4
    ids, wts = ops.gate_topk(logits.to(cuda_device), k, renormalize=renorm)
    prob = torch.softmax(logits.float(), dim=-1)
    want_w, want_i = prob.topk(k, dim=-1)
    if renorm:
        want_w = want_w / want_w.sum(dim=-1, keepdim=True)
    assert torch.equal(ids.cpu().long(), want_i), "expert ids differ from torch.topk"
    assert torch.allclose(wts.cpu(), want_w, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("world,rank", [(1, 0), (3, 1), (4, 3)])
def test_device_exchange_plan_expert_major(cuda_device, world, rank):
    """Layout 1 of mxmoe_ep_plan: the receive store is ordered (expert, source rank).  Segment tables, the per-expert
    tables, the senders' first rows, the expert of every received row and the address of every row's result against
    plain numpy on made-up counts."""
    import ctypes as C
    from mxmoe_b200 import _lib
    from mxmoe_b200.ep import expert_ranges
    from mxmoe_b200.gg import current_stream_ptr
    rng = np.random.default_rng(17 + world)
    E, row_bytes = 13, 64
    counts = rng.integers(0, 40, (world, E)).astype(np.int64)
    counts[:, 2] = 0
    ranges = expert_ranges(E, world)
    lo, hi = ranges[rank]
    el = hi - lo
    total = int(counts[:, lo:hi].sum())
    cap = total + 5
    i32 = dict(dtype=torch.int32, device=cuda_device)
    bases = [1 << 40 | (s << 30) for s in range(world)]              # made-up buffer addresses, never dereferenced
    t = {
        "counts_all": torch.tensor(counts.reshape(-1), **i32), "range_lo": torch.tensor([r[0] for r in ranges] + [E], **i32),
        "seg_m": torch.zeros(max(world * el, 1), **i32), "seg_row0": torch.zeros(max(world * el, 1), **i32),
        "seg_src_row0": torch.zeros(max(world * el, 1), **i32), "recv_row_expert": torch.full((cap,), -1, **i32),
        "total_recv": torch.zeros(2, **i32), "dst_row0": torch.zeros(E, **i32), "exp_owner": torch.zeros(E, **i32),
        "exp_m": torch.zeros(max(el, 1), **i32), "exp_row0": torch.zeros(max(el, 1), **i32),
        "row_dst": torch.zeros(cap, dtype=torch.int64, device=cuda_device),
        "peer_ret": torch.tensor(bases, dtype=torch.int64, device=cuda_device),
    }
    a = _lib.EpPlanArgs()
    for name, ten in t.items():
        setattr(a, name, ten.data_ptr())
    a.world, a.rank, a.num_experts, a.experts_local, a.recv_capacity = world, rank, E, el, cap
    a.layout, a.ret_row_bytes = 1, row_bytes
    _lib.check(_lib.lib().mxmoe_ep_plan(C.byref(a), current_stream_ptr()))
    torch.cuda.synchronize()
    exp_m = [int(counts[:, lo + j].sum()) for j in range(el)]
    exp_row0 = [int(counts[:, lo:lo + j].sum()) for j in range(el)]
    assert t["exp_m"].tolist()[:el] == exp_m and t["exp_row0"].tolist()[:el] == exp_row0
    seg_row0 = [exp_row0[j] + int(counts[:s, lo + j].sum()) for s in range(world) for j in range(el)]
    seg_m = [int(counts[s, lo + j]) for s in range(world) for j in range(el)]
    assert t["seg_row0"].tolist()[:world * el] == seg_row0 and t["seg_m"].tolist()[:world * el] == seg_m
    assert t["total_recv"].tolist() == [total, 0]
    owner = [next(r for r, (a0, b0) in enumerate(ranges) if a0 <= e < b0) for e in range(E)]
    want_dst = []
    for e in range(E):
        dlo, _ = ranges[owner[e]]
        want_dst.append(int(counts[:, dlo:e].sum() + counts[:rank, e].sum()))
    assert t["dst_row0"].tolist() == want_dst
    want_exp = np.full(cap, -1)
    want_ptr = np.zeros(cap, dtype=np.int64)
    for s in range(world):
        for j in range(el):
            r0, m = seg_row0[s * el + j], seg_m[s * el + j]
            want_exp[r0:r0 + m] = lo + j
            src0 = int(counts[s, :lo + j].sum())
            want_ptr[r0:r0 + m] = bases[s] + (src0 + np.arange(m)) * row_bytes
    assert np.array_equal(t["recv_row_expert"].cpu().numpy(), want_exp)
    assert np.array_equal(t["row_dst"].cpu().numpy()[:total], want_ptr[:total])


def test_fetch_host_reads_page_locked_memory_with_a_kernel(cuda_device):
    """mxmoe_fetch_host: page-locked source (kernel path), pageable source and odd sizes (copy-engine path)."""
    from mxmoe_b200 import _lib
    from mxmoe_b200.gg import current_stream_ptr
    lib = _lib.lib()
    rng = np.random.default_rng(3)
    for n, pinned in ((8192 * 4, True), (1000, True), (8192 * 4, False), (37, True)):
        src = torch.from_numpy(rng.integers(-2**31, 2**31 - 1, n, dtype=np.int64).astype(np.int32))
        if pinned:
            src = src.pin_memory()
        dst = torch.zeros(n, dtype=torch.int32, device=cuda_device)
        _lib.check(lib.mxmoe_fetch_host(dst.data_ptr(), src.data_ptr(), n * 4, current_stream_ptr()))
        torch.cuda.synchronize()
        assert torch.equal(dst.cpu(), src)
