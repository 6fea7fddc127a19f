"""Host logic of the expert-parallel layer on CPU ranks (gloo, world size 2 and 3): expert ranges,
split sizes and receive-side segments from the gathered counts, and the two row exchanges."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mxmoe_b200.ep import ExchangePlan, exchange_rows, expert_ranges, strided_placement


def test_expert_ranges():
    assert expert_ranges(60, 8) == [(0, 8), (8, 16), (16, 24), (24, 32), (32, 39), (39, 46), (46, 53), (53, 60)]
    assert expert_ranges(64, 8)[-1] == (56, 64)
    assert expert_ranges(8, 8) == [(i, i + 1) for i in range(8)]
    assert expert_ranges(8, 1) == [(0, 8)]


def test_strided_placement():
    remap, inverse, ranges = strided_placement(10, 4)
    assert inverse == [0, 4, 8, 1, 5, 9, 2, 6, 3, 7]
    assert ranges == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [remap[e] for e in inverse] == list(range(10))
    for r, (lo, hi) in enumerate(ranges):
        assert all(inverse[n] % 4 == r for n in range(lo, hi))
    assert strided_placement(8, 8)[2] == [(i, i + 1) for i in range(8)]


def test_plan_from_counts():
    counts = [[3, 0, 2, 1], [1, 1, 0, 5]]           # [source][expert]
    r = expert_ranges(4, 2)
    p0 = ExchangePlan.build(counts, r, 0)
    assert p0.send_rows == [3, 3] and p0.recv_rows == [3, 2]
    assert p0.seg_m == [3, 0, 1, 1] and p0.seg_row0 == [0, 3, 3, 4] and p0.total_recv == 5
    p1 = ExchangePlan.build(counts, r, 1)
    assert p1.send_rows == [2, 5] and p1.recv_rows == [3, 5] and p1.total_recv == 8
    assert p1.seg_m == [2, 1, 0, 5]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, experts):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        rows = 40 + 7 * rank
        expert_of_row = torch.sort(torch.randint(0, experts, (rows,), generator=g)).values     # sorted = grouped by rank
        counts = torch.bincount(expert_of_row, minlength=experts).to(torch.int32)
        gathered = [torch.zeros(experts, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, counts)
        counts_all = torch.stack(gathered).tolist()
        ranges = expert_ranges(experts, world)
        plan = ExchangePlan.build(counts_all, ranges, rank)
        assert sum(plan.send_rows) == rows
        # record = (source rank, row index at the source, expert)
        send = torch.stack([torch.full((rows,), float(rank)), torch.arange(rows, dtype=torch.float32),
                            expert_of_row.float()], dim=1)
        recv = torch.full((plan.total_recv + 3, 3), -1.0)
        exchange_rows(recv, send, plan.recv_rows, plan.send_rows)
        lo, hi = ranges[rank]
        i = 0
        for s in range(world):
            for e in range(lo, hi):
                m, r0 = plan.seg_m[i], plan.seg_row0[i]
                seg = recv[r0:r0 + m]
                assert (seg[:, 0] == s).all() and (seg[:, 2] == e).all()
                assert (seg[1:, 1] > seg[:-1, 1]).all()          # source order is kept inside a segment
                i += 1
        assert (recv[plan.total_recv:] == -1).all()
        # "expert compute": scale every row by (expert + 1), then send the rows home
        out = recv[: plan.total_recv] * (recv[: plan.total_recv, 2:3] + 1)
        back = torch.zeros(rows, 3)
        exchange_rows(back, out, plan.send_rows, plan.recv_rows)
        assert torch.equal(back, send * (expert_of_row.float()[:, None] + 1))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,experts", [(2, 6), (3, 8)])
def test_row_exchange_on_cpu_ranks(world, experts):
    mp.spawn(_worker, args=(world, _free_port(), experts), nprocs=world, join=True)


def test_balanced_placement_is_a_permutation_and_balances():
    from mxmoe_b200.ep import balanced_placement
    loads = [1000 / (e + 1) ** 1.2 for e in range(60)]
    for world in (1, 2, 4, 8):
        remap, inverse, ranges = balanced_placement(loads, world)
        assert sorted(remap) == list(range(60)) and sorted(inverse) == list(range(60))
        assert all(inverse[remap[e]] == e for e in range(60))
        assert ranges[0][0] == 0 and ranges[-1][1] == 60
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert max(hi - lo for lo, hi in ranges) <= -(-60 // world)
        per_rank = [sum(loads[inverse[n]] for n in range(lo, hi)) for lo, hi in ranges]
        strided = [sum(loads[r::world]) for r in range(world)]
        assert max(per_rank) <= max(strided) + 1e-9
