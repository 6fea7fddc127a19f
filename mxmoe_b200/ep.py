"""Expert-parallel MoE layer: one process per GPU, experts sharded in contiguous ranges,
tokens data-parallel, quantised rows dispatched with an all-to-all over NCCL / NVLink and fp16
rows combined back.  (The reference has no distributed code; this is the multi-GPU form of the
path described by the benchmark configurations.)

Per step and rank::

    route_topk (global expert ids)  ->  rows sorted by expert = grouped by destination rank
    quant_tokens + gather_rows      ->  send records [T*topk, P + 8] (packed row + its scale)
    all_gather(counts)              ->  one small device->host copy: every split size of the step
    all_to_all_single(records)      ->  receive store in local HBM, grouped (source rank, expert)
    ExpertCompute                   ->  one problem per (source rank, local expert), no re-sort
    all_to_all_single(fp16 rows)    ->  back to the owners, in their original row order
    combine_topk (+ shared expert, computed locally on the rank's own tokens)

TMA only ever reads this GPU's own memory (the receive store); no load uses cluster multicast.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from . import _lib
from .gg import current_stream_ptr
from .layer import ExpertCompute, MoELayer, TokenQuant, record_stride, tag_of


def expert_ranges(num_experts: int, world: int) -> list[tuple[int, int]]:
    """Contiguous expert range [lo, hi) of every rank; the first ``E % world`` ranks own one more."""
    base, extra = divmod(num_experts, world)
    out, lo = [], 0
    for r in range(world):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def strided_placement(num_experts: int, world: int):
    """Expert e lives on rank ``e % world`` (spreads the hot head of a skewed routing distribution
    over the ranks).  Returns ``(remap, inverse, ranges)``: experts are renumbered rank-major so that
    every rank owns a contiguous range of the NEW ids and rows sorted by new id are grouped by
    destination rank; ``remap[e]`` is the new id of expert e, ``inverse`` the opposite map."""
    inverse = [e for r in range(world) for e in range(r, num_experts, world)]
    remap = [0] * num_experts
    for new, e in enumerate(inverse):
        remap[e] = new
    ranges, lo = [], 0
    for r in range(world):
        n = len(range(r, num_experts, world))
        ranges.append((lo, lo + n))
        lo += n
    return remap, inverse, ranges


@dataclasses.dataclass
class ExchangePlan:
    """Split sizes (in rows) and receive-side segments of one step, from the gathered counts."""
    send_rows: list[int]          # rows this rank sends to every rank
    recv_rows: list[int]          # rows this rank receives from every rank
    seg_m: list[int]              # rows of segment (source s, local expert j), s-major
    seg_row0: list[int]           # first row of each segment in the receive store
    total_recv: int

    @staticmethod
    def build(counts_all, ranges: list[tuple[int, int]], rank: int) -> "ExchangePlan":
        """``counts_all[s][e]``: rows rank s routes to expert e (nested lists or an int array)."""
        import numpy as np
        c = np.asarray(counts_all, dtype=np.int64)
        lo, hi = ranges[rank]
        csum = np.concatenate(([0], np.cumsum(c[rank])))
        send = [int(csum[b] - csum[a]) for a, b in ranges]
        mine = c[:, lo:hi]
        recv = mine.sum(axis=1).tolist()
        seg_m = mine.reshape(-1)
        seg_row0 = np.cumsum(seg_m) - seg_m
        return ExchangePlan(send, recv, seg_m.tolist(), seg_row0.tolist(), int(seg_m.sum()))


def exchange_rows(out2d: torch.Tensor, inp2d: torch.Tensor, out_rows: list[int], in_rows: list[int], group=None):
    """Variable-size all-to-all of whole rows (first dimension)."""
    dist.all_to_all_single(out2d[: sum(out_rows)], inp2d[: sum(in_rows)], out_rows, in_rows, group=group)


class EPMoELayer:
    """Expert-parallel layer for ``spec`` (a :class:`mxmoe_b200.workload.LayerSpec`): ``spec.tokens`` tokens per rank."""

    def __init__(self, spec, device, gen_device="cpu", capacity_factor: float = 3.0, group=None,
                 placement: str = "strided"):
        from . import workload
        self.spec, self.device, self.group = spec, torch.device(device), group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        E, T, k, H, I = spec.num_experts, spec.tokens, spec.topk, spec.hidden, spec.inter
        if placement == "strided":
            remap, inverse, self.ranges = strided_placement(E, self.world)
        else:
            remap, inverse, self.ranges = list(range(E)), list(range(E)), expert_ranges(E, self.world)
        lo, hi = self.ranges[self.rank]
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        f16 = dict(dtype=torch.float16, device=dev)
        self.remap = torch.tensor(remap, **i32)

        # weights of the local experts, keyed by their NEW ids (the shared expert keeps key E)
        gu_o, dn_o, signs, (gu_s, dn_s) = workload.build_layer_weights(
            spec, experts=[inverse[n] for n in range(lo, hi)], gen_device=gen_device, device=dev)
        gate_up = {(remap[e] if e < E else E): w for e, w in gu_o.items()}
        down = {(remap[e] if e < E else E): w for e, w in dn_o.items()}
        self.has_shared = spec.shared_inter > 0
        # activation format of EVERY expert (also the remote ones) by new id: decides what is sent
        tags_orig = [tag_of(workload.parse_scheme(s)) for s in gu_s]
        self._tag1 = [tags_orig[inverse[n]] for n in range(E)] + [tags_orig[E] if self.has_shared else 0]
        # routing + per-token quantiser reuse the single-GPU layer's machinery without its compute core
        self.front = MoELayer.__new__(MoELayer)
        f = self.front
        f.E, f.topk, f.H, f.I, f.Is, f.device, f.T, f.R = E, k, H, I, spec.shared_inter, dev, T, T * k
        f.counts = torch.zeros(E, **i32)
        f.row_start = torch.zeros(E + 1, **i32)
        f.row_expert = torch.zeros(T * k, **i32)
        f.row_token = torch.zeros(T * k, dtype=torch.int64, device=dev)
        f.slot_row = torch.zeros(T * k, **i32)
        f.route_ws = torch.zeros(_lib.lib().mxmoe_route_workspace_bytes(T * k, 1, E) // 4 + 1, **i32)
        f.tag1 = torch.tensor(self._tag1, **i32)
        used = set(self._tag1[:E]) | ({self._tag1[E]} if self.has_shared else set())
        self.tq = TokenQuant(T, H, used, spec.rotate, signs, dev)

        # records: packed row (P fp16 elements) + 8 elements carrying the per-token scale
        self.P = record_stride(H, set(self._tag1[:E]))
        self.rec = self.P + 8
        self.R_send = T * k
        self.R_recv = int(T * k * capacity_factor)
        self.send = torch.zeros(self.R_send, self.rec, **f16)
        self.recv = torch.zeros(self.R_recv, self.rec, **f16)
        self.ret = torch.zeros(self.R_send, H, **f16)            # expert outputs coming home
        self.out = torch.zeros(T, H, **f16)

        nseg = self.world * (hi - lo)
        self.seg_expert = [e for _ in range(self.world) for e in range(lo, hi)]
        self.seg_tab = torch.zeros(2, max(nseg, 1), **i32)                      # [m; row0]
        self.seg_tab_host = torch.zeros(2, max(nseg, 1), dtype=torch.int32).pin_memory()
        self.seg_expert_dev = torch.tensor(self.seg_expert or [0], **i32)
        self.recv_row_expert = torch.zeros(self.R_recv, **i32)
        self.counts_all = torch.zeros(self.world * E, **i32)
        self.counts_host = torch.zeros(self.world, E, dtype=torch.int32).pin_memory()
        self.ids_new = torch.zeros(T, k, **i32)
        self._gate_up, self._down = gate_up, down
        self._core = None
        self.launches_per_step = 9
        self.profile = False          # record CUDA events between the phases of forward()
        self.phase_ms = {}

    def _build_core(self, hidden):
        spec = self.spec
        shared = None
        if self.has_shared:
            a_ptr, sa_ptr = self.tq.rows_of(self._tag1[spec.num_experts], hidden)
            shared = {"tokens": spec.tokens, "a_ptr": a_ptr, "sa_ptr": sa_ptr}
        self._core = ExpertCompute(
            spec.num_experts, spec.hidden, spec.inter, self._gate_up, self._down, self.R_recv, self.seg_expert,
            self.seg_tab[0], self.seg_tab[1], self.recv_row_expert, self.recv.view(-1), self.rec,
            self.recv.data_ptr() + self.P * 2, self.rec, self.device, shared=shared, shared_inter=spec.shared_inter,
            tag_fn=tag_of)     # dispatched rows stay packed (half the NVLink bytes of the expanded format)

    def _mark(self, marks, name):
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

    def forward(self, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor | None = None):
        spec, f = self.spec, self.front
        T, k, H = spec.tokens, spec.topk, spec.hidden
        marks = []
        with torch.cuda.device(self.device):
            if self._core is None:
                self._build_core(hidden)
            self._mark(marks, "start")
            torch.index_select(self.remap, 0, topk_ids.reshape(-1), out=self.ids_new.view(-1))
            f.route(self.ids_new)
            t = self.tq.run(hidden)
            f.gather(t, T * k, self.send.view(-1), self.rec, None, rec_scale_off=self.P)
            self._mark(marks, "route+quant+gather")
            # every split size of this step: one all-gather of the counts and one small copy to the host
            dist.all_gather_into_tensor(self.counts_all, f.counts, group=self.group)
            self.counts_host.view(-1).copy_(self.counts_all, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            plan = ExchangePlan.build(self.counts_host.numpy(), self.ranges, self.rank)
            if plan.total_recv > self.R_recv:
                raise RuntimeError(f"rank {self.rank} receives {plan.total_recv} rows, capacity is {self.R_recv}: "
                                   "raise capacity_factor")
            nseg = len(plan.seg_m)
            if nseg:
                tab = self.seg_tab_host.numpy()
                tab[0, :nseg] = plan.seg_m
                tab[1, :nseg] = plan.seg_row0
                self.seg_tab.copy_(self.seg_tab_host, non_blocking=True)
                if plan.total_recv:
                    self.recv_row_expert[: plan.total_recv].copy_(torch.repeat_interleave(
                        self.seg_expert_dev[:nseg], self.seg_tab[0, :nseg].long(), output_size=plan.total_recv))
            self._mark(marks, "counts+plan")
            exchange_rows(self.recv, self.send, plan.recv_rows, plan.send_rows, self.group)
            self._mark(marks, "dispatch")
            self._core.run(plan.total_recv)
            o2 = self._core.o2.view(self.R_recv, H)
            self._mark(marks, "experts")
            exchange_rows(self.ret, o2, plan.send_rows, plan.recv_rows, self.group)
            self._mark(marks, "combine-a2a")
            _lib.check(_lib.lib().mxmoe_combine_topk(
                self.ret.data_ptr(), f.slot_row.data_ptr(),
                None if topk_weights is None else topk_weights.data_ptr(),
                self._core.o2s.data_ptr() if self.has_shared else None, self.out.data_ptr(), T, k, H,
                current_stream_ptr()))
            self._mark(marks, "combine")
            self.last_plan = plan
            if self.profile:
                torch.cuda.synchronize()
                for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                    self.phase_ms.setdefault(name, []).append(a.elapsed_time(b))
        return self.out

    def check(self) -> None:
        self._core.check()
