"""Expert-parallel MoE layer: one process per GPU, experts sharded, tokens data-parallel.  (The reference has
no distributed code; this is the multi-GPU form of the path described by the benchmark configurations.)

Two transports move the rows:

``p2p`` (default) - no host round trip and no library all-to-all.  Per step and rank::

    route_topk (global expert ids)  ->  rows sorted by expert = grouped by destination rank
    quant_tokens                    ->  token-major quantised stores
    ep_sync(counts)                 ->  every rank's counts written into every peer + flag barrier: every rank knows
                                        every split size, on the device, without a library collective
    ep_plan (device)                ->  receive-side segment tables, send-side row offsets
    ep_dispatch_rows                ->  packed row + scale written straight into the owner's receive store
                                        (plain stores to peer memory over NVLink)
    ep_sync                         ->  flag barrier in peer-mapped memory, stream ordered, bounded wait
    grouped GEMM, silu*mul+quantise, grouped GEMM
                                    ->  one problem per (source rank, local expert); the epilogue of the down
                                        projection stores every segment straight into the buffer of the rank its
                                        rows came from, at their place in that rank's order (peer stores again)
    ep_sync, combine_topk (+ shared expert, computed locally on the rank's own tokens)

The p2p step contains no NCCL call and never returns to the host, so it is replayed from a CUDA graph
(``forward_graph``).

``nccl`` - ``all_to_all_single`` for both exchanges; NCCL needs the split sizes on the host, which costs one
device->host copy and a stream synchronisation per step.

TMA only ever reads this GPU's own memory (the receive store); no load uses cluster multicast.
"""
from __future__ import annotations

import dataclasses
import ctypes as C
import os

import torch
import torch.distributed as dist

from . import _lib
from .gg import current_stream_ptr
from .layer import ExpertCompute, MoELayer, TokenQuant, internal_tag, record_stride, tag_of


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


def balanced_placement(loads, world: int):
    """Experts placed by longest-processing-time-first on expected loads (e.g. the row counts of a calibration
    gate trace), every rank holding at most ceil(E / world) experts.  Same return value as
    :func:`strided_placement`: experts renumbered rank-major."""
    num_experts = len(loads)
    cap = -(-num_experts // world)
    order = sorted(range(num_experts), key=lambda e: (-float(loads[e]), e))
    total, members = [0.0] * world, [[] for _ in range(world)]
    for e in order:
        r = min((r for r in range(world) if len(members[r]) < cap), key=lambda r: (total[r], r))
        total[r] += float(loads[e])
        members[r].append(e)
    inverse = [e for r in range(world) for e in sorted(members[r])]
    remap = [0] * num_experts
    for new, e in enumerate(inverse):
        remap[e] = new
    ranges, lo = [], 0
    for r in range(world):
        ranges.append((lo, lo + len(members[r])))
        lo += len(members[r])
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
                 placement: str = "balanced", transport: str | None = None, loads=None, granularity: int = 2,
                 dispatch_format: str | None = None):
        from . import workload
        self.spec, self.device, self.group = spec, torch.device(device), group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.transport = transport or os.environ.get("MXMOE_EP_TRANSPORT", "p2p")
        # int4 activation rows cross NVLink either packed (two codes per byte: half the bytes, but the receiving
        # GEMM then has to expand them in shared memory, which costs it about a third of its speed) or already
        # expanded to one byte per code (the layer's internal format): expanded is the default on NVLink
        self.dispatch_format = dispatch_format or os.environ.get("MXMOE_EP_DISPATCH", "expanded")
        if self.dispatch_format not in ("expanded", "packed"):
            raise ValueError(f"unknown dispatch format {self.dispatch_format!r}")
        self._tag_fn = internal_tag if self.dispatch_format == "expanded" else tag_of
        if self.transport not in ("p2p", "nccl"):
            raise ValueError(f"unknown transport {self.transport!r}")
        E0, T, k, H, I = spec.num_experts, spec.tokens, spec.topk, spec.hidden, spec.inter
        # Virtual experts: an expert whose expected load exceeds 1 / (world * granularity) of the rows is
        # REPLICATED (same weights on several ranks) and its rows are dealt to the replicas by token index, so
        # that no single expert can hold more than a rank's fair share (the hottest expert of a skewed routing
        # otherwise bounds the step).  Everything below works on the virtual experts; vorig maps them back.
        reps = [1] * E0
        if placement == "balanced":
            # expected rows per expert: a calibration routing sample of the workload unless the caller has a trace
            if loads is None:
                cal, _ = workload.make_routing(spec, seed=1234)
                loads = torch.bincount(cal.reshape(-1).long(), minlength=E0).tolist()
            if self.world > 1 and granularity > 0:
                target = max(1.0, float(sum(loads)) / (self.world * granularity))
                reps = [max(1, min(self.world, -(-int(l) // int(target + 0.5)))) for l in loads]
        self.vorig = [e for e in range(E0) for _ in range(reps[e])]
        E = len(self.vorig)
        self.replicated = E > E0
        if placement == "balanced":
            vloads = [float(loads[e]) / reps[e] for e in self.vorig]
            remap, inverse, self.ranges = balanced_placement(vloads, self.world)
        elif placement == "strided":
            remap, inverse, self.ranges = strided_placement(E, self.world)
        else:
            remap, inverse, self.ranges = list(range(E)), list(range(E)), expert_ranges(E, self.world)
        lo, hi = self.ranges[self.rank]
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        f16 = dict(dtype=torch.float16, device=dev)
        self.remap = torch.tensor(remap, **i32)                       # virtual expert -> new (rank-major) id
        vbase = [0] * E0
        for e in range(1, E0):
            vbase[e] = vbase[e - 1] + reps[e - 1]
        self.vbase = torch.tensor(vbase, **i32)                       # original expert -> its first virtual expert
        self.vrep = torch.tensor(reps, **i32)

        # weights of the local experts, keyed by their NEW ids (the shared expert keeps key E)
        local_orig = [self.vorig[inverse[n]] for n in range(lo, hi)]
        gu_o, dn_o, signs, (gu_s, dn_s) = workload.build_layer_weights(
            spec, experts=sorted(set(local_orig)), gen_device=gen_device, device=dev)
        gate_up = {n: gu_o[self.vorig[inverse[n]]] for n in range(lo, hi)}
        down = {n: dn_o[self.vorig[inverse[n]]] for n in range(lo, hi)}
        self.has_shared = spec.shared_inter > 0
        if self.has_shared:
            gate_up[E], down[E] = gu_o[E0], dn_o[E0]
        # activation format of EVERY expert (also the remote ones) by new id: decides what is sent
        tags_orig = [self._tag_fn(workload.parse_scheme(s)) for s in gu_s]
        self._tag1 = [tags_orig[self.vorig[inverse[n]]] for n in range(E)] + [tags_orig[E0] if self.has_shared else 0]
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
        # the routing kernels renumber the ids as they read them: original expert -> one of its copies (by token
        # index) -> the copy's rank-major id
        f.id_map, f.num_ids = self.remap, E0
        f.rep_base, f.rep_count = (self.vbase, self.vrep) if self.replicated else (None, None)
        used = set(self._tag1[:E]) | ({self._tag1[E]} if self.has_shared else set())
        self.tq = TokenQuant(T, H, used, spec.rotate, signs, dev)

        # records: packed row (P fp16 elements) + 8 elements carrying the per-token scale
        self.P = record_stride(H, set(self._tag1[:E]))
        self.rec = self.P + 8
        self.E = E
        self.R_send = T * k
        self.R_recv = int(T * k * capacity_factor)
        self.out = torch.zeros(T, H, **f16)
        if self.transport == "p2p":
            # receive store and home-coming buffer live in symmetric memory: every rank maps every peer's copy
            import torch.distributed._symmetric_memory as symm
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer mappings only
            grp = group if group is not None else dist.group.WORLD
            self.recv = symm.empty((self.R_recv, self.rec), dtype=torch.float16, device=dev)
            self.ret = symm.empty((self.R_send, H), dtype=torch.float16, device=dev)
            self.recv.zero_()
            self.ret.zero_()
            self._h_recv = symm.rendezvous(self.recv, grp)
            self._h_ret = symm.rendezvous(self.ret, grp)
            self.peer_recv = torch.tensor([int(p) for p in self._h_recv.buffer_ptrs], dtype=torch.int64, device=dev)
            self.peer_ret = [int(p) for p in self._h_ret.buffer_ptrs]
            self.peer_ret_dev = torch.tensor(self.peer_ret, dtype=torch.int64, device=dev)
            self.send = None
            # sync block: arrival flags, error word, epoch, and one payload slot per rank that receives the ranks'
            # per-expert row counts (see mxmoe_ep_sync)
            self.sync = symm.empty((128 + self.world * E,), dtype=torch.int32, device=dev)
            self.sync.zero_()
            self._h_sync = symm.rendezvous(self.sync, grp)
            self.peer_sync = torch.tensor([int(p) for p in self._h_sync.buffer_ptrs], dtype=torch.int64, device=dev)
            torch.cuda.synchronize(dev)
            dist.barrier(group=group)        # every rank's sync block is zeroed before anybody's first barrier
        else:
            self.send = torch.zeros(self.R_send, self.rec, **f16)
            self.recv = torch.zeros(self.R_recv, self.rec, **f16)
            self.ret = torch.zeros(self.R_send, H, **f16)        # expert outputs coming home

        nseg = self.world * (hi - lo)
        # p2p: the receive store is ordered (expert, source rank), so the grouped GEMMs take one problem per local
        # expert; nccl (all-to-all): (source rank, expert), one problem per segment
        self.expert_major = self.transport == "p2p"
        self.seg_expert = list(range(lo, hi)) if self.expert_major else [e for _ in range(self.world) for e in range(lo, hi)]
        self.exp_tab = torch.zeros(2, max(hi - lo, 1), **i32)                   # [rows; first row] of every local expert
        self.row_dst = torch.zeros(self.R_recv, dtype=torch.int64, device=dev)  # where every received row's result goes
        self.seg_tab = torch.zeros(2, max(nseg, 1), **i32)                      # [m; row0]
        self.seg_tab_host = torch.zeros(2, max(nseg, 1), dtype=torch.int32).pin_memory()
        self.seg_expert_dev = torch.tensor(self.seg_expert or [0], **i32)
        self.recv_row_expert = torch.zeros(self.R_recv, **i32)
        # all ranks' per-expert row counts: the payload slots of the sync block (p2p) or an all-gather buffer (nccl)
        self.counts_all = self.sync[128:] if self.transport == "p2p" else torch.zeros(self.world * E, **i32)
        self.counts_host = torch.zeros(self.world, E, dtype=torch.int32).pin_memory()
        # device-side plan of the p2p transport
        self.range_lo = torch.tensor([r[0] for r in self.ranges] + [E], **i32)
        self.seg_src_row0 = torch.zeros(max(nseg, 1), **i32)
        self.dst_row0 = torch.zeros(E, **i32)
        self.exp_owner = torch.zeros(E, **i32)
        self.total_recv = torch.zeros(2, **i32)
        self._gate_up, self._down = gate_up, down
        self._core = None
        self.launches_per_step = 9
        self.profile = False          # record CUDA events between the phases of forward()
        self.phase_ms = {}

    def _build_core(self, hidden):
        spec = self.spec
        shared = None
        if self.has_shared:
            a_ptr, sa_ptr = self.tq.rows_of(self._tag1[self.E], hidden)
            shared = {"tokens": spec.tokens, "a_ptr": a_ptr, "sa_ptr": sa_ptr}
        p2p = self.transport == "p2p"
        # p2p: one problem per local expert over the rows of all source ranks; every result row goes to the address
        # the plan put into row_dst (its row in the home-coming buffer of the rank it came from)
        tab = self.exp_tab if p2p else self.seg_tab
        self._core = ExpertCompute(
            self.E, spec.hidden, spec.inter, self._gate_up, self._down, self.R_recv, self.seg_expert,
            tab[0], tab[1], self.recv_row_expert, self.recv.view(-1), self.rec,
            self.recv.data_ptr() + self.P * 2, self.rec, self.device, shared=shared, shared_inter=spec.shared_inter,
            tag_fn=self._tag_fn,
            down_row_ptrs=self.row_dst if p2p else None, rows_dev=self.total_recv if p2p else None)

    def _mark(self, marks, name):
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

    def _sync(self, payload: torch.Tensor | None = None):
        """Every rank's earlier kernels on this stream (their peer stores included) are complete before any
        rank's later kernels start: flags in peer-mapped memory, ordered on the stream, no host involvement and
        no library collective.  ``payload``: this rank's per-expert counts, delivered to every rank on the way."""
        a = _lib.EpSyncArgs()
        a.peer_sync, a.local_sync = self.peer_sync.data_ptr(), self.sync.data_ptr()
        a.payload = None if payload is None else payload.data_ptr()
        a.world, a.rank = self.world, self.rank
        a.payload_len, a.payload_cap = (0 if payload is None else payload.numel()), self.E
        a.timeout_ms = 0
        _lib.check(_lib.lib().mxmoe_ep_sync(C.byref(a), current_stream_ptr()))

    def _forward_p2p(self, hidden, topk_ids, topk_weights):
        spec, f = self.spec, self.front
        T, k, H, E = spec.tokens, spec.topk, spec.hidden, self.E
        lib = _lib.lib()
        marks = []
        with torch.cuda.device(self.device):
            if self._core is None:
                self._build_core(hidden)
            self._mark(marks, "start")
            f.route(topk_ids)
            t = self.tq.run(hidden)
            self._mark(marks, "route+quant")
            self._sync(payload=f.counts)
            lo, hi = self.ranges[self.rank]
            pa = _lib.EpPlanArgs()
            pa.counts_all, pa.range_lo = self.counts_all.data_ptr(), self.range_lo.data_ptr()
            pa.world, pa.rank, pa.num_experts, pa.experts_local = self.world, self.rank, E, hi - lo
            pa.recv_capacity = self.R_recv
            pa.seg_m, pa.seg_row0 = self.seg_tab[0].data_ptr(), self.seg_tab[1].data_ptr()
            pa.seg_src_row0, pa.recv_row_expert = self.seg_src_row0.data_ptr(), self.recv_row_expert.data_ptr()
            pa.total_recv, pa.dst_row0, pa.exp_owner = self.total_recv.data_ptr(), self.dst_row0.data_ptr(), self.exp_owner.data_ptr()
            pa.layout = 1
            pa.exp_m, pa.exp_row0, pa.row_dst = self.exp_tab[0].data_ptr(), self.exp_tab[1].data_ptr(), self.row_dst.data_ptr()
            pa.peer_ret, pa.ret_row_bytes = self.peer_ret_dev.data_ptr(), H * 2
            _lib.check(lib.mxmoe_ep_plan(C.byref(pa), current_stream_ptr()))
            da = _lib.EpDispatchArgs()
            da.peer_base, da.row_expert, da.row_token = self.peer_recv.data_ptr(), f.row_expert.data_ptr(), f.row_token.data_ptr()
            da.exp_row_start, da.exp_qtag = f.row_start.data_ptr(), f.tag1.data_ptr()
            da.dst_row0, da.exp_owner = self.dst_row0.data_ptr(), self.exp_owner.data_ptr()
            da.rows, da.k, da.rec_bytes, da.scale_off_bytes, da.recv_capacity = T * k, H, self.rec * 2, self.P * 2, self.R_recv
            _lib.check(lib.mxmoe_ep_dispatch_rows(C.byref(da), C.byref(t), current_stream_ptr()))
            self._mark(marks, "plan+dispatch")
            self._sync()
            self._mark(marks, "barrier")
            self._core.run(self.R_recv)
            self._mark(marks, "experts")
            self._sync()
            self._mark(marks, "barrier2")
            _lib.check(lib.mxmoe_combine_topk(
                self.ret.data_ptr(), f.slot_row.data_ptr(),
                None if topk_weights is None else topk_weights.data_ptr(),
                self._core.o2s.data_ptr() if self.has_shared else None, self.out.data_ptr(), T, k, H,
                current_stream_ptr()))
            self._mark(marks, "combine")
            if self.profile:
                torch.cuda.synchronize()
                for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                    self.phase_ms.setdefault(name, []).append(a.elapsed_time(b))
        return self.out

    def forward(self, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor | None = None):
        if self.transport == "p2p":
            return self._forward_p2p(hidden, topk_ids, topk_weights)
        spec, f = self.spec, self.front
        T, k, H = spec.tokens, spec.topk, spec.hidden
        marks = []
        with torch.cuda.device(self.device):
            if self._core is None:
                self._build_core(hidden)
            self._mark(marks, "start")
            f.route(topk_ids)
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

    def forward_graph(self, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor | None = None):
        """Same as :meth:`forward` with the ``p2p`` transport, replayed from a CUDA graph: the step never returns to
        the host (its two collectives, the all-gather of the counts and the barriers, are stream-ordered and are
        captured with the kernels), so its ~20 launches become one.  Captured once per set of argument buffers."""
        if self.transport != "p2p":
            return self.forward(hidden, topk_ids, topk_weights)
        key = (hidden.data_ptr(), topk_ids.data_ptr(), None if topk_weights is None else topk_weights.data_ptr())
        if getattr(self, "_graph_key", None) != key:
            with torch.cuda.device(self.device):
                profile, self.profile = self.profile, False
                for _ in range(2):
                    self.forward(hidden, topk_ids, topk_weights)        # builds descriptors, warms up the collectives
                self.check()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.forward(hidden, topk_ids, topk_weights)
                self._graph, self._graph_key, self.profile = g, key, profile
        self._graph.replay()
        return self.out

    def check(self) -> None:
        self._core.check()
        if self.transport == "p2p":
            missing = int(self.sync[64].item())
            if missing:
                self.sync[64].zero_()
                raise RuntimeError(f"rank {self.rank}: a barrier gave up waiting for rank {missing - 1}")
            wanted = int(self.total_recv[1].item())
            if wanted:
                # the report is taken: clear it, so that later steps that fit are not blamed for this one.  The rows
                # beyond the capacity were dropped by their senders, so the outputs of the steps since the last
                # check() are not valid for the tokens that were routed here.
                self.total_recv[1].zero_()
                raise RuntimeError(f"rank {self.rank} was sent {wanted} rows, capacity is {self.R_recv}: raise capacity_factor")
