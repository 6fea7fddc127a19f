"""One mixed-precision MoE layer on one GPU, host-sync free.

Pipeline of one forward (all on the current CUDA stream)::

    route_topk            counts / row offsets / permutation on the device
    quant_act             gather + (Hadamard) + per-token quantise + pack      -> gate_up operands
    grouped GEMM          gate_up of every expert (+ shared expert), one launch
    silu_mul_then_quant   h = silu(gate) * up, quantise + pack                 -> down operands
    grouped GEMM          down of every expert (+ shared expert), one launch
    combine_topk          weighted un-permute (+ shared expert output)

Both problem lists are prepared once: their row counts and row offsets are read
by the kernel from the routing result in device memory, so nothing returns to
the host between layers (the reference synchronises three times per layer:
``.cpu()`` of the counts, ``cudaMalloc`` and ``cudaFree``; ref_bind.cu:449-453,
kernel_sketch.py:87-104, :142-143).

Activation stores use a slot layout: every row owns one fp16-sized slot of its
row length; an expert's packed rows start at the slot of its first row and
follow each other at their own packed pitch.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .gg import GroupedGemm, Problem, current_stream_ptr
from .weights import PackedWeight


def _tag_of(qp) -> int:
    a_bits = qp[0]
    return 0 if a_bits >= 16 else (1 if a_bits == 8 else 2)


def _pack_of(tag: int) -> int:
    return (1, 2, 4)[tag]


class MoELayer:
    """Expert weights of one layer plus preallocated activation buffers for up to ``max_tokens`` tokens.

    ``gate_up`` / ``down`` map expert id -> :class:`PackedWeight`; key ``num_experts`` is the
    shared expert.  ``local_experts`` (expert parallelism) restricts the routed experts this
    instance owns: ids outside of it are ignored by the routing kernel's caller.
    """

    def __init__(self, num_experts: int, topk: int, hidden: int, inter: int, gate_up: dict, down: dict,
                 max_tokens: int, shared_inter: int = 0, signs: torch.Tensor | None = None, rotate: bool = False,
                 device=None, max_rows: int | None = None, with_shared: bool | None = None):
        self.E, self.topk, self.H, self.I, self.Is = num_experts, topk, hidden, inter, shared_inter
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.T = max_tokens
        self.has_shared = (shared_inter > 0 and num_experts in gate_up) if with_shared is None else with_shared
        self.rows_cap = max_tokens * topk if max_rows is None else max_rows   # routed rows this instance can hold
        self.rotate = rotate
        self.per_token_quant = True    # quantise once per token, then gather (False: fused per-row kernel)
        self.gate_up, self.down = gate_up, down
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        f16 = dict(dtype=torch.float16, device=dev)
        R, T, H, I, Is, E = self.rows_cap, self.T, hidden, inter, shared_inter, num_experts
        Ts = T if self.has_shared else 0

        # routing state
        self.counts = torch.zeros(E, **i32)
        self.row_start = torch.zeros(E + 1, **i32)
        self.row_expert = torch.zeros(max(R, 1), **i32)
        self.row_token = torch.zeros(max(R, 1), dtype=torch.int64, device=dev)
        self.slot_row = torch.zeros(max(R, 1), **i32)
        ws = _lib.lib().mxmoe_route_workspace_bytes(max(R, 1), 1, E)
        self.route_ws = torch.zeros(ws // 4 + 1, **i32)
        self.signs = None if signs is None else signs.to(device=dev, dtype=torch.int8).contiguous()

        # per-expert activation tags (static): index E is the shared expert
        def tags(block):
            t = [0] * (E + 1)
            for e, w in block.items():
                t[e] = _tag_of(w.qparams)
            return t
        self._tag1, self._tag2 = tags(gate_up), tags(down)
        self.tag1 = torch.tensor(self._tag1, **i32)
        self.tag2 = torch.tensor(self._tag2, **i32)

        # stores (slot layout) and outputs
        self.q1 = torch.zeros((R + Ts) * H, **f16)
        self.s1 = torch.zeros(R + Ts, **f16)
        self.o1 = torch.zeros(R * 2 * I, **f16)                 # gate_up out, routed rows [R, 2I]
        self.o1s = torch.zeros(Ts * 2 * Is, **f16) if Ts else None
        self.q2 = torch.zeros(R * I + Ts * Is, **f16)
        self.s2 = torch.zeros(R + Ts, **f16)
        self.o2 = torch.zeros(R * H, **f16)                     # down out, routed rows [R, H]
        self.o2s = torch.zeros(Ts * H, **f16) if Ts else None
        self.out = torch.zeros(T * H, **f16)

        # token-major stores of the once-per-token quantiser (one per activation format in use)
        used = {self._tag1[e] for e in gate_up}
        self.tq_f16 = torch.zeros(T * H, **f16) if (0 in used and rotate) else None
        self.tq_q8 = torch.zeros(T * H // 2, **f16) if 1 in used else None
        self.tq_s8 = torch.zeros(T, **f16) if 1 in used else None
        self.tq_q4 = torch.zeros(T * H // 4, **f16) if 2 in used else None
        self.tq_s4 = torch.zeros(T, **f16) if 2 in used else None

        self.gg1 = GroupedGemm(self._problems(gate_up, self._tag1, self.q1, self.s1, self.o1, self.o1s,
                                               K=H, N=2 * I, Ks=H, Ns=2 * Is), device=dev)
        self.gg2 = GroupedGemm(self._problems(down, self._tag2, self.q2, self.s2, self.o2, self.o2s,
                                               K=I, N=H, Ks=Is, Ns=H), device=dev)

    # ------------------------------------------------------------------
    def _problems(self, block: dict, tag: list, q, s, o, o_shared, K, N, Ks, Ns):
        R, T, E = self.rows_cap, self.T, self.E
        probs = []
        esz = 2
        for e in sorted(k for k in block if k < E):
            w: PackedWeight = block[e]
            p = _pack_of(tag[e])
            probs.append(Problem(
                A=q, B=w.data, C=o, M=R, N=N, K=K, qparams=w.qparams,
                scale_a=s if tag[e] else None, scale_b=w.scale,
                a_rows=R * p, a_row_mul=p,
                m_dev=self.counts.data_ptr() + 4 * e, row0_dev=self.row_start.data_ptr() + 4 * e))
        if self.has_shared:
            w = block[E]
            # shared rows follow the routed slots; their count (T) and position are static
            probs.append(Problem(
                A=q.data_ptr() + R * K * esz, B=w.data, C=o_shared, M=T, N=Ns, K=Ks, qparams=w.qparams,
                scale_a=(s.data_ptr() + R * esz) if tag[E] else None, scale_b=w.scale))
        return probs

    def _act(self, fn, **kw):
        a = _lib.ActArgs()
        for k, v in kw.items():
            setattr(a, k, v.data_ptr() if isinstance(v, torch.Tensor) else v)
        _lib.check(fn(C.byref(a), current_stream_ptr()))

    # ------------------------------------------------------------------
    def route(self, topk_ids: torch.Tensor) -> None:
        T, k = topk_ids.shape
        assert T * k <= self.rows_cap and topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()
        a = _lib.RouteArgs()
        a.topk_ids, a.counts, a.row_start = topk_ids.data_ptr(), self.counts.data_ptr(), self.row_start.data_ptr()
        a.row_expert, a.row_token, a.slot_row = (self.row_expert.data_ptr(), self.row_token.data_ptr(),
                                                 self.slot_row.data_ptr())
        a.workspace, a.workspace_bytes = self.route_ws.data_ptr(), self.route_ws.numel() * 4
        a.num_tokens, a.topk, a.num_experts = T, k, self.E
        _lib.check(_lib.lib().mxmoe_route_topk(C.byref(a), current_stream_ptr()))

    def experts_forward(self, hidden: torch.Tensor, rows: int) -> None:
        """quant -> gate_up -> silu*mul+quant -> down over the rows already described by the routing state.

        ``rows`` is the number of routed rows (static upper bound of this step: T * topk locally,
        or the receive capacity under expert parallelism); ``hidden`` is what ``row_token`` indexes.
        """
        lib = _lib.lib()
        T = hidden.shape[0] if self.has_shared else 0
        R = self.rows_cap
        assert rows <= R
        # the shared expert's rows sit right after the R routed slots: describe them by rows_routed = R
        # when a shared expert is present (rows between `rows` and R are simply not produced).
        if self.has_shared:
            assert rows == R, "with a shared expert the routed row count must equal the capacity"
        if self.per_token_quant:
            t = _lib.TokenQuantArgs()
            t.inp, t.k, t.num_tokens, t.rotate = hidden.data_ptr(), self.H, hidden.shape[0], 1 if self.rotate else 0
            t.signs = None if self.signs is None else self.signs.data_ptr()
            for name in ("f16", "q8", "s8", "q4", "s4"):
                buf = getattr(self, "tq_" + name)
                setattr(t, name, None if buf is None else buf.data_ptr())
            _lib.check(lib.mxmoe_quant_tokens(C.byref(t), current_stream_ptr()))
            a = _lib.ActArgs()
            a.q_store, a.s_store = self.q1.data_ptr(), self.s1.data_ptr()
            a.row_expert, a.row_token = self.row_expert.data_ptr(), self.row_token.data_ptr()
            a.exp_qtag, a.exp_row_start = self.tag1.data_ptr(), self.row_start.data_ptr()
            a.k, a.k_shared, a.rows_routed, a.rows_total, a.num_experts = self.H, self.H, rows, rows + T, self.E
            _lib.check(lib.mxmoe_gather_rows(C.byref(a), C.byref(t), current_stream_ptr()))
        else:
            self._act(lib.mxmoe_quant_act, inp=hidden, in_shared=None, q_store=self.q1, s_store=self.s1,
                      row_expert=self.row_expert, row_token=self.row_token, exp_qtag=self.tag1,
                      exp_row_start=self.row_start, exp_q_off=None, exp_s_off=None, signs=self.signs,
                      k=self.H, k_shared=self.H, rows_routed=rows, rows_total=rows + T, num_experts=self.E,
                      rotate=1 if self.rotate else 0)
        self.gg1.run()
        self._act(lib.mxmoe_silu_mul_then_quant, inp=self.o1, in_shared=self.o1s, q_store=self.q2, s_store=self.s2,
                  row_expert=self.row_expert, row_token=None, exp_qtag=self.tag2, exp_row_start=self.row_start,
                  exp_q_off=None, exp_s_off=None, signs=None, k=self.I, k_shared=self.Is if self.has_shared else self.I,
                  rows_routed=rows, rows_total=rows + T, num_experts=self.E, rotate=0)
        self.gg2.run()

    def forward(self, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor | None = None):
        """``[T, H]`` fp16 hidden states + ``[T, topk]`` int32 expert ids (+ fp32 gate weights) -> ``[T, H]`` fp16."""
        T = hidden.shape[0]
        assert T == self.T, "this layer instance was sized for a fixed token count"
        with torch.cuda.device(self.device):
            self.route(topk_ids)
            self.experts_forward(hidden, T * self.topk)
            out = self.out.view(self.T, self.H)
            _lib.check(_lib.lib().mxmoe_combine_topk(
                self.o2.data_ptr(), self.slot_row.data_ptr(),
                None if topk_weights is None else topk_weights.data_ptr(),
                self.o2s.data_ptr() if self.has_shared else None, out.data_ptr(), T, self.topk, self.H,
                current_stream_ptr()))
        return out

    def check(self) -> None:
        self.gg1.check()
        self.gg2.check()

    # algorithmic traffic of the two grouped GEMMs for given per-expert row counts (bytes)
    def gemm_bytes(self, counts: list[int]) -> int:
        total = 0
        for block, K, N, Ks, Ns in ((self.gate_up, self.H, 2 * self.I, self.H, 2 * self.Is),
                                    (self.down, self.I, self.H, self.Is, self.H)):
            for e, w in block.items():
                m = self.T if e == self.E else counts[e]
                if m == 0:
                    continue
                k, n = (Ks, Ns) if e == self.E else (K, N)
                a_bits = w.qparams[0]
                total += m * k * a_bits // 8 + w.nbytes() + m * n * 2 + (m * 2 if a_bits < 16 else 0)
        return total
