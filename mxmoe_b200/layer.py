"""One mixed-precision MoE layer on one GPU, host-sync free.

Pipeline of one forward (all on the current CUDA stream)::

    route_topk            counts / row offsets / permutation on the device
    quant_tokens_scatter  (Hadamard) + per-token quantise + pack, once per token, written from registers
                          into the expert-sorted record of each of the token's routed slots
                          (top-k > 8: quant_tokens into token-major stores, then gather_rows)
    grouped GEMM          gate_up of every expert (+ shared expert), one launch
    silu_mul_then_quant   h = silu(gate) * up, quantise + pack
    grouped GEMM          down of every expert (+ shared expert), one launch
    combine_topk          weighted un-permute (+ shared expert output)

Both problem lists are prepared once: their row counts and row offsets are read
by the kernel from device memory, so nothing returns to the host between layers
(the reference synchronises three times per layer: ``.cpu()`` of the counts,
``cudaMalloc`` and ``cudaFree``; ref_bind.cu:449-453, kernel_sketch.py:87-104,
:142-143).

Activation stores use a *record layout*: every row owns one record of fixed size
(the widest packed row among the experts that can appear in the store); row r is
at ``r * stride`` whatever its format, and each expert's TMA descriptor uses that
stride as its row pitch.  Offsets therefore never depend on per-expert counts and
a store can be handed to another GPU as it is.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib
from .gg import OUT_FP16, OUT_SILU, GroupedGemm, Problem, current_stream_ptr
from .weights import PackedWeight


def default_fuse_silu() -> bool:
    """Whether layers apply silu(gate) * up in the epilogue of the gate_up GEMM when nobody says otherwise
    (environment variable MXMOE_FUSE_SILU = 1 | 0, read when a layer is built)."""
    return os.environ.get("MXMOE_FUSE_SILU", "0") == "1"


def tag_of(qp) -> int:
    """Activation format of a scheme: 0 fp16, 1 int8 per token, 2 int4 per token."""
    a_bits = qp[0]
    return 0 if a_bits >= 16 else (1 if a_bits == 8 else 2)


def internal_tag(qp) -> int:
    """Format the layer uses internally: 4-bit activations are kept expanded (tag 3: one byte 16*q per
    code), so that the grouped GEMM only has to convert the weights."""
    t = tag_of(qp)
    return 3 if t == 2 else t


def pack_of(tag: int) -> int:
    """Codes per fp16-sized element of a stored row: fp16 1, int8 2, int4 packed 4, int4 expanded 2."""
    return (1, 2, 4, 2)[tag]


def record_stride(row_len: int, tags) -> int:
    """Record size (fp16 elements) that holds a row of ``row_len`` values in the widest of ``tags``."""
    return max(row_len // pack_of(t) for t in tags)


def _act_call(fn, **kw):
    a = _lib.ActArgs()
    for k, v in kw.items():
        setattr(a, k, v.data_ptr() if isinstance(v, torch.Tensor) else v)
    _lib.check(fn(C.byref(a), current_stream_ptr()))


class ExpertCompute:
    """gate_up GEMM -> silu*mul+quantise -> down GEMM over rows that already sit in a record store.

    The rows are described by *segments*: segment i holds ``seg_m[i]`` consecutive rows starting at
    row ``seg_row0[i]`` that all belong to expert ``seg_expert[i]`` (both numbers live in device
    memory).  On one GPU a segment is an expert; under expert parallelism it is a (source rank,
    expert) pair.  ``row_expert`` gives the expert of every row (for the format of the second
    quantiser).  An optional shared expert runs over ``shared["tokens"]`` token-major rows in the
    same two launches.
    """

    def __init__(self, num_experts, hidden, inter, gate_up: dict, down: dict, rows_cap: int,
                 seg_expert, seg_m: torch.Tensor, seg_row0: torch.Tensor, row_expert: torch.Tensor,
                 q1: torch.Tensor, rec1: int, scale1_ptr: int, scale1_stride: int, device,
                 shared: dict | None = None, shared_inter: int = 0, tag_fn=internal_tag,
                 down_out: list | None = None, rows_dev: torch.Tensor | None = None,
                 online_had: torch.Tensor | None = None, fuse_silu: bool | None = None,
                 down_row_ptrs: torch.Tensor | None = None):
        self.E, self.H, self.I, self.Is = num_experts, hidden, inter, shared_inter
        fuse_silu = default_fuse_silu() if fuse_silu is None else fuse_silu
        self.R, self.device = rows_cap, device
        self.gate_up, self.down = gate_up, down
        self.row_expert, self.seg_expert = row_expert, list(seg_expert)
        self.shared = shared
        # down_out[i] = (C pointer, pointer to the first C row) of segment i: the down projection then stores the
        # segment's rows there (e.g. straight into the buffer of the rank they came from) instead of into o2.
        # down_row_ptrs: int64 device table with the address of every row's result (rows of one segment may then go
        # to different buffers); excludes down_out.
        # rows_dev: live row count on the device (sizes the work of the second quantiser)
        self.rows_dev = rows_dev
        dev, R, H, I = device, rows_cap, hidden, inter
        # online rotation of the down-projection input of the routed experts (rotation.py:403-421): a K x K Hadamard
        # factor (fp16, on the device); the down weights must have been rotated with the same matrix offline
        self.had_k = None if online_had is None else online_had.to(device=dev, dtype=torch.float16).contiguous()
        f16 = dict(dtype=torch.float16, device=dev)
        local = sorted(set(self.seg_expert))

        def tags(block, fn):
            t = [0] * (num_experts + 1)
            for e, w in block.items():
                t[e] = fn(w.qparams)
            return t
        # the first GEMM reads whatever format the caller stored (tag_fn); the second one reads this
        # object's own store, always in the internal format
        self._tag1, self._tag2 = tags(gate_up, tag_fn), tags(down, internal_tag)
        self.tag2 = torch.tensor(self._tag2, dtype=torch.int32, device=dev)
        self.rec2 = record_stride(I, {self._tag2[e] for e in local}) if local else I
        self.o1 = torch.zeros(max(R, 1) * 2 * I, **f16)        # gate_up output rows [R, 2I]
        self.q2 = torch.zeros(max(R, 1) * self.rec2, **f16)    # down input records
        self.s2 = torch.zeros(max(R, 1), **f16)
        self.o2 = torch.zeros(max(R, 1) * H, **f16)            # down output rows [R, H]
        # silu(gate) * up in the epilogue of the first GEMM (the 2 I wide fp16 rows never reach memory): available
        # when every routed expert's gate_up weights are packed along K and I is a multiple of 64
        self.fused_silu = bool(fuse_silu) and I % 64 == 0 and bool(local) and \
            all(gate_up[e].qparams[1] != 4 or gate_up[e].qparams[0] != 16 for e in local)
        if self.had_k is not None or self.fused_silu:
            self.h16 = torch.zeros(max(R, 1), I, **f16)        # silu(gate) * up rows (rotated in place if had_k)
            self.tag0 = torch.zeros(num_experts + 1, dtype=torch.int32, device=dev)

        p1, p2 = [], []
        # Launch order: the segments of one expert next to each other.  The tiles of a launch are walked in problem
        # order by all CTAs together, so an expert's weights are then read from HBM once however many segments
        # (source ranks) it has, and outputs that go to different ranks (down_out) are in flight at the same time
        # instead of one destination after the other.
        for i in sorted(range(len(self.seg_expert)), key=lambda i: (self.seg_expert[i], i)):
            e = self.seg_expert[i]
            m_ptr, r_ptr = seg_m.data_ptr() + 4 * i, seg_row0.data_ptr() + 4 * i
            w1: PackedWeight = gate_up[e]
            w2: PackedWeight = down[e]
            p1.append(Problem(A=q1, B=w1.data, C=self.h16 if self.fused_silu else self.o1, M=R, N=2 * I, K=H,
                              qparams=w1.qparams, out_mode=OUT_SILU if self.fused_silu else OUT_FP16,
                              scale_a=scale1_ptr if self._tag1[e] else None, scale_b=w1.scale,
                              a_rows=R, lda_bytes=rec1 * 2, sa_stride=scale1_stride, m_dev=m_ptr, row0_dev=r_ptr,
                              a_expanded=1 if self._tag1[e] == 3 else 0))
            c_out, c_row0 = (self.o2, None) if down_out is None else down_out[i]
            p2.append(Problem(A=self.q2, B=w2.data, C=c_out, M=R, N=H, K=I, qparams=w2.qparams,
                              scale_a=self.s2 if self._tag2[e] else None, scale_b=w2.scale,
                              a_rows=R, lda_bytes=self.rec2 * 2, m_dev=m_ptr, row0_dev=r_ptr,
                              a_expanded=1 if self._tag2[e] == 3 else 0, c_row0_dev=c_row0, c_row_ptrs=down_row_ptrs))
        if shared is not None:
            T, Is, E = shared["tokens"], shared_inter, num_experts
            w1, w2 = gate_up[E], down[E]
            t2 = self._tag2[E]
            self.rec2s = Is // pack_of(t2)
            self.o1s = torch.zeros(T * 2 * Is, **f16)
            self.q2s = torch.zeros(T * self.rec2s, **f16)
            self.s2s = torch.zeros(T, **f16)
            self.o2s = torch.zeros(T * H, **f16)
            # the shared expert reads the token-major store of its format directly: no copy.  Its row count lives on
            # the device like the routed experts' (always T; a benchmark that times a subset of the problems zeroes it)
            self.shared_m = torch.tensor([T], dtype=torch.int32, device=dev)
            p1.append(Problem(A=shared["a_ptr"], B=w1.data, C=self.o1s, M=T, N=2 * Is, K=H, qparams=w1.qparams,
                              scale_a=shared["sa_ptr"] if self._tag1[E] else None, scale_b=w1.scale,
                              a_expanded=1 if self._tag1[E] == 3 else 0, m_dev=self.shared_m))
            p2.append(Problem(A=self.q2s, B=w2.data, C=self.o2s, M=T, N=H, K=Is, qparams=w2.qparams,
                              scale_a=self.s2s if t2 else None, scale_b=w2.scale, a_expanded=1 if t2 == 3 else 0,
                              m_dev=self.shared_m))
        else:
            self.o2s = None
        self.gg1 = GroupedGemm(p1, device=dev)
        self.gg2 = GroupedGemm(p2, device=dev)
        # row counts live on the device; few rows per segment on average (a decode batch): small token tiles
        if self.seg_expert and rows_cap / len(self.seg_expert) <= 16 and (shared is None or shared["tokens"] <= 64):
            self.gg1.set_small_tiles(True)
            self.gg2.set_small_tiles(True)
        self.launches = 3 + (1 if shared is not None else 0)

    def run(self, rows: int) -> None:
        """``rows``: upper bound of the rows in use this step (sizes the silu launch)."""
        lib = _lib.lib()
        self.gg1.run()
        if self.fused_silu and self.had_k is None:
            # the first GEMM left h = silu(gate) * up as fp16 rows: quantise them per expert format
            _act_call(lib.mxmoe_quant_act, inp=self.h16, in_shared=None, q_store=self.q2, s_store=self.s2,
                      row_expert=self.row_expert, row_token=None, exp_qtag=self.tag2, exp_row_start=None,
                      exp_q_off=None, exp_s_off=None, signs=None, k=self.I, k_shared=self.I, rows_routed=rows,
                      rows_total=rows, num_experts=self.E, rotate=0, rec_stride=self.rec2, rec_scale_off=-1,
                      rows_dev=self.rows_dev)
        elif self.had_k is None:
            _act_call(lib.mxmoe_silu_mul_then_quant, inp=self.o1, in_shared=None, q_store=self.q2, s_store=self.s2,
                      row_expert=self.row_expert, row_token=None, exp_qtag=self.tag2, exp_row_start=None,
                      exp_q_off=None, exp_s_off=None, signs=None, k=self.I, k_shared=self.I, rows_routed=rows,
                      rows_total=rows, num_experts=self.E, rotate=0, rec_stride=self.rec2, rec_scale_off=-1,
                      rows_dev=self.rows_dev)
        else:
            # h = silu(gate) * up as fp16 rows -> h (had_K (x) H_m) / sqrt(I) in place -> quantise per expert format
            from .hadamard import hadamard_kron
            if not self.fused_silu:
                _act_call(lib.mxmoe_silu_mul_then_quant, inp=self.o1, in_shared=None, q_store=self.h16, s_store=self.s2,
                          row_expert=self.row_expert, row_token=None, exp_qtag=self.tag0, exp_row_start=None,
                          exp_q_off=None, exp_s_off=None, signs=None, k=self.I, k_shared=self.I, rows_routed=rows,
                          rows_total=rows, num_experts=self.E, rotate=0, rec_stride=self.I, rec_scale_off=-1,
                          rows_dev=self.rows_dev)
            hadamard_kron(self.h16[:rows], self.had_k, out=self.h16[:rows])
            _act_call(lib.mxmoe_quant_act, inp=self.h16, in_shared=None, q_store=self.q2, s_store=self.s2,
                      row_expert=self.row_expert, row_token=None, exp_qtag=self.tag2, exp_row_start=None,
                      exp_q_off=None, exp_s_off=None, signs=None, k=self.I, k_shared=self.I, rows_routed=rows,
                      rows_total=rows, num_experts=self.E, rotate=0, rec_stride=self.rec2, rec_scale_off=-1,
                      rows_dev=self.rows_dev)
        if self.shared is not None:
            T = self.shared["tokens"]
            _act_call(lib.mxmoe_silu_mul_then_quant, inp=self.o1s, in_shared=self.o1s, q_store=self.q2s,
                      s_store=self.s2s, row_expert=None, row_token=None, exp_qtag=self.tag2, exp_row_start=None,
                      exp_q_off=None, exp_s_off=None, signs=None, k=self.Is, k_shared=self.Is, rows_routed=0,
                      rows_total=T, num_experts=self.E, rotate=0, rec_stride=self.rec2s, rec_scale_off=-1)
        self.gg2.run()

    def check(self) -> None:
        self.gg1.check()
        self.gg2.check()


class TokenQuant:
    """Token-major stores of the once-per-token quantiser: one per activation format in use."""

    def __init__(self, tokens: int, hidden: int, tags_used, rotate: bool, signs, device):
        f16 = dict(dtype=torch.float16, device=device)
        self.T, self.H, self.rotate = tokens, hidden, rotate
        self.signs = None if signs is None else signs.to(device=device, dtype=torch.int8).contiguous()
        self.f16 = torch.zeros(tokens * hidden, **f16) if (0 in tags_used and rotate) else None
        self.q8 = torch.zeros(tokens * hidden // 2, **f16) if 1 in tags_used else None
        self.s8 = torch.zeros(tokens, **f16) if 1 in tags_used else None
        self.q4 = torch.zeros(tokens * hidden // 4, **f16) if 2 in tags_used else None
        self.q4x = torch.zeros(tokens * hidden // 2, **f16) if 3 in tags_used else None
        self.s4 = torch.zeros(tokens, **f16) if (2 in tags_used or 3 in tags_used) else None
        self.args = _lib.TokenQuantArgs()

    def fill(self, hidden: torch.Tensor) -> _lib.TokenQuantArgs:
        t = self.args
        t.inp, t.k, t.num_tokens, t.rotate = hidden.data_ptr(), self.H, hidden.shape[0], 1 if self.rotate else 0
        t.signs = None if self.signs is None else self.signs.data_ptr()
        for name in ("f16", "q8", "s8", "q4", "s4", "q4x"):
            buf = getattr(self, name)
            setattr(t, name, None if buf is None else buf.data_ptr())
        return t

    def run(self, hidden: torch.Tensor) -> _lib.TokenQuantArgs:
        t = self.fill(hidden)
        _lib.check(_lib.lib().mxmoe_quant_tokens(C.byref(t), current_stream_ptr()))
        return t

    def rows_of(self, tag: int, hidden: torch.Tensor):
        """(address of the token-major rows in format ``tag``, address of their scales or None)."""
        if tag == 0:
            return (self.f16.data_ptr() if self.f16 is not None else hidden.data_ptr()), None
        if tag == 1:
            return self.q8.data_ptr(), self.s8.data_ptr()
        return (self.q4x if tag == 3 else self.q4).data_ptr(), self.s4.data_ptr()


class MoELayer:
    """Expert weights of one layer plus preallocated activation buffers for ``max_tokens`` tokens.

    ``gate_up`` / ``down`` map expert id -> :class:`PackedWeight`; key ``num_experts`` is the shared
    expert.  ``forward`` takes a fixed-address hidden tensor per instance size (the shared expert's
    descriptor is bound to the address of the first ``hidden`` it sees when no rotation or quantiser
    produces a token-major copy).
    """

    def __init__(self, num_experts: int, topk: int, hidden: int, inter: int, gate_up: dict, down: dict,
                 max_tokens: int, shared_inter: int = 0, signs: torch.Tensor | None = None, rotate: bool = False,
                 device=None, online_had: torch.Tensor | None = None, fuse_silu: bool | None = None):
        self.E, self.topk, self.H, self.I, self.Is = num_experts, topk, hidden, inter, shared_inter
        self.fuse_silu = fuse_silu       # silu(gate) * up in the first GEMM's epilogue where the schemes allow it
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.T = max_tokens
        self.has_shared = shared_inter > 0 and num_experts in gate_up
        self.rotate = rotate
        self.online_had = online_had     # K x K Hadamard factor of the online rotation of the down-projection input
        self.gate_up, self.down = gate_up, down
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        f16 = dict(dtype=torch.float16, device=dev)
        R, T, H, E = max_tokens * topk, max_tokens, hidden, num_experts
        self.R = R

        # routing state
        self.counts = torch.zeros(E, **i32)
        self.row_start = torch.zeros(E + 1, **i32)
        self.row_expert = torch.zeros(max(R, 1), **i32)
        self.row_token = torch.zeros(max(R, 1), dtype=torch.int64, device=dev)
        self.slot_row = torch.zeros(max(R, 1), **i32)
        ws = _lib.lib().mxmoe_route_workspace_bytes(max(R, 1), 1, E)
        self.route_ws = torch.zeros(ws // 4 + 1, **i32)

        tag1 = [0] * (E + 1)
        for e, w in gate_up.items():
            tag1[e] = internal_tag(w.qparams)
        self._tag1 = tag1
        self.tag1 = torch.tensor(tag1, **i32)
        routed = [e for e in sorted(gate_up) if e < E]
        # top-k up to 8: one launch quantises every token and writes its routed rows; the token-major stores are
        # then kept only for the shared expert, which reads them in place
        self.one_pass_quant = 1 <= topk <= 8 and os.environ.get("MXMOE_QUANT_PASSES", "1") == "1"
        store_tags = {tag1[e] for e in gate_up if e >= E} if self.one_pass_quant else {tag1[e] for e in gate_up}
        self.tq = TokenQuant(T, H, store_tags, rotate, signs, dev)
        self.rec1 = record_stride(H, {tag1[e] for e in routed}) if routed else H
        self.q1 = torch.zeros(max(R, 1) * self.rec1, **f16)
        self.s1 = torch.zeros(max(R, 1), **f16)
        self.out = torch.zeros(T * H, **f16)
        self._routed = routed
        self._core = None   # built on the first forward (needs the address of `hidden` for an fp16 shared expert)

    def _build_core(self, hidden: torch.Tensor) -> None:
        shared = None
        if self.has_shared:
            a_ptr, sa_ptr = self.tq.rows_of(self._tag1[self.E], hidden)
            shared = {"tokens": self.T, "a_ptr": a_ptr, "sa_ptr": sa_ptr}
        self._hidden_ptr = hidden.data_ptr()
        # one segment per routed expert: rows [row_start[e], row_start[e] + counts[e])
        seg_m = self.counts
        seg_row0 = self.row_start
        # segments must index seg_m / seg_row0 by position: experts are 0..E-1 in order here
        assert self._routed == list(range(len(self._routed))), "single-GPU layer owns experts 0..E-1"
        self._core = ExpertCompute(self.E, self.H, self.I, self.gate_up, self.down, self.R, self._routed, seg_m,
                                   seg_row0, self.row_expert, self.q1, self.rec1, self.s1.data_ptr(), 1, self.device,
                                   shared=shared, shared_inter=self.Is, online_had=self.online_had,
                                   fuse_silu=self.fuse_silu)
        self.gg1, self.gg2 = self._core.gg1, self._core.gg2

    # buffers of the compute core, exposed for tests and benchmarks
    @property
    def o1(self):
        return self._core.o1

    @property
    def o2(self):
        return self._core.o2

    @property
    def o1s(self):
        return self._core.o1s

    @property
    def o2s(self):
        return self._core.o2s

    def route(self, topk_ids: torch.Tensor) -> None:
        T, k = topk_ids.shape
        assert T * k <= self.R and topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()
        a = _lib.RouteArgs()
        a.topk_ids, a.counts, a.row_start = topk_ids.data_ptr(), self.counts.data_ptr(), self.row_start.data_ptr()
        a.row_expert, a.row_token, a.slot_row = (self.row_expert.data_ptr(), self.row_token.data_ptr(),
                                                 self.slot_row.data_ptr())
        a.workspace, a.workspace_bytes = self.route_ws.data_ptr(), self.route_ws.numel() * 4
        a.num_tokens, a.topk, a.num_experts = T, k, self.E
        id_map = getattr(self, "id_map", None)          # expert-parallel front end: renumbering inside the routing kernels
        if id_map is not None:
            a.id_map, a.num_ids = id_map.data_ptr(), self.num_ids
            if self.rep_base is not None:
                a.rep_base, a.rep_count = self.rep_base.data_ptr(), self.rep_count.data_ptr()
        _lib.check(_lib.lib().mxmoe_route_topk(C.byref(a), current_stream_ptr()))

    def _row_args(self, rows: int, q_store: torch.Tensor, rec_stride: int, s_store: torch.Tensor | None,
                  rec_scale_off: int = -1) -> _lib.ActArgs:
        a = _lib.ActArgs()
        a.q_store = q_store.data_ptr()
        a.s_store = None if s_store is None else s_store.data_ptr()
        a.row_expert, a.row_token = self.row_expert.data_ptr(), self.row_token.data_ptr()
        a.exp_qtag = self.tag1.data_ptr()
        a.k, a.k_shared, a.rows_routed, a.rows_total, a.num_experts = self.H, self.H, rows, rows, self.E
        a.rec_stride, a.rec_scale_off = rec_stride, rec_scale_off
        return a

    def gather(self, t: _lib.TokenQuantArgs, rows: int, q_store: torch.Tensor, rec_stride: int,
               s_store: torch.Tensor | None, rec_scale_off: int = -1) -> None:
        a = self._row_args(rows, q_store, rec_stride, s_store, rec_scale_off)
        _lib.check(_lib.lib().mxmoe_gather_rows(C.byref(a), C.byref(t), current_stream_ptr()))

    def quant_scatter(self, hidden: torch.Tensor, rows: int) -> None:
        """Rotate + quantise every token once and write its row to each of its routed slots (one launch)."""
        t = self.tq.fill(hidden)
        a = self._row_args(rows, self.q1, self.rec1, self.s1)
        _lib.check(_lib.lib().mxmoe_quant_tokens_scatter(C.byref(t), C.byref(a), self.slot_row.data_ptr(), self.topk,
                                                         current_stream_ptr()))

    def forward(self, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor | None = None):
        """``[T, H]`` fp16 hidden states + ``[T, topk]`` int32 expert ids (+ fp32 gate weights) -> ``[T, H]`` fp16."""
        T = hidden.shape[0]
        assert T == self.T, "this layer instance was sized for a fixed token count"
        with torch.cuda.device(self.device):
            if self._core is None:
                self._build_core(hidden)
            if self.has_shared and self._tag1[self.E] == 0 and not self.rotate:
                assert hidden.data_ptr() == self._hidden_ptr, \
                    "an fp16 shared expert reads `hidden` in place: pass the same buffer every step"
            self.route(topk_ids)
            if self.one_pass_quant:
                self.quant_scatter(hidden, T * self.topk)
            else:
                t = self.tq.run(hidden)
                self.gather(t, T * self.topk, self.q1, self.rec1, self.s1)
            self._core.run(T * self.topk)
            out = self.out.view(self.T, self.H)
            _lib.check(_lib.lib().mxmoe_combine_topk(
                self._core.o2.data_ptr(), self.slot_row.data_ptr(),
                None if topk_weights is None else topk_weights.data_ptr(),
                self._core.o2s.data_ptr() if self.has_shared else None, out.data_ptr(), T, self.topk, self.H,
                current_stream_ptr()))
        return out

    def forward_graph(self, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor | None = None):
        """Same as :meth:`forward`, replayed from a CUDA graph.

        The step launches eight kernels (nine with a shared expert) and never returns to the host, so it is captured once per set
        of argument buffers (their addresses are baked into the graph: refill the same tensors for
        the next step) and replayed with a single launch.
        """
        key = (hidden.data_ptr(), topk_ids.data_ptr(), None if topk_weights is None else topk_weights.data_ptr())
        if getattr(self, "_graph_key", None) != key:
            with torch.cuda.device(self.device):
                self.forward(hidden, topk_ids, topk_weights)        # builds descriptors, warms up
                self.check()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.forward(hidden, topk_ids, topk_weights)
                self._graph, self._graph_key = g, key
        self._graph.replay()
        return self.out.view(self.T, self.H)

    # route (3 launches; 1 when all (token, slot) pairs fit one block of 1024), quant_tokens_scatter, GEMM, silu,
    # GEMM, combine (+1 launch with the two-pass quantiser)
    @property
    def launches_per_step(self) -> int:
        route = 1 if 0 < self.T * self.topk <= 1024 else 3
        return (route + (5 if self.one_pass_quant else 6) + (1 if self.has_shared else 0)   # + the shared expert's silu
                + (2 if self.online_had is not None else 0))                               # + rotation, quantiser

    def check(self) -> None:
        self._core.check()

    def gemm_bytes(self, counts: list[int]) -> int:
        """Algorithmic traffic of the two grouped GEMMs for given per-expert row counts (bytes)."""
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


class HostPipeline:
    """Serving loop over HOST buffers: the host->device copy of step i + 1, the layer pass of step i and the
    device->host copy of the result of step i - 1 run concurrently (copy-in stream, compute stream, copy-out
    stream, two sets of device buffers, events between them).  ``layer`` is a :class:`MoELayer` (replayed from
    its CUDA graph) or any object with ``forward(hidden, ids, weights) -> [T, H]``.

        pipe = HostPipeline(layer, T, H, topk)
        for hidden_host, ids_host, wts_host, out_host in batches:     # pinned host tensors
            pipe.submit(hidden_host, ids_host, wts_host, out_host)
        pipe.drain()                                                  # out_host of every submitted step is complete

    The host tensors of a step (int32 ids, fp32 weights, fp16 hidden states; contiguous, page-locked) must stay
    unchanged until the step has run: the routing tables are read from them by a kernel when the step's compute
    starts, the hidden states by the copy engine before that.
    """

    def __init__(self, layer, tokens: int, hidden: int, topk: int, device=None, use_graph: bool = True,
                 inputs=None):
        self.layer = layer
        self.device = torch.device(device) if device is not None else layer.device
        dev = self.device
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.bufs = [dict(hidden=torch.empty(tokens, hidden, dtype=torch.float16, device=dev),
                          out=torch.empty(tokens, hidden, dtype=torch.float16, device=dev),
                          ev_in=torch.cuda.Event(), ev_comp=torch.cuda.Event(), ev_out=torch.cuda.Event())
                     for _ in range(2)]
        # the layer's graph bakes in the addresses of its inputs: one static set, filled by device copies
        # (`inputs` = (hidden, ids, weights) device tensors the layer has already been run on: a layer with an fp16
        # shared expert and no rotation reads `hidden` in place and is bound to that address)
        if inputs is not None:
            self.x, self.i, self.w = inputs
        else:
            self.x = torch.empty(tokens, hidden, dtype=torch.float16, device=dev)
            self.i = torch.empty(tokens, topk, dtype=torch.int32, device=dev)
            self.w = torch.empty(tokens, topk, dtype=torch.float32, device=dev)
        self.use_graph = use_graph and hasattr(layer, "forward_graph")
        self.step = 0

    def submit(self, hidden_host, ids_host, wts_host, out_host) -> None:
        b = self.bufs[self.step & 1]
        comp = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.s_in):
            if self.step >= 2:
                self.s_in.wait_event(b["ev_comp"])          # step - 2 no longer reads this input set
            b["hidden"].copy_(hidden_host, non_blocking=True)
            b["ev_in"].record(self.s_in)
        comp.wait_event(b["ev_in"])
        if self.step >= 2:
            comp.wait_event(b["ev_out"])                    # step - 2's result has left this output buffer
        self.x.copy_(b["hidden"], non_blocking=True)
        # the routing tables (131 KB each) are read from the page-locked host tensors by a kernel on the compute
        # stream: as DMA copies behind the hidden states they cost the copy-in stream 0.11 ms per step (0.83 -> 0.72)
        assert ids_host.dtype == self.i.dtype and wts_host.dtype == self.w.dtype and ids_host.is_contiguous() \
            and wts_host.is_contiguous() and ids_host.numel() == self.i.numel() and wts_host.numel() == self.w.numel()
        stream = current_stream_ptr()
        lib = _lib.lib()
        _lib.check(lib.mxmoe_fetch_host(self.i.data_ptr(), ids_host.data_ptr(), ids_host.numel() * ids_host.element_size(), stream))
        _lib.check(lib.mxmoe_fetch_host(self.w.data_ptr(), wts_host.data_ptr(), wts_host.numel() * wts_host.element_size(), stream))
        fwd = self.layer.forward_graph if self.use_graph else self.layer.forward
        b["out"].copy_(fwd(self.x, self.i, self.w), non_blocking=True)
        b["ev_comp"].record(comp)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(b["ev_comp"])
            out_host.copy_(b["out"], non_blocking=True)
            b["ev_out"].record(self.s_out)
        self.step += 1

    def drain(self) -> None:
        """Block the host until every submitted step has finished: its result is in ``out_host`` on return."""
        comp = torch.cuda.current_stream(self.device)
        comp.wait_stream(self.s_in)
        comp.wait_stream(self.s_out)
        self.s_out.synchronize()
        comp.synchronize()
