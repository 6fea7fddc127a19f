"""Python operator API: the functions of the reference's pybind module ``mxmoe_ops``
(``mxmoe/kernels/src/ref_bind.cu:759-768``) with the same names, argument order,
return tuples and error behaviour (``TORCH_CHECK`` -> Python exception), running
on the sm_100a kernels of ``libmxmoe_b200.so``.

    import mxmoe_b200.ops as mxmoe_ops

Tensors holding packed operands are opaque 2-byte buffers exactly as in the
reference (it reinterprets ``data_ptr()`` as ``at::Half*``); fp16 and int16
tensors are both accepted.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib
from .gg import Problem, GroupedGemm, current_stream_ptr

QParamsTuple = tuple  # (a_bits, w_bits, gsize, sym), the element type of the reference's qparams_per_exp


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _qtag(qbits: int, gsize: int) -> int:
    """Activation storage tag (ref_bind.cu:461-473)."""
    if qbits >= 16:
        return 0
    if qbits == 8 and gsize == -1:
        return 1
    if qbits == 4 and gsize == -1:
        return 2
    if qbits == 4 and gsize == 128:
        return 3
    return -1


def _act_tag(qp: QParamsTuple) -> int:
    return _qtag(int(qp[0]), int(qp[2]) if int(qp[0]) < 16 else -1)


# ---------------------------------------------------------------------------
# grouped GEMM
# ---------------------------------------------------------------------------
def gg_mxmoe_share_fused(inp: Sequence[torch.Tensor], experts: Sequence[torch.Tensor],
                         scale_zp_a: Sequence[torch.Tensor], scale_zp_b: Sequence[torch.Tensor],
                         output: list, N: int, K: int, shared_N: int, shared_K: int,
                         qparams_per_exp: Sequence[QParamsTuple], recv_tokens_per_exp: torch.Tensor,
                         verbose: bool = False) -> list:
    """Mixed-precision grouped GEMM over the non-empty experts (+ the shared expert last).

    Mirrors ``moe_mxmoe_share_fused`` (ref_bind.cu:312-431): ``inp`` / ``scale_zp_a``
    / ``output`` are indexed by problem (non-empty experts in order, shared expert
    last), ``experts`` / ``scale_zp_b`` / ``qparams_per_exp`` by expert id.  Unlike
    the reference, which is hard-wired to one generated w4a16+w8a8 kernel
    (ref_bind.cu:412), every supported scheme may appear.
    """
    E = int(recv_tokens_per_exp.size(0))
    num_problems = len(inp)
    _check(num_problems > 0, "inp must not be empty")
    num_tokens = int(inp[-1].size(0))
    has_shared = len(experts) > E
    tokens = recv_tokens_per_exp.tolist()
    problems = []
    pidx = 0
    for e in range(E + (1 if has_shared else 0)):
        m = num_tokens if e == E else int(tokens[e])
        if m == 0:
            continue
        _check(pidx < num_problems, "fewer inputs than non-empty experts")
        a_bits, w_bits, gsize, sym = qparams_per_exp[e]
        n_, k_ = (shared_N, shared_K) if e == E else (N, K)
        sa = scale_zp_a[pidx] if pidx < len(scale_zp_a) else None
        sb = scale_zp_b[e] if e < len(scale_zp_b) else None
        problems.append(Problem(
            A=inp[pidx], B=experts[e], C=output[pidx], M=m, N=n_, K=k_,
            qparams=(int(a_bits), int(w_bits), int(gsize), bool(sym)),
            scale_a=sa if (sa is not None and sa.numel() > 0) else None,
            scale_b=sb if (sb is not None and sb.numel() > 0) else None))
        if verbose:
            print(f"problem {pidx}: [{m},{n_},{k_}] qparams: [{a_bits} {w_bits}] {gsize} {sym}")
        pidx += 1
    _check(pidx == num_problems, f"{num_problems} inputs for {pidx} non-empty experts")
    g = GroupedGemm(problems, device=inp[0].device)
    g.run()
    g.check()
    return output


def gg_cutlass(inp: torch.Tensor, experts: torch.Tensor, topk_ids: torch.Tensor, output: torch.Tensor,
               num_problems_=None, inp_buffer_=None, perm_indices_=None, recv_tokens_per_exp_=None) -> torch.Tensor:
    """fp16 grouped GEMM with the signature of ``moe_cutlass`` (ref_bind.cu:68-182).

    The reference runs CUTLASS ``GemmGrouped`` here; this build runs the fp16
    scheme of the same persistent kernel.  ``output`` is ``[num_tokens*topk, N]``.
    """
    _check(inp.dim() == 2, "hidden must be 2D")
    _check(inp.is_cuda and experts.is_cuda, "dev must be on cuda")
    E, N, K = experts.shape
    topk = topk_ids.size(1)
    if perm_indices_ is not None:
        inp_buffer, recv = inp_buffer_, recv_tokens_per_exp_
    else:
        values_sorted, indices = torch.sort(topk_ids.reshape(-1), stable=True)
        indices = indices.floor_divide(topk)
        inp_buffer = inp.index_select(0, indices)
        recv = torch.bincount(values_sorted, minlength=E).cpu()
    problems, st = [], 0
    for e, m in enumerate(recv.tolist()):
        if m == 0:
            continue
        problems.append(Problem(A=inp_buffer[st:st + m], B=experts[e], C=output[st:st + m], M=m, N=N, K=K,
                                qparams=(16, 16, -1, True)))
        st += m
    g = GroupedGemm(problems, device=inp.device)
    g.run()
    g.check()
    return output


def gg_cutlass_share_fused(inp, experts, shared_experts, topk_ids, output, shared_output,
                           num_problems_=None, inp_buffer_=None, perm_indices_=None, recv_tokens_per_exp_=None):
    """``moe_cutlass_share_fused`` (ref_bind.cu:184-310): routed experts plus the shared expert in one launch."""
    _check(inp.dim() == 2, "hidden must be 2D")
    _check(inp.is_cuda and experts.is_cuda, "dev must be on cuda")
    E, N, K = experts.shape
    topk = topk_ids.size(1)
    if perm_indices_ is not None:
        inp_buffer, recv = inp_buffer_, recv_tokens_per_exp_
    else:
        values_sorted, indices = torch.sort(topk_ids.reshape(-1), stable=True)
        indices = indices.floor_divide(topk)
        inp_buffer = inp.index_select(0, indices)
        recv = torch.bincount(values_sorted, minlength=E).cpu()
    problems, st = [], 0
    for e, m in enumerate(recv.tolist()):
        if m == 0:
            continue
        problems.append(Problem(A=inp_buffer[st:st + m], B=experts[e], C=output[st:st + m], M=m, N=N, K=K,
                                qparams=(16, 16, -1, True)))
        st += m
    problems.append(Problem(A=inp, B=shared_experts, C=shared_output, M=inp.size(0), N=shared_experts.size(0),
                            K=shared_experts.size(1), qparams=(16, 16, -1, True)))
    g = GroupedGemm(problems, device=inp.device)
    g.run()
    g.check()
    return output, shared_output


# ---------------------------------------------------------------------------
# activation prologues
# ---------------------------------------------------------------------------
def _expert_tables(tokens_per_exp, num_tokens, num_experts, has_shared, qparams_per_exp, row_len, row_len_shared):
    """Host tables of ref_bind.cu:475-505 / :636-668: tag, first row, write offsets (fp16 elements)."""
    n_all = num_experts + (1 if has_shared else 0)
    tag, st, qoff, soff, qsize, ssize = [], [], [], [], [], []
    acc = q = s = 0
    for e in range(n_all):
        t = _act_tag(qparams_per_exp[e])
        _check(t in (0, 1, 2), f"activation scheme of expert {e} is not supported (a_bits={qparams_per_exp[e][0]}, "
                               f"gsize={qparams_per_exp[e][2]})")
        ld_in = row_len_shared if e == num_experts else row_len
        q_ld = ld_in if t == 0 else (ld_in // 2 if t == 1 else ld_in // 4)
        s_ld = 0 if t == 0 else 1
        m = num_tokens if e == num_experts else int(tokens_per_exp[e])
        tag.append(t); st.append(acc); qoff.append(q); soff.append(s)
        qsize.append(q_ld * m); ssize.append(s_ld * m)
        q += q_ld * m
        s += s_ld * m
        acc += m
    return tag, st, qoff, soff, qsize, ssize, q, s


def _launch_act(fn, dev, **kw) -> None:
    a = _lib.ActArgs()
    for k, v in kw.items():
        setattr(a, k, v.data_ptr() if isinstance(v, torch.Tensor) else v)
    with torch.cuda.device(dev):
        _lib.check(fn(C.byref(a), current_stream_ptr()))


def quant_inp_act(hidden: torch.Tensor, topk_ids: torch.Tensor, num_experts: int, N: int, num_shared_experts: int,
                  qparams_per_exp: Sequence[QParamsTuple], verbose: bool = False, *,
                  rotate: bool = False, signs: torch.Tensor | None = None, fused: bool | str = False):
    """Permute tokens by expert and quantise + pack each row with its expert's activation scheme.

    Mirrors ``quant_inp_act`` (ref_bind.cu:434-592) including the nine-element return tuple
    ``(inp_list, inp_scale_list, out_list, inp_store, inp_scale_store, out_store,
    recv_tokens_per_exp[CPU int64], perm_indices, dst_exp_sorted)``.  ``rotate`` / ``signs``
    (keyword-only, not in the reference) apply the Hadamard rotation of the hidden
    dimension before quantising.  By default rows are quantised once per token and then
    copied to their experts; ``fused=True`` runs the single gather+quantise kernel instead and
    ``fused="scatter"`` (top-k up to 8) the once-per-token kernel that writes the routed rows itself
    (same bits all three).
    """
    _check(hidden.dim() == 2 and hidden.is_cuda, "hidden must be a 2D cuda tensor")
    _check(hidden.dtype == torch.float16, "hidden must be fp16")
    _check(topk_ids.dtype == torch.int32, "topk_ids must be int32")
    num_tokens, K = hidden.shape
    topk = topk_ids.size(1)
    has_shared = num_shared_experts > 0
    dev = hidden.device
    hidden = hidden.contiguous()

    dst_exp_sorted, perm_slots = torch.sort(topk_ids.reshape(-1), stable=True)
    perm_indices = perm_slots.floor_divide(topk)
    recv_tokens_per_exp = torch.bincount(dst_exp_sorted, minlength=num_experts).cpu()
    tokens = recv_tokens_per_exp.tolist()

    tag, st, qoff, soff, qsize, ssize, q_total, s_total = _expert_tables(
        tokens, num_tokens, num_experts, has_shared, qparams_per_exp, K, K)
    n_all = num_experts + (1 if has_shared else 0)
    tables = torch.tensor([tag, st, qoff, soff], dtype=torch.int32).to(dev)

    alloc_tokens = num_tokens * topk + (num_tokens if has_shared else 0)
    inp_store = torch.empty(q_total, dtype=torch.float16, device=dev)
    inp_scale_store = torch.empty(s_total, dtype=torch.float16, device=dev)
    out_store = torch.empty((num_shared_experts + topk) * num_tokens * N * 2, dtype=torch.float16, device=dev)
    if signs is not None:
        signs = signs.to(device=dev, dtype=torch.int8).contiguous()

    common = dict(q_store=inp_store, s_store=inp_scale_store if s_total else None,
                  row_expert=dst_exp_sorted, row_token=perm_indices,
                  exp_qtag=tables[0], exp_row_start=tables[1], exp_q_off=tables[2], exp_s_off=tables[3],
                  k=K, k_shared=K, rows_routed=num_tokens * topk, rows_total=alloc_tokens, num_experts=num_experts)
    if fused == "scatter":
        # one pass per TOKEN: the routed rows are written from registers; the shared expert's rows map one-to-one
        # onto tokens, so its slice of the stores IS the token-major store of its format
        slot_row = torch.empty(num_tokens * topk, dtype=torch.int32, device=dev)
        slot_row[perm_slots] = torch.arange(num_tokens * topk, dtype=torch.int32, device=dev)
        t = _lib.TokenQuantArgs()
        t.inp, t.k, t.num_tokens, t.rotate = hidden.data_ptr(), K, num_tokens, 1 if rotate else 0
        t.signs = None if signs is None else signs.data_ptr()
        if has_shared:
            q_ptr = inp_store.data_ptr() + 2 * qoff[num_experts]
            s_ptr = inp_scale_store.data_ptr() + 2 * soff[num_experts] if s_total else None
            if tag[num_experts] == 0:
                t.f16 = q_ptr
            elif tag[num_experts] == 1:
                t.q8, t.s8 = q_ptr, s_ptr
            else:
                t.q4, t.s4 = q_ptr, s_ptr
        a = _lib.ActArgs()
        for k_, v in dict(common, rows_total=num_tokens * topk).items():
            setattr(a, k_, v.data_ptr() if isinstance(v, torch.Tensor) else v)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().mxmoe_quant_tokens_scatter(C.byref(t), C.byref(a), slot_row.data_ptr(), topk,
                                                             current_stream_ptr()))
        slot_row.record_stream(torch.cuda.current_stream())
    elif fused:
        _launch_act(_lib.lib().mxmoe_quant_act, dev, inp=hidden, in_shared=None, signs=signs,
                    rotate=1 if rotate else 0, **common)
    else:
        used = {tag[e] for e in range(n_all) if (num_tokens if e == num_experts else tokens[e]) > 0}
        t = _lib.TokenQuantArgs()
        keep = []

        def store(n):
            buf = torch.empty(n, dtype=torch.float16, device=dev)
            keep.append(buf)
            return buf.data_ptr()
        t.inp, t.k, t.num_tokens, t.rotate = hidden.data_ptr(), K, num_tokens, 1 if rotate else 0
        t.signs = None if signs is None else signs.data_ptr()
        if 0 in used and rotate:
            t.f16 = store(num_tokens * K)
        if 1 in used:
            t.q8, t.s8 = store(num_tokens * K // 2), store(num_tokens)
        if 2 in used:
            t.q4, t.s4 = store(num_tokens * K // 4), store(num_tokens)
        a = _lib.ActArgs()
        for k_, v in common.items():
            setattr(a, k_, v.data_ptr() if isinstance(v, torch.Tensor) else v)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().mxmoe_quant_tokens(C.byref(t), current_stream_ptr()))
            _lib.check(_lib.lib().mxmoe_gather_rows(C.byref(a), C.byref(t), current_stream_ptr()))
        # the token-major stores may be recycled by the allocator once the stream has consumed them
        for buf in keep:
            buf.record_stream(torch.cuda.current_stream())

    inp_list, inp_scale_list, out_list = [], [], []
    qout_off = 0
    for e in range(n_all):
        m = num_tokens if e == num_experts else tokens[e]
        if m == 0:
            continue
        out_ld = N * 2 * num_shared_experts if e == num_experts else N * 2
        pack = 1 if tag[e] == 0 else (2 if tag[e] == 1 else 4)
        if verbose:
            print(f"exp: {e} qinp_size: {qsize[e]} qinp_scale_size: {ssize[e]} qinp: [{m}, {K // pack}]")
        inp_list.append(inp_store[qoff[e]:qoff[e] + qsize[e]].view(m, K // pack))
        if s_total > 0:
            inp_scale_list.append(inp_scale_store[soff[e]:soff[e] + ssize[e]])
        else:
            inp_scale_list.append(torch.empty(0, dtype=torch.float16, device=dev))
        out_list.append(out_store[qout_off:qout_off + m * out_ld].view(m, out_ld))
        qout_off += m * out_ld
    return (inp_list, inp_scale_list, out_list, inp_store, inp_scale_store, out_store,
            recv_tokens_per_exp, perm_indices, dst_exp_sorted)


def silu_mul_then_quant(inp: torch.Tensor, num_problems: int, num_experts: int, K: int, N: int,
                        num_shared_experts: int, num_tokens: int, topk: int, values_sorted: torch.Tensor,
                        recv_tokens_per_exp: torch.Tensor, qparams_per_exp: Sequence[QParamsTuple]):
    """``h = silu(gate) * up`` on the gate_up output, then quantise + pack for the down projection.

    Mirrors ``silu_mul_then_quant`` (ref_bind.cu:595-757): ``inp`` is the flat gate_up
    ``out_store`` (routed rows ``[T*topk, 2N]`` then shared rows ``[T, 2N*ns]``), ``K`` is the
    hidden size (output width of the down projection), ``N`` the expert intermediate size.
    Returns ``(inp_list, inp_scale_list, out_list, inp_store, inp_scale_store, out_store)``.
    """
    _check(inp.is_cuda and inp.dtype == torch.float16, "inp must be an fp16 cuda tensor")
    has_shared = num_shared_experts > 0
    dev = inp.device
    tokens = recv_tokens_per_exp.tolist()
    n_shared = N * num_shared_experts
    tag, st, qoff, soff, qsize, ssize, q_total, s_total = _expert_tables(
        tokens, num_tokens, num_experts, has_shared, qparams_per_exp, N, n_shared)
    n_all = num_experts + (1 if has_shared else 0)
    tables = torch.tensor([tag, st, qoff, soff], dtype=torch.int32).to(dev)
    rows_routed = num_tokens * topk
    alloc_tokens = rows_routed + (num_tokens if has_shared else 0)

    inp_store = torch.empty(q_total, dtype=torch.float16, device=dev)
    inp_scale_store = torch.empty(s_total, dtype=torch.float16, device=dev)
    out_store = torch.empty((1 + topk) * num_tokens * K, dtype=torch.float16, device=dev)
    flat = inp.reshape(-1)
    shared_in = flat[rows_routed * N * 2:] if has_shared else None

    _launch_act(_lib.lib().mxmoe_silu_mul_then_quant, dev,
                inp=flat, in_shared=shared_in, q_store=inp_store, s_store=inp_scale_store if s_total else None,
                row_expert=values_sorted, row_token=None,
                exp_qtag=tables[0], exp_row_start=tables[1], exp_q_off=tables[2], exp_s_off=tables[3],
                signs=None, k=N, k_shared=n_shared if has_shared else N, rows_routed=rows_routed,
                rows_total=alloc_tokens, num_experts=num_experts, rotate=0)

    inp_list, inp_scale_list, out_list = [], [], []
    qout_off = 0
    for e in range(n_all):
        m = num_tokens if e == num_experts else tokens[e]
        if m == 0:
            continue
        ld = n_shared if e == num_experts else N
        pack = 1 if tag[e] == 0 else (2 if tag[e] == 1 else 4)
        inp_list.append(inp_store[qoff[e]:qoff[e] + qsize[e]].view(m, ld // pack))
        if s_total > 0:
            inp_scale_list.append(inp_scale_store[soff[e]:soff[e] + ssize[e]])
        else:
            inp_scale_list.append(torch.empty(0, dtype=torch.float16, device=dev))
        out_list.append(out_store[qout_off:qout_off + m * K].view(m, K))
        qout_off += m * K
    return inp_list, inp_scale_list, out_list, inp_store, inp_scale_store, out_store


def gate_topk(router_logits: torch.Tensor, topk: int, renormalize: bool = True):
    """Router gate on the device (no counterpart in ``mxmoe_ops``, which receives the routing result from the
    framework, ref_bind.cu:47-64): ``softmax(router_logits, dim=-1, dtype=float)`` -> top-k -> optional
    renormalisation.  ``router_logits``: fp32 or fp16 ``[T, E]``.  Returns ``(topk_ids int32 [T, k],
    topk_weights fp32 [T, k])``, ready for the routing and combine kernels."""
    _check(router_logits.is_cuda and router_logits.dim() == 2, "router_logits must be a CUDA [T, E] tensor")
    _check(router_logits.dtype in (torch.float32, torch.float16), "router_logits must be fp32 or fp16")
    logits = router_logits.contiguous()
    T, E = logits.shape
    ids = torch.empty((T, topk), dtype=torch.int32, device=logits.device)
    wts = torch.empty((T, topk), dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().mxmoe_gate_topk(logits.data_ptr(), 1 if logits.dtype == torch.float16 else 0, T, E, topk,
                                              1 if renormalize else 0, ids.data_ptr(), wts.data_ptr(),
                                              current_stream_ptr()))
    return ids, wts
