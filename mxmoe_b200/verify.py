"""Self-check of a layer that has just run: its two grouped GEMMs against plain torch arithmetic on the
operands that are actually in the layer's device buffers.

For a handful of experts (by default the one with the most rows, a median one and the one with the fewest;
plus the shared expert) and for both linear blocks:

* w8a8 / w4a4: the problem is launched once more with raw-accumulator output and the int32 sums must equal
  the exact integer product of the codes found in the activation store and in the packed weight (computed
  as an fp64 matmul: every partial sum is an integer far below 2**53), bit for bit; the fp16 rows the layer
  produced must equal ``fp16(float(acc) * float(fp16(sa * sb)))`` (the reference's epilogue order,
  mm_tile.cuh:490-493) bit for bit;
* fp16 / w4a16 group-128: the fp16 rows against an fp64 product of the fp16 operands (weights dequantised
  as ``fp16(fma(q, s, z))``, quantize.cuh:189-190) in relative L2 norm.

This decodes the layouts the kernels read (record stores, expanded int4 rows, packed weights), so it also
catches a wrong row offset, a stale descriptor or a wrong scale pointer at full problem sizes.  Torch is the
only dependency; nothing here is used on the compute path.
"""
from __future__ import annotations

import torch

from . import gg
from .weights import unpack_along_k, unpack_along_n4

REL_L2_FP = 1e-3


def _rows_bytes(store: torch.Tensor, stride_elems: int, row0: int, m: int, nbytes: int) -> torch.Tensor:
    """``[m, nbytes]`` uint8 view of rows row0 .. row0+m of a record store (fp16 tensor, ``stride_elems`` per row)."""
    b = store.view(torch.uint8).reshape(-1)
    rows = b[row0 * stride_elems * 2: (row0 + m) * stride_elems * 2].reshape(m, stride_elems * 2)
    return rows[:, :nbytes]


def decode_rows(store: torch.Tensor, stride_elems: int, row0: int, m: int, k: int, tag: int) -> torch.Tensor:
    """Activation rows of format ``tag`` as logical values ``[m, k]``: fp16 (tag 0) or integer codes as fp64."""
    if tag == 0:
        return _rows_bytes(store, stride_elems, row0, m, 2 * k).contiguous().view(torch.float16).reshape(m, k)
    if tag == 1:        # int8, two codes per 16-bit word with the first k in the HIGH byte
        by = _rows_bytes(store, stride_elems, row0, m, k).contiguous().view(torch.int8).reshape(m, k // 2, 2)
        return by.flip(-1).reshape(m, k).double()
    if tag == 3:
        # int4 expanded: byte 16*q.  Every 16 bytes of the packed row (8 words of 4 codes, first k in the top nibble,
        # little-endian: byte 2w holds codes 4w+2, 4w+3 and byte 2w+1 codes 4w, 4w+1) became their 16 high nibbles
        # followed by their 16 low nibbles: stored index 16*h + 2*w + j holds code 4*w + 2*(1-j) + h.
        by = _rows_bytes(store, stride_elems, row0, m, k).contiguous().view(torch.int8)
        q = torch.div(by.to(torch.int32), 16, rounding_mode="floor").reshape(m, k // 32, 2, 8, 2)   # [.., h, w, j]
        return q.flip(-1).permute(0, 1, 3, 4, 2).reshape(m, k).double()                            # [.., w, 1-j, h]
    if tag == 2:        # int4 packed, four codes per 16-bit word
        w = _rows_bytes(store, stride_elems, row0, m, k // 2).contiguous().view(torch.int16).reshape(m, k // 4)
        return unpack_along_k(w, 4).double()
    raise ValueError(tag)


def decode_weight(w) -> tuple[torch.Tensor, torch.Tensor | None]:
    """``(values [N, K], per-channel scale or None)``: fp16 weights (dequantised for w4a16) or integer codes as fp64."""
    a_bits, w_bits, gsize, _sym = w.qparams
    if w_bits >= 16:
        return w.data.reshape(w.n, w.k), None
    if a_bits < 16:
        return unpack_along_k(w.data.reshape(w.n, -1), w_bits).double(), w.scale
    q = unpack_along_n4(w.data.reshape(w.n // 4, w.k)).to(torch.float16)
    gsize = w.k if gsize == -1 else gsize
    sz = w.scale.reshape(w.k // gsize, w.n, 2)
    s = sz[..., 0].t().repeat_interleave(gsize, dim=1)
    z = sz[..., 1].t().repeat_interleave(gsize, dim=1)
    # q*s + z is exact in fp64 (4-bit x 11-bit significand + an fp16): one rounding = the fused multiply-add
    return (q.double() * s.double() + z.double()).to(torch.float16), None


def _rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    den = ref.double().norm().item()
    return float((x.double() - ref.double()).norm().item() / den) if den > 0 else float(x.double().norm().item())


def _rerun(a_store, a_stride, a_scale, row0, m, k, tag, w, out_mode, dtype, dev):
    """The same problem once more on its own (operand pointers moved to the first row: C starts at row 0)."""
    c = torch.empty((m, w.n), dtype=dtype, device=dev)
    p = gg.Problem(A=a_store.data_ptr() + row0 * a_stride * 2, B=w.data, C=c, M=m, N=w.n, K=k, qparams=w.qparams,
                   scale_a=None if a_scale is None else a_scale.data_ptr() + row0 * 2, scale_b=w.scale,
                   out_mode=out_mode, lda_bytes=a_stride * 2, a_expanded=1 if tag == 3 else 0)
    g = gg.GroupedGemm([p], device=dev)
    g.run()
    g.check()
    return c


def _silu_rows(gate_up_rows: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` of fp16 rows [m, 2 I] by the stand-alone device kernel, as fp16 [m, I]."""
    import ctypes as C
    from . import _lib
    from .layer import _act_call
    m, n2 = gate_up_rows.shape
    dev = gate_up_rows.device
    h = torch.empty((m, n2 // 2), dtype=torch.float16, device=dev)
    zeros = torch.zeros(max(m, 2), dtype=torch.int32, device=dev)
    _act_call(_lib.lib().mxmoe_silu_mul_then_quant, inp=gate_up_rows.contiguous(), in_shared=None, q_store=h, s_store=h,
              row_expert=zeros, row_token=None, exp_qtag=zeros, exp_row_start=None, exp_q_off=None, exp_s_off=None,
              signs=None, k=n2 // 2, k_shared=n2 // 2, rows_routed=m, rows_total=m, num_experts=1, rotate=0,
              rec_stride=n2 // 2, rec_scale_off=-1)
    return h


def check_problem(a_store, a_stride, a_scale, row0, m, k, tag, w, out_rows: torch.Tensor | None,
                  silu_rows: torch.Tensor | None = None) -> dict:
    """One (expert, block) problem: ``out_rows`` = the fp16 [m, N] rows the layer produced for it.  A layer that
    applies silu(gate) * up in the GEMM's epilogue has no such rows: pass ``silu_rows`` = its fp16 [m, N/2] rows
    instead; the scaled results are then produced by a launch of the same problem on its own, and the layer's rows
    must equal, bit for bit, what the stand-alone silu-mul kernel makes of them."""
    a = decode_rows(a_store, a_stride, row0, m, k, tag)
    b, sb = decode_weight(w)
    res = {"rows": int(m), "scheme": w.scheme}
    if out_rows is None:
        out_rows = _rerun(a_store, a_stride, a_scale, row0, m, k, tag, w, gg.OUT_FP16, torch.float16, silu_rows.device)
        res["silu_mismatch"] = int((_silu_rows(out_rows).view(torch.int16) != silu_rows.view(torch.int16)).sum().item())
    if tag == 0:
        ref = (a.double() @ b.double().t())
        res["rel_l2"] = _rel_l2(out_rows, ref)
        res["ok"] = res["rel_l2"] <= REL_L2_FP and res.get("silu_mismatch", 0) == 0
        return res
    acc = (a @ b.t())                                             # exact integers in fp64
    dev = out_rows.device
    # the same problem once more with raw accumulators
    c_acc = _rerun(a_store, a_stride, a_scale, row0, m, k, tag, w, gg.OUT_ACC, torch.int32, dev)
    res["acc_mismatch"] = int((c_acc.double() != acc).sum().item())
    sa = a_scale[row0: row0 + m].float().reshape(m, 1)
    prod = (sa * sb.float().reshape(1, -1)).half().float()        # exact product, one rounding to fp16
    ref16 = (acc.float() * prod).half()
    res["out_mismatch"] = int((out_rows.view(torch.int16) != ref16.view(torch.int16)).sum().item())
    res["ok"] = res["acc_mismatch"] == 0 and res["out_mismatch"] == 0 and res.get("silu_mismatch", 0) == 0
    return res


def pick_experts(counts: list[int]) -> list[int]:
    """The expert with the most rows, a median one and the one with the fewest (non-empty)."""
    live = sorted((c, e) for e, c in enumerate(counts) if c > 0)
    if not live:
        return []
    picks = [live[-1][1], live[len(live) // 2][1], live[0][1]]
    return list(dict.fromkeys(picks))


def check_layer(layer, experts: list[int] | None = None, include_shared: bool = True) -> dict:
    """Check a :class:`mxmoe_b200.layer.MoELayer` whose ``forward`` has just run (its buffers still hold the step).

    Returns ``{"ok": bool, "problems": [...]}`` with one entry per checked (expert, block)."""
    torch.cuda.synchronize(layer.device)
    core = layer._core
    counts = layer.counts.cpu().tolist()
    starts = layer.row_start.cpu().tolist()
    experts = pick_experts(counts) if experts is None else experts
    out = []
    H, I = layer.H, layer.I
    o1 = core.o1.view(-1, 2 * I)
    o2 = core.o2.view(-1, H)
    fused = getattr(core, "fused_silu", False)
    for e in experts:
        m, r0 = counts[e], starts[e]
        if m == 0:
            continue
        r = check_problem(layer.q1, layer.rec1, layer.s1, r0, m, H, layer._tag1[e], layer.gate_up[e],
                          None if fused else o1[r0:r0 + m], silu_rows=core.h16[r0:r0 + m] if fused else None)
        r.update(expert=e, block="gate_up")
        out.append(r)
        r = check_problem(core.q2, core.rec2, core.s2, r0, m, I, core._tag2[e], layer.down[e], o2[r0:r0 + m])
        r.update(expert=e, block="down")
        out.append(r)
    if include_shared and layer.has_shared:
        E, T, Is = layer.E, layer.T, layer.Is
        tag = layer._tag1[E]
        if tag == 0:
            store = layer.tq.f16 if layer.tq.f16 is not None else None
            scale = None
        elif tag == 1:
            store, scale = layer.tq.q8, layer.tq.s8
        else:
            store, scale = layer.tq.q4x, layer.tq.s4
        if store is not None:      # an fp16 shared expert without rotation reads the caller's hidden states in place
            r = check_problem(store, H // (1, 2, 4, 2)[tag], scale, 0, T, H, tag, layer.gate_up[E],
                              core.o1s.view(T, 2 * Is))
            r.update(expert=E, block="gate_up(shared)")
            out.append(r)
        tag2 = core._tag2[E]
        r = check_problem(core.q2s, core.rec2s, core.s2s, 0, T, Is, tag2, layer.down[E], core.o2s.view(T, H))
        r.update(expert=E, block="down(shared)")
        out.append(r)
    return {"ok": all(p["ok"] for p in out) and len(out) > 0, "problems": out}
