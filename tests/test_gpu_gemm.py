"""Parity of the sm_100a grouped GEMM against the CPU oracle, through the C ABI.

Integer schemes (w8a8, w4a4): int32 accumulators and the scaled fp16 output are
compared bit for bit.  Floating-point schemes (fp16, w4a16 group-128):
rel-L2 <= 1e-3 against the oracle (fp64 accumulation rounded once), the bound the
specification states for fp16 outputs.
"""
import numpy as np
import pytest
import torch

from oracle import gemm as og
from mxmoe_b200 import gg
from mxmoe_b200._lib import MxMoEError
from tests import util

pytestmark = pytest.mark.gpu

REL_L2 = 1e-3


@pytest.fixture(autouse=True, params=["swap", "swap-small", "swap2", "pair", "single"])
def gg_kernel(request, monkeypatch):
    """Every test of this file runs once per kernel: swapped operands (128 channels x up to 176 tokens, 4-bit
    weights through tensor memory; "swap-small" forces its geometry for few rows - 32-token tiles, ring of 10 stages -
    on every shape), CTA pairs (256 x 256 tiles, cta_group::2) and single CTAs (128 x 256 tiles)."""
    kernel = request.param.split("-")[0]
    monkeypatch.setenv("MXMOE_GG_KERNEL", kernel)
    if request.param == "swap-small":
        monkeypatch.setenv("MXMOE_GG_TILES", "small")
    else:
        monkeypatch.delenv("MXMOE_GG_TILES", raising=False)
    yield kernel

# (M, N, K): one tile / one k-block; ragged M; ragged N tile; several k-blocks; layer shapes
SHAPES_INT = [(128, 256, 128), (1, 256, 128), (17, 256, 256), (129, 512, 384), (300, 2816, 2048), (77, 2048, 1408),
              (256, 264, 128)]
SHAPES_FP = [(128, 256, 64), (1, 256, 128), (17, 256, 128), (129, 512, 384), (300, 2816, 2048), (77, 2048, 1408),
             (64, 264, 64)]
SHAPES_W4A16 = [(128, 256, 128), (1, 256, 128), (17, 288, 256), (129, 512, 384), (300, 2816, 2048), (77, 2048, 1408)]


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("shape", SHAPES_INT)
def test_int_accumulators_bit_exact(cuda_device, bits, shape):
    rng = np.random.default_rng(hash((bits,) + shape) % 2**32)
    c = util.WxAxCase(rng, *shape, bits)
    util.run([c.problem(cuda_device, gg.OUT_ACC)])
    got = c.C.cpu().numpy()
    assert np.array_equal(got, c.acc), f"{np.count_nonzero(got != c.acc)} of {got.size} accumulators differ"


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("shape", SHAPES_INT)
def test_int_scaled_output_bit_exact(cuda_device, bits, shape):
    rng = np.random.default_rng(hash((bits, 1) + shape) % 2**32)
    c = util.WxAxCase(rng, *shape, bits)
    util.run([c.problem(cuda_device)])
    got = c.C.cpu().numpy()
    assert np.array_equal(got.view(np.uint16), c.ref.view(np.uint16)), \
        f"{np.count_nonzero(got.view(np.uint16) != c.ref.view(np.uint16))} of {got.size} outputs differ"


@pytest.mark.parametrize("shape", SHAPES_INT)
def test_w4a4_expanded_activations_bit_exact(cuda_device, shape):
    """Activations stored as one byte 16*q per code (what the layer's own prologue writes): accumulators
    and scaled output are the same bits as with packed activations."""
    rng = np.random.default_rng(hash((44,) + shape) % 2**32)
    c = util.WxAxCase(rng, *shape, 4, expanded=True)
    util.run([c.problem(cuda_device, gg.OUT_ACC)])
    assert np.array_equal(c.C.cpu().numpy(), c.acc)
    util.run([c.problem(cuda_device)])
    assert np.array_equal(c.C.cpu().numpy().view(np.uint16), c.ref.view(np.uint16))


def test_int_extreme_codes(cuda_device):
    """All codes at +-max: the largest accumulator magnitude the scheme can produce."""
    for bits, k in ((8, 2048), (4, 14336)):
        hi = 2 ** (bits - 1) - 1
        rng = np.random.default_rng(bits)
        c = util.WxAxCase(rng, 130, 256, k, bits)
        c.qa[:] = hi
        c.qb[:] = -hi
        c.qb[::2] = hi
        c.acc = og.int_accumulate(c.qa, c.qb)
        util.run([c.problem(cuda_device, gg.OUT_ACC)])
        assert np.array_equal(c.C.cpu().numpy(), c.acc)


@pytest.mark.parametrize("shape", SHAPES_FP)
def test_fp16(cuda_device, shape):
    rng = np.random.default_rng(hash(shape) % 2**32)
    c = util.Fp16Case(rng, *shape)
    util.run([c.problem(cuda_device)])
    err = og.rel_l2(c.C.cpu().numpy(), c.ref)
    assert err <= REL_L2, err


@pytest.mark.parametrize("shape", SHAPES_W4A16)
def test_w4a16_g128(cuda_device, shape):
    rng = np.random.default_rng(hash(shape) % 2**32)
    c = util.W4A16Case(rng, *shape)
    util.run([c.problem(cuda_device)])
    err = og.rel_l2(c.C.cpu().numpy(), c.ref)
    assert err <= REL_L2, err
    # fp32 accumulators of the same problem
    util.run([c.problem(cuda_device, gg.OUT_ACC)])
    ref32 = c.a.astype(np.float64) @ c.w.astype(np.float64).T
    assert og.rel_l2(c.C.cpu().numpy(), ref32) <= 1e-4


def test_mixed_schemes_one_launch(cuda_device):
    """Four schemes, ragged and empty problems, in one grouped launch."""
    rng = np.random.default_rng(7)
    cases = [util.WxAxCase(rng, 200, 512, 256, 4), util.Fp16Case(rng, 33, 256, 192),
             util.W4A16Case(rng, 140, 512, 256), util.WxAxCase(rng, 1, 256, 384, 8),
             util.WxAxCase(rng, 257, 768, 128, 8), util.W4A16Case(rng, 5, 256, 128),
             util.Fp16Case(rng, 129, 520, 64), util.WxAxCase(rng, 64, 256, 2048, 4)]
    probs = [c.problem(cuda_device) for c in cases]
    # an expert without tokens is dropped by the launcher (ref_bind.cu:345)
    empty = util.Fp16Case(rng, 1, 256, 64).problem(cuda_device)
    empty.M = 0
    g = util.run(probs[:3] + [empty] + probs[3:])
    assert g.kept == len(cases)
    for c in cases:
        got = c.C.cpu().numpy()
        if isinstance(c, util.WxAxCase):
            assert np.array_equal(got.view(np.uint16), c.ref.view(np.uint16))
        else:
            assert og.rel_l2(got, c.ref) <= REL_L2


@pytest.mark.parametrize("num_ctas", [1, 2, 3, 7, -2, -4, -6])
def test_few_ctas_walk_many_tiles_of_alternating_schemes(cuda_device, num_ctas):
    """With a handful of CTAs every CTA processes a long sequence of tiles whose schemes alternate
    (direct / converted, int / float): ring positions, barrier parities and TMEM buffers must stay
    consistent across every kind of transition.  Negative counts select the CTA-pair kernel."""
    rng = np.random.default_rng(100 + num_ctas)
    cases = [util.WxAxCase(rng, 300, 512, 384, 8), util.WxAxCase(rng, 200, 768, 256, 4),
             util.Fp16Case(rng, 140, 512, 192), util.WxAxCase(rng, 129, 256, 640, 8),
             util.W4A16Case(rng, 260, 512, 256), util.WxAxCase(rng, 64, 1024, 128, 4),
             util.WxAxCase(rng, 257, 512, 512, 8), util.W4A16Case(rng, 30, 768, 128),
             util.Fp16Case(rng, 200, 264, 64), util.WxAxCase(rng, 500, 256, 1408, 4),
             util.WxAxCase(rng, 333, 512, 256, 4, expanded=True), util.WxAxCase(rng, 70, 768, 384, 4, expanded=True)]
    util.run([c.problem(cuda_device) for c in cases], num_ctas=num_ctas)
    for i, c in enumerate(cases):
        got = c.C.cpu().numpy()
        if isinstance(c, util.WxAxCase):
            assert np.array_equal(got.view(np.uint16), c.ref.view(np.uint16)), f"problem {i}"
        else:
            assert og.rel_l2(got, c.ref) <= REL_L2, f"problem {i}"


def test_direct_only_launch_uses_no_converter(cuda_device):
    rng = np.random.default_rng(11)
    cases = [util.WxAxCase(rng, 150, 512, 512, 8), util.Fp16Case(rng, 150, 512, 512)]
    g = util.run([c.problem(cuda_device) for c in cases])
    assert g._plan.needs_cvt == 0
    assert np.array_equal(cases[0].C.cpu().numpy().view(np.uint16), cases[0].ref.view(np.uint16))
    assert og.rel_l2(cases[1].C.cpu().numpy(), cases[1].ref) <= REL_L2


def test_device_side_rows_and_offsets(cuda_device):
    """Several experts share one activation buffer; row counts and offsets live in device memory."""
    rng = np.random.default_rng(5)
    counts = [130, 0, 1, 300]
    k, n, bits = 256, 512, 8
    total = sum(counts)
    qa = util.rand_codes(rng, total, k, bits)
    sa = util.rand_scales(rng, total, 0.01, 0.5)
    from oracle import pack as op
    A = util.t16(op.pack_k(qa, bits), cuda_device)
    SA = util.t16(sa, cuda_device)
    Cbuf = torch.full((total, n), float("nan"), dtype=torch.float16, device=cuda_device)
    cnt = torch.tensor(counts, dtype=torch.int32, device=cuda_device)
    starts = torch.tensor(np.concatenate(([0], np.cumsum(counts)[:-1])), dtype=torch.int32, device=cuda_device)
    probs, refs, keep = [], [], []
    for e, m in enumerate(counts):
        qb = util.rand_codes(rng, n, k, bits)
        sb = util.rand_scales(rng, n)
        B, SB = util.t16(op.pack_k(qb, bits), cuda_device), util.t16(sb, cuda_device)
        keep += [B, SB]
        r0 = int(starts[e])
        refs.append(og.wxax_epilogue(og.int_accumulate(qa[r0:r0 + m], qb), sa[r0:r0 + m], sb))
        probs.append(gg.Problem(A=A, B=B, C=Cbuf, M=total, N=n, K=k, qparams=util.Q_W8A8, scale_a=SA, scale_b=SB,
                                a_rows=total, m_dev=cnt.data_ptr() + 4 * e, row0_dev=starts.data_ptr() + 4 * e))
    util.run(probs)
    got = Cbuf.cpu().numpy()
    r0 = 0
    for m, ref in zip(counts, refs):
        assert np.array_equal(got[r0:r0 + m].view(np.uint16), ref.view(np.uint16))
        r0 += m


def test_linearity_at_layer_size(cuda_device):
    """Size-independent property at a full expert shape: the int32 accumulators are additive in A."""
    rng = np.random.default_rng(3)
    m, n, k = 1024, 2816, 2048
    c1 = util.WxAxCase.__new__(util.WxAxCase)
    qa1 = rng.integers(-3, 4, (m, k), dtype=np.int32)
    qa2 = rng.integers(-3, 4, (m, k), dtype=np.int32)
    qb = util.rand_codes(rng, n, k, 4)
    outs = []
    from oracle import pack as op
    B = util.t16(op.pack_k(qb, 4), cuda_device)
    for qa in (qa1, qa2, qa1 + qa2):
        A = util.t16(op.pack_k(qa, 4), cuda_device)
        Cacc = torch.zeros((m, n), dtype=torch.int32, device=cuda_device)
        util.run([gg.Problem(A=A, B=B, C=Cacc, M=m, N=n, K=k, qparams=util.Q_W4A4, out_mode=gg.OUT_ACC)])
        outs.append(Cacc)
    assert torch.equal(outs[0] + outs[1], outs[2])
    # and a checksum against the oracle on a row sample
    rows = rng.choice(m, 16, replace=False)
    assert np.array_equal(outs[2][rows].cpu().numpy(), og.int_accumulate((qa1 + qa2)[rows], qb))


def test_bad_arguments_raise(cuda_device):
    from mxmoe_b200._lib import MxMoEError
    rng = np.random.default_rng(1)
    c = util.Fp16Case(rng, 8, 256, 64)
    p = c.problem(cuda_device)
    p.qparams = (16, 3, -1, True)        # unsupported scheme
    with pytest.raises(MxMoEError) as ei:
        gg.GroupedGemm([p])
    assert ei.value.status == 2
    p = c.problem(cuda_device)
    p.N = 252                             # N not a multiple of 8
    with pytest.raises(MxMoEError) as ei:
        gg.GroupedGemm([p])
    assert ei.value.status == 1
    p = c.problem(cuda_device)
    p.A = c.A.data_ptr() + 2              # misaligned operand
    with pytest.raises(MxMoEError):
        gg.GroupedGemm([p])


def test_result_rows_at_given_addresses(cuda_device, gg_kernel):
    """c_row_ptrs: every result row is stored at the address its table entry gives (here: a permutation of the rows
    of one buffer and a second buffer for every third row), whole rows through the copy engine."""
    if gg_kernel not in ("swap", "swap2"):
        pytest.skip("per-row destinations exist in the kernel with swapped operands")
    rng = np.random.default_rng(77)
    for bits, (m, n, k) in ((8, (300, 384, 256)), (4, (177, 2048, 1408)), (8, (5, 256, 128))):
        c = util.WxAxCase(rng, m, n, k, bits, expanded=(bits == 4))
        p = c.problem(cuda_device)
        buf0 = torch.full((m, n), float("nan"), dtype=torch.float16, device=cuda_device)
        buf1 = torch.full((m, n), float("nan"), dtype=torch.float16, device=cuda_device)
        perm = rng.permutation(m)
        which = (np.arange(m) % 3 == 0)
        ptrs = np.where(which, buf1.data_ptr(), buf0.data_ptr()).astype(np.int64) + perm.astype(np.int64) * n * 2
        table = torch.from_numpy(ptrs).to(cuda_device)
        p.c_row_ptrs = table
        util.run([p])
        got0, got1 = buf0.cpu().numpy(), buf1.cpu().numpy()
        for r in range(m):
            got = (got1 if which[r] else got0)[perm[r]]
            assert np.array_equal(got.view(np.uint16), c.ref[r].view(np.uint16)), (bits, r)
        assert np.isnan(c.C.cpu().numpy()).all()          # C itself is not written
        rows_written = np.zeros(m, dtype=int)
        rows_written[perm[~which]] += 1
        assert np.array_equal(~np.isnan(got0).any(axis=1), rows_written == 1)



def test_redirected_c_rows(cuda_device, gg_kernel):
    """c_row0_dev: the rows of C start somewhere else than the rows of A (what lets an expert-parallel rank store
    a segment straight into another rank's buffer).  Only the kernel with swapped operands offers it."""
    rng = np.random.default_rng(11)
    counts, c_starts = [200, 3, 77], [400, 0, 100]
    k, n, bits = 256, 384, 8
    total = sum(counts)
    qa = util.rand_codes(rng, total, k, bits)
    sa = util.rand_scales(rng, total, 0.01, 0.5)
    from oracle import pack as op
    A, SA = util.t16(op.pack_k(qa, bits), cuda_device), util.t16(sa, cuda_device)
    Cbuf = torch.full((700, n), float("nan"), dtype=torch.float16, device=cuda_device)
    cnt = torch.tensor(counts, dtype=torch.int32, device=cuda_device)
    starts = torch.tensor(np.concatenate(([0], np.cumsum(counts)[:-1])), dtype=torch.int32, device=cuda_device)
    cst = torch.tensor(c_starts, dtype=torch.int32, device=cuda_device)
    probs, refs, keep = [], [], []
    for e, m in enumerate(counts):
        qb = util.rand_codes(rng, n, k, bits)
        sb = util.rand_scales(rng, n)
        B, SB = util.t16(op.pack_k(qb, bits), cuda_device), util.t16(sb, cuda_device)
        keep += [B, SB]
        r0 = int(starts[e])
        refs.append(og.wxax_epilogue(og.int_accumulate(qa[r0:r0 + m], qb), sa[r0:r0 + m], sb))
        probs.append(gg.Problem(A=A, B=B, C=Cbuf, M=total, N=n, K=k, qparams=util.Q_W8A8, scale_a=SA, scale_b=SB,
                                a_rows=total, m_dev=cnt.data_ptr() + 4 * e, row0_dev=starts.data_ptr() + 4 * e,
                                c_row0_dev=cst.data_ptr() + 4 * e))
    g = gg.GroupedGemm(probs)
    assert g._plan.flags & 1
    if gg_kernel not in ("swap", "swap2"):
        with pytest.raises(MxMoEError):
            g.run()
        return
    g.run()
    g.check()
    got = Cbuf.cpu().numpy()
    written = np.zeros(700, dtype=bool)
    for m, c0, ref in zip(counts, c_starts, refs):
        assert np.array_equal(got[c0:c0 + m].view(np.uint16), ref.view(np.uint16))
        written[c0:c0 + m] = True
    assert np.isnan(got[~written].astype(np.float32)).all(), "rows outside the redirected ranges were written"


def test_more_problems_than_one_launch_walks(cuda_device):
    """A list longer than the 256 problems one launch can walk (a 256-expert layer plus its shared expert) is
    split into several launches by GroupedGemm; the reference launcher takes any problem count."""
    rng = np.random.default_rng(257)
    cases = [util.WxAxCase(rng, 1 + (i % 5), 128, 128, 8) for i in range(257)]
    g = util.run([c.problem(cuda_device) for c in cases])
    assert g.kept == 257
    for i in (0, 100, 255, 256):
        assert np.array_equal(cases[i].C.cpu().numpy().view(np.uint16), cases[i].ref.view(np.uint16)), i
