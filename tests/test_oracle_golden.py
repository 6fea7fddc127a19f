"""The oracle against golden vectors produced by the reference's own code (tests/golden/make_golden.py)."""
import os

import numpy as np
import torch

from oracle import gemm as og
from oracle import hadamard as oh
from oracle import pack as op
from oracle import quant as oq

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_quantiser_matches_reference():
    z = np.load(os.path.join(G, "quant.npz"))
    x16, w16 = torch.from_numpy(z["x16"]), torch.from_numpy(z["w16"])
    for name, t, bits, gs, sym in (("a4", x16, 4, -1, True), ("a8", x16, 8, -1, True), ("w4", w16, 4, -1, True),
                                   ("w8", w16, 8, -1, True), ("w4g128", w16, 4, 128, False)):
        q, s, zero = oq.minmax_quantize(t.clone(), bits, gs, sym)
        assert np.array_equal(q.numpy().astype(np.int8), z[f"{name}_codes"]), name
        assert np.array_equal(s.numpy().view(np.uint16), z[f"{name}_scale"].view(np.uint16)), name
        if not sym:
            assert np.array_equal(zero.numpy().view(np.uint16), z[f"{name}_zero"].view(np.uint16))
        fq = oq.fake_quant(t.clone(), bits, gs, sym)
        assert np.array_equal(fq.numpy().view(np.uint16), z[f"{name}_fake"].view(np.uint16)), name


def test_hadamard_matches_reference():
    z = np.load(os.path.join(G, "hadamard.npz"))
    for n in (64, 2048, 4096):
        y = oh.hadamard_rows(torch.from_numpy(z[f"x{n}"]))
        assert np.array_equal(y.numpy(), z[f"y{n}"]), n
    q = oh.random_hadamard(128, torch.Generator().manual_seed(4))
    assert np.array_equal(q.numpy(), z["Q128_seed4"])
    # Q = diag(s) H / sqrt(n): orthogonal up to the fp32 rounding of sqrt(n)
    assert np.allclose(q.numpy() @ q.numpy().T, np.eye(128), atol=1e-6)


def test_hadamard_kron_matches_reference():
    """Sizes with a Kronecker factor (1408 = 176 x 8, 14336 = 28 x 512) against the reference's matmul_hadU."""
    z = np.load(os.path.join(G, "hadamard_kron.npz"))
    for n in (1408, 14336):
        had = torch.from_numpy(z[f"had{n}"].astype(np.float64))
        assert had.shape[0] == int(z[f"k{n}"]) and torch.equal(had @ had.t(), had.shape[0] * torch.eye(had.shape[0], dtype=torch.float64))
        y = oh.hadamard_kron_rows(torch.from_numpy(z[f"x{n}"]), had)
        assert np.allclose(y.numpy(), z[f"y{n}"], rtol=0, atol=1e-12), n


def test_pack_matches_reference_packers():
    z = np.load(os.path.join(G, "pack.npz"))
    for bits in (4, 8):
        for side in ("act", "wgt"):
            codes = z[f"k{bits}_{side}"].astype(np.int32)
            assert np.array_equal(op.pack_k(codes, bits), z[f"k{bits}_{side}_packed"])
            assert np.array_equal(op.unpack_k(z[f"k{bits}_{side}_packed"], bits), codes)
    assert z["probe_9abc"][0, 0] == 0x9ABC
    assert op.pack_k(np.array([[-7, -6, -5, -4]]), 4)[0, 0] == 0x9ABC
    w = z["n4_wgt"].astype(np.int32)
    assert np.array_equal(op.pack_n4(w), z["n4_wgt_packed"])
    assert np.array_equal(op.unpack_n4(z["n4_wgt_packed"]), w)
    sz = z["n4_scale_zero"]
    got = op.group_major_scales(sz[..., 0], sz[..., 1])
    assert np.array_equal(got.view(np.uint16), z["n4_scale_zero_packed"].view(np.uint16))


def test_layer_slice_matches_reference():
    """Rotation -> quantiser -> exact accumulators -> epilogue, on the config-1-shaped golden slice."""
    z = np.load(os.path.join(G, "layer_w4a4_had.npz"))
    signs = torch.from_numpy(z["signs"].astype(np.float64))
    for tag in ("hot", "median", "cold"):
        x = torch.from_numpy(z[f"{tag}_x"])
        xr = oh.hadamard_rows(x.double() * signs).half()
        # the reference rotates with an fp64 matmul; the butterfly differs in the last fp64 bits only
        same = (xr.numpy().view(np.uint16) == z[f"{tag}_xr"].view(np.uint16)).mean()
        assert same > 0.999, same
        qa, sa, _ = oq.minmax_quantize(torch.from_numpy(z[f"{tag}_xr"]), 4, -1, True)
        qb, sb, _ = oq.minmax_quantize(torch.from_numpy(z[f"{tag}_wr"]), 4, -1, True)
        assert np.array_equal(qa.numpy().astype(np.int8), z[f"{tag}_qa"])
        assert np.array_equal(qb.numpy().astype(np.int8), z[f"{tag}_qb"])
        acc = og.int_accumulate(z[f"{tag}_qa"], z[f"{tag}_qb"])
        assert np.array_equal(acc, z[f"{tag}_acc"])
        if og.c_port() is not None:
            assert np.array_equal(og.int_accumulate_c(z[f"{tag}_qa"], z[f"{tag}_qb"]), z[f"{tag}_acc"])
            assert np.array_equal(og.wxax_epilogue_c(acc, z[f"{tag}_sa"], z[f"{tag}_sb"]).view(np.uint16),
                                  og.wxax_epilogue(acc, z[f"{tag}_sa"], z[f"{tag}_sb"]).view(np.uint16))
        out = og.wxax_epilogue(acc, z[f"{tag}_sa"], z[f"{tag}_sb"])
        # the scaled output agrees with the reference's fake-quant product to fp16 rounding
        assert og.rel_l2(out, z[f"{tag}_fake"]) < 2e-3


def test_w4a16_dequant_is_one_rounding():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, (32, 256))
    s = rng.uniform(0.001, 0.01, (32, 2)).astype(np.float16)
    zp = rng.uniform(-0.1, 0.0, (32, 2)).astype(np.float16)
    w = og.dequant_w4a16(q, s, zp)
    # against the quantiser's own dequantisation (two fp16 roundings) the difference is at most one ulp
    ref = (q.astype(np.float16) * np.repeat(s, 128, 1)) + np.repeat(zp, 128, 1)
    assert np.abs(w.astype(np.float32) - ref.astype(np.float32)).max() <= 2 ** -10 * 0.2
