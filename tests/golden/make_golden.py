"""Generate the golden vectors under tests/golden/ from the REFERENCE's own code.

Run where the MxMoE checkout is mounted, after ``make -C oracle ref REF_ROOT=/path/to/MxMoE`` has
compiled the reference's host packers:

    python tests/golden/make_golden.py /path/to/MxMoE        (or REF_ROOT=/path/to/MxMoE)

Sources of truth used here (nothing from this repository's oracle or product code):
  * ``mxmoe.quant.quant.quant_minmax`` / ``Quantizer``            (quant.py:40-109)
  * ``mxmoe.quant.hadamard_utils.matmul_hadU`` / ``random_hadamard_matrix`` (hadamard_utils.py:62-94)
  * ``pack_wxax`` / ``permute_weight`` + ``pack_weightonly`` / ``permute_scale``
    (quantize.cuh:299-475) through oracle/_ref/libref_pack.so
  * exact integer matmul (torch.int32) for the accumulators.
The vectors travel with the repository; the reference checkout does not.
"""
import ctypes
import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REF_ROOT")
if not REF or not os.path.isdir(os.path.join(REF, "mxmoe")):
    raise SystemExit("make_golden.py: pass the MxMoE checkout as the first argument (or set REF_ROOT)")
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REF)
# the CUDA Hadamard extension is an un-vendored submodule; only its import is stubbed, never its math
sys.modules.setdefault("fast_hadamard_transform", types.ModuleType("fast_hadamard_transform"))

from mxmoe.quant.quant import quant_minmax, Quantizer  # noqa: E402
from mxmoe.quant import hadamard_utils as hu  # noqa: E402

lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_pack.so"))
VP = ctypes.c_void_p


def ptr(a):
    return a.ctypes.data_as(VP)


def golden_quant():
    g = torch.Generator().manual_seed(11)
    out = {}
    x16 = torch.randn(24, 256, generator=g).half()
    x16[5] *= 30
    w16 = (torch.randn(48, 256, generator=g) * 0.02).half()
    out["x16"], out["w16"] = x16.numpy(), w16.numpy()
    for name, t, bits, gs, sym in (("a4", x16, 4, -1, True), ("a8", x16, 8, -1, True), ("w4", w16, 4, -1, True),
                                   ("w8", w16, 8, -1, True), ("w4g128", w16, 4, 128, False)):
        q, s, z = quant_minmax(t.clone(), bits, gs, sym)
        out[f"{name}_codes"] = q.numpy().astype(np.int8)
        out[f"{name}_scale"] = s.numpy()
        out[f"{name}_zero"] = z.numpy() if torch.is_tensor(z) else np.zeros_like(s.numpy())
        out[f"{name}_fake"] = Quantizer(bits, sym, gs).fake_quant(t.clone()).numpy()
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **out)


def golden_hadamard():
    g = torch.Generator().manual_seed(12)
    out = {}
    for n in (64, 2048, 4096):
        x = torch.randn(3, n, generator=g, dtype=torch.float64)
        out[f"x{n}"] = x.numpy()
        out[f"y{n}"] = hu.matmul_hadU(x).numpy()
    torch.manual_seed(4)
    out["Q128_seed4"] = hu.random_hadamard_matrix(128).numpy()
    np.savez_compressed(os.path.join(HERE, "hadamard.npz"), **out)


def golden_hadamard_kron():
    """Sizes that are not powers of two: ``matmul_hadU`` with the Kronecker factor ``get_hadK`` picks
    (hadamard_utils.py:5-59): 1408 = 176 x 8 (Qwen1.5-MoE expert intermediate) and 14336 = 28 x 512 (Mixtral).
    Stores the reference's K x K factor (+-1), the inputs and the transformed rows."""
    g = torch.Generator().manual_seed(15)
    out = {}
    for n in (1408, 14336):
        had, k = hu.get_hadK(n)
        x = torch.randn(3, n, generator=g, dtype=torch.float64)
        out[f"k{n}"] = np.array(k)
        out[f"had{n}"] = had.numpy().astype(np.int8)
        out[f"x{n}"] = x.numpy()
        out[f"y{n}"] = hu.matmul_hadU(x).numpy()
    np.savez_compressed(os.path.join(HERE, "hadamard_kron.npz"), **out)


def golden_tile_repr():
    """``repr`` of the reference's TileConfig dataclass (mxmoe/kernels/tile_config.py:195-207) - the key of
    perf/performance_table.json that bits_solver.py:541 looks up - for the tile numbers of the B200 kernel, with the
    quantisation descriptors the solver attaches (``set_qcfg(QCFG_MAP[scheme])``, bits_solver.py:519)."""
    import json
    from mxmoe.kernels.tile_config import QCFG_MAP, TileConfig
    sys.path.insert(0, ROOT)
    from mxmoe_b200 import perf_table
    out = {}
    for scheme in ("fp16", "w8a8_g-1_sym", "w4a4_g-1_sym", "w4a16_g128_asym", "w4a16_g-1_asym"):
        t = perf_table.b200_tile(scheme)
        ref = TileConfig(BM=t.BM, BN=t.BN, BK=t.BK, WM=t.WM, WN=t.WN, WK=t.WK, STAGE=t.STAGE, SPLITK=t.SPLITK, MMA=t.MMA)
        out[scheme] = repr(ref.set_qcfg(QCFG_MAP[scheme]))
    with open(os.path.join(HERE, "tile_repr.json"), "w") as f:
        json.dump(out, f, indent=1)


def golden_pack():
    rng = np.random.default_rng(13)
    out = {}
    for bits in (4, 8):
        hi = 2 ** (bits - 1) - 1
        m, n, k = 9, 16, 128
        a = rng.integers(-hi, hi + 1, (m, k), dtype=np.int32)
        w = rng.integers(-hi, hi + 1, (n, k), dtype=np.int32)
        pa = np.zeros((m, k * bits // 16), np.uint16)
        pw = np.zeros((n, k * bits // 16), np.uint16)
        assert lib.ref_pack_wxax(ptr(a), ptr(w), m, n, k, bits, ptr(pa), ptr(pw)) == 0
        out[f"k{bits}_act"], out[f"k{bits}_wgt"] = a.astype(np.int8), w.astype(np.int8)
        out[f"k{bits}_act_packed"], out[f"k{bits}_wgt_packed"] = pa, pw
    # the documented probe: codes -7,-6,-5,-4 pack to 0x9abc
    a = np.array([[-7, -6, -5, -4]], dtype=np.int32)
    pa = np.zeros((1, 1), np.uint16)
    pw = np.zeros((1, 1), np.uint16)
    assert lib.ref_pack_wxax(ptr(a), ptr(a), 1, 1, 4, 4, ptr(pa), ptr(pw)) == 0
    out["probe_9abc"] = pa
    n, k = 64, 256
    w = rng.integers(0, 16, (n, k), dtype=np.int32)
    pw = np.zeros((n // 4, k), np.uint16)
    assert lib.ref_permute_pack_weightonly(ptr(w), n, k, 4, 0, ptr(pw)) == 0
    out["n4_wgt"], out["n4_wgt_packed"] = w.astype(np.int8), pw
    sz = rng.standard_normal((n, k // 128, 2)).astype(np.float16)
    ps = np.zeros(sz.size, np.uint16)
    assert lib.ref_permute_scale(ptr(sz.view(np.uint16)), sz.size, n, k, 128, 4, 0, ptr(ps)) == 0
    out["n4_scale_zero"], out["n4_scale_zero_packed"] = sz, ps.view(np.float16).reshape(k // 128, n, 2)
    np.savez_compressed(os.path.join(HERE, "pack.npz"), **out)


def golden_layer():
    """Config-1-shaped slice: Qwen1.5-MoE expert (H=2048), w4a4 per-token / per-channel, Hadamard-rotated.

    Three experts' worth of rows (hot / median / cold row counts 48 / 13 / 2) against a 64-row slice
    of the gate_up weight: reference-rotated inputs, reference codes and scales, exact int32
    accumulators and the reference's fake-quant product.
    """
    H = 2048
    torch.manual_seed(4)
    Q = hu.random_hadamard_matrix(H)                       # fp64, global generator as in the reference
    g = torch.Generator().manual_seed(14)
    out = {"signs": np.sign(Q[:, 0].numpy()).astype(np.int8)}
    for tag, m in (("hot", 48), ("median", 13), ("cold", 2)):
        x = torch.randn(m, H, generator=g).half()
        w = (torch.randn(64, H, generator=g) * 0.02).half()
        xr = (x.double() @ Q).half()                       # rotation.py:353-358 (fp64 matmul, stored fp16)
        wr = (w.double() @ Q).half()
        qa, sa, _ = quant_minmax(xr.clone(), 4, -1, True)
        qb, sb, _ = quant_minmax(wr.clone(), 4, -1, True)
        acc = qa.to(torch.int32) @ qb.to(torch.int32).t()
        fa = Quantizer(4, True, -1).fake_quant(xr.clone())
        fb = Quantizer(4, True, -1).fake_quant(wr.clone())
        out[f"{tag}_x"] = x.numpy()
        out[f"{tag}_xr"], out[f"{tag}_wr"] = xr.numpy(), wr.numpy()
        out[f"{tag}_qa"], out[f"{tag}_qb"] = qa.numpy().astype(np.int8), qb.numpy().astype(np.int8)
        out[f"{tag}_sa"], out[f"{tag}_sb"] = sa.numpy().reshape(-1), sb.numpy().reshape(-1)
        out[f"{tag}_acc"] = acc.numpy()
        out[f"{tag}_fake"] = (fa.float() @ fb.float().t()).numpy()
    np.savez_compressed(os.path.join(HERE, "layer_w4a4_had.npz"), **out)


if __name__ == "__main__":
    golden_quant()
    golden_hadamard()
    golden_hadamard_kron()
    golden_tile_repr()
    golden_pack()
    golden_layer()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
