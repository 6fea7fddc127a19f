"""CPU tests of the host side: C-ABI exports, weight preparation, workload generation, error paths."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

from oracle import pack as op
from oracle import quant as oq
from mxmoe_b200 import _lib, weights, workload

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "mxmoe_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(mxmoe_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = _lib.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(_lib.EXPORTS)


def test_struct_layouts_match_header():
    assert ctypes.sizeof(_lib.QParams) == 16
    assert ctypes.sizeof(_lib.GGProblem) == 136
    assert ctypes.sizeof(_lib.GGPlan) == 16
    assert ctypes.sizeof(_lib.EpPlanArgs) == 13 * 8 + 8 * 4
    assert ctypes.sizeof(_lib.EpDispatchArgs) == 7 * 8 + 6 * 4
    assert ctypes.sizeof(_lib.ActArgs) == 12 * 8 + 8 * 4
    assert ctypes.sizeof(_lib.RouteArgs) == 11 * 8 + 4 * 4
    assert ctypes.sizeof(_lib.TokenQuantArgs) == 8 * 8 + 4 * 4


def test_no_device_is_an_error_not_a_fallback():
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    lib = _lib.lib()
    assert lib.mxmoe_device_sm_count() == -6
    plan = _lib.GGPlan()
    p = (_lib.GGProblem * 1)()
    rc = lib.mxmoe_gg_prepare(ctypes.byref(p), 1, 256, 4096, None, ctypes.byref(plan))
    assert rc == 6 and b"no CUDA device" in lib.mxmoe_last_error()
    assert lib.mxmoe_gg_workspace_bytes(10) == 256 + 10 * (384 + 640)


def test_argument_validation_without_device():
    lib = _lib.lib()
    assert lib.mxmoe_gg_prepare(None, 3, 256, 1 << 20, None, None) == 1
    assert lib.mxmoe_gg_prepare(None, 0, None, 0, None, None) == 4
    assert lib.mxmoe_gg_prepare(None, 100000, 256, 1 << 20, None, None) == 1
    assert lib.mxmoe_quant_act(None, None) == 1
    a = _lib.ActArgs()
    assert lib.mxmoe_quant_act(ctypes.byref(a), None) == 1
    r = _lib.RouteArgs()
    r.num_tokens, r.topk, r.num_experts = 4, 2, 100000
    assert lib.mxmoe_route_topk(ctypes.byref(r), None) == 1


@pytest.mark.parametrize("scheme", weights.SCHEMES + weights.EXTRA_SCHEMES)
def test_prepare_weight_matches_oracle_layouts(scheme):
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(64, 256, generator=g) * 0.02).half()
    pw = weights.prepare_weight(w, scheme, keep_codes=True)
    a, wb, gs, sym = weights.parse_scheme(scheme)
    assert pw.qparams == (a, wb, gs, sym) == oq.scheme_tuple(scheme)
    if scheme == "fp16":
        assert torch.equal(pw.data, w) and pw.scale is None
        return
    codes, scale, zero = oq.minmax_quantize(w, wb, gs, sym)
    assert torch.equal(pw.codes.to(torch.float16), codes)
    packed = pw.data.numpy().view(np.uint16)
    if a < 16:
        assert np.array_equal(packed, op.pack_k(codes.numpy().astype(np.int32), wb))
        assert np.array_equal(pw.scale.numpy().view(np.uint16), scale.reshape(-1).numpy().view(np.uint16))
    else:
        assert np.array_equal(packed, op.pack_n4(codes.numpy().astype(np.int32)))
        want = op.group_major_scales(scale.reshape(64, -1).numpy(), zero.reshape(64, -1).numpy())
        assert np.array_equal(pw.scale.numpy().view(np.uint16), want.view(np.uint16))


def test_prepare_weight_rejects_unknown_scheme():
    w = torch.zeros(32, 128, dtype=torch.float16)
    with pytest.raises(ValueError):
        weights.prepare_weight(w, "w3a16_g64_asym")
    with pytest.raises(ValueError):
        weights.prepare_weight(w, "bogus")
    with pytest.raises(ValueError):
        weights.prepare_weight(torch.zeros(30, 128, dtype=torch.float16), "w4a16_g128_asym")


def test_routing_is_seeded_and_valid():
    spec = workload.CONFIGS["qwen15-w4a4-512"]
    ids, w = workload.make_routing(spec)
    ids2, _ = workload.make_routing(spec)
    assert torch.equal(ids, ids2) and ids.dtype == torch.int32 and ids.shape == (512, 4)
    assert (ids.sort(dim=1).values.diff(dim=1) != 0).all(), "top-k without replacement"
    assert torch.allclose(w.sum(1), torch.ones(512))
    cnt = torch.bincount(ids.reshape(-1).long(), minlength=60)
    assert cnt[0] > 4 * cnt.float().median(), "Zipf skew"
    spec5 = workload.CONFIGS["mixtral-mixed-16384"]
    ids5, _ = workload.make_routing(spec5, tokens=2000)
    c5 = torch.bincount(ids5.reshape(-1).long(), minlength=8)
    assert c5[0] == c5.max()


def test_mixed_scheme_draw_hits_five_bits():
    spec = workload.CONFIGS["qwen15-mixed-8192"]
    gu, dn = workload.draw_schemes(spec)
    assert len(gu) == len(dn) == 61
    assert set(gu + dn) == set(weights.SCHEMES)
    assert abs(workload.mean_weight_bits(spec, gu, dn) - 5.0) <= 0.02
    assert (gu, dn) == workload.draw_schemes(spec)
    gu5, dn5 = workload.draw_schemes(workload.CONFIGS["mixtral-mixed-16384"])
    assert gu5 == dn5 and set(gu5) == {"w8a8_g-1_sym", "w4a4_g-1_sym"}


def test_rotation_matches_oracle():
    from oracle import hadamard as oh
    spec = workload.CONFIGS["qwen15-w4a4-512"]
    s = workload.rotation_signs(spec)
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(8, spec.hidden, generator=g) * 0.02).half()
    got = workload.rotate_rows(w, s)
    ref = oh.hadamard_rows(w.double() * s.double()).half()
    assert torch.equal(got, ref)


def test_workload_json_schema():
    spec = workload.CONFIGS["ds2lite-w4a16-32"]
    gu, dn = workload.draw_schemes(spec)
    js = json.loads(workload.workload_json(spec, [1] * 64, gu, dn, layer=3))
    assert js["num_tokens"] == 32
    blk = js["layer-3"]
    assert len(blk["gate_up"]) == 65 and len(blk["down"]) == 65
    assert blk["gate_up"][0] == {"shape": [1, 2816, 2048], "w_bits": 4, "a_bits": 16, "gsize": 128, "sym": False}
    assert blk["down"][-1]["shape"] == [32, 2048, 2816]


def test_flops_formula():
    spec = workload.CONFIGS["qwen15-w4a4-8192"]
    assert spec.flops() == 2 * 32768 * (2816 * 2048 + 2048 * 1408)


def test_perf_table_schema_matches_the_solver_input():
    """Keys and fields the reference solver reads (bits_solver.py:518-542): table[scheme]["1"|"3"][repr(tile)]["inc"]."""
    from mxmoe_b200 import perf_table
    path = os.path.join(ROOT, "mxmoe_b200", "perf", "performance_table.json")
    table = json.load(open(path))
    assert set(table) == set(weights.SCHEMES + weights.EXTRA_SCHEMES)
    # the key is the very string the reference's TileConfig.__repr__ gives (golden made from the reference's dataclass)
    golden = json.load(open(os.path.join(ROOT, "tests", "golden", "tile_repr.json")))
    for scheme in table:
        assert repr(perf_table.b200_tile(scheme)) == golden[scheme]
    assert perf_table.get_best_tile_configs(8192, ["fp16", "w4a4_g-1_sym"])["w4a4_g-1_sym"] == [perf_table.b200_tile("w4a4_g-1_sym")]
    for scheme, by_key in table.items():
        sk = "1" if ("a16" in scheme or scheme == "fp16") else "3"
        assert list(by_key) == [sk]
        key = repr(perf_table.b200_tile(scheme))
        assert key.startswith("TileConfig(BM=176, BN=128, BK=") and key in by_key[sk]
        cost = by_key[sk][key]
        assert {"first_iter_cost", "inc", "stderr"} <= set(cost) and cost["inc"] > 0
    # int8 tiles must be cheaper than fp16 tiles of the same shape, 4-bit weight-only the most expensive
    inc = {s: next(iter(next(iter(v.values())).values()))["inc"] for s, v in table.items()}
    assert inc["w8a8_g-1_sym"] < inc["fp16"] < inc["w4a16_g128_asym"]


def test_verify_decodes_the_stored_layouts():
    """mxmoe_b200.verify reads activation rows and packed weights back into logical order: checked against the
    oracle's packers (which are pinned to the reference's)."""
    from oracle import pack as op
    from mxmoe_b200 import verify
    rng = np.random.default_rng(0)
    q4 = rng.integers(-7, 8, (5, 256)).astype(np.int32)
    q8 = rng.integers(-127, 128, (5, 256)).astype(np.int32)

    def carrier(a):
        return torch.from_numpy(a.copy()).view(torch.float16).reshape(-1)
    got = verify.decode_rows(carrier(op.expand_k4(q4)), 128, 0, 5, 256, 3)
    assert np.array_equal(got.numpy().astype(np.int32), q4)
    got = verify.decode_rows(carrier(op.pack_k(q8, 8).view(np.int16)), 128, 0, 5, 256, 1)
    assert np.array_equal(got.numpy().astype(np.int32), q8)
    got = verify.decode_rows(carrier(op.pack_k(q4, 4).view(np.int16)), 64, 1, 3, 256, 2)
    assert np.array_equal(got.numpy().astype(np.int32), q4[1:4])
    w = (torch.randn(64, 256, generator=torch.Generator().manual_seed(0)) * 0.02).half()
    for scheme in ("w4a4_g-1_sym", "w8a8_g-1_sym", "w4a16_g128_asym"):
        pw = weights.prepare_weight(w, scheme, keep_codes=True)
        vals, _ = verify.decode_weight(pw)
        if scheme == "w4a16_g128_asym":
            s = pw.scale[..., 0].t().repeat_interleave(128, dim=1).double()
            z = pw.scale[..., 1].t().repeat_interleave(128, dim=1).double()
            assert torch.equal(vals, (pw.codes.double() * s + z).half())
        else:
            assert torch.equal(vals, pw.codes.double())


def test_torch_extension_exposes_the_reference_operator_names():
    """mxmoe_ops.so (torch C++ extension over the C ABI) loads without a GPU and has the five functions of the
    reference's pybind module (ref_bind.cu:759-768)."""
    mxmoe_ops = pytest.importorskip("mxmoe_b200.mxmoe_ops")
    for name in ("gg_cutlass", "gg_cutlass_share_fused", "gg_mxmoe_share_fused", "quant_inp_act", "silu_mul_then_quant"):
        assert callable(getattr(mxmoe_ops, name))
    with pytest.raises(RuntimeError):                      # TORCH_CHECK -> Python exception, as in the reference
        mxmoe_ops.gg_mxmoe_share_fused([], [], [], [], [], 1, 1, 0, 0, [], torch.zeros(1, dtype=torch.int64), False)


def test_workload_and_qconfig_files_round_trip(tmp_path):
    """The reference's two JSON formats: a qconfig (qconfig.py:66-80) decides the schemes of a workload file
    (gen_workload.py:86-101), and the workload file parses back into the problem lists the bench runs."""
    from mxmoe_b200 import run_gg
    spec = workload.CONFIGS["qwen15-mixed-8192"]
    gu, dn = workload.draw_schemes(spec)
    qpath, wpath = tmp_path / "q.json", tmp_path / "w.json"
    qpath.write_text(run_gg.qconfig_json(spec, gu, dn, layer=11))
    q = json.loads(qpath.read_text())
    assert set(q["11"]["experts"]["0"]) == {"gate", "up", "down"}
    assert set(q["11"]["experts"]["0"]["gate"]) == {"w_bits", "w_gsize", "w_sym", "w_clip", "a_bits", "a_gsize", "a_sym", "a_clip"}
    assert run_gg.qconfig_schemes(str(qpath), "11", 61) == (gu, dn)
    run_gg.write_workload("qwen15-mixed-8192", str(qpath), str(wpath), layer=11)
    layers = run_gg.parse_workload(str(wpath))
    assert list(layers) == ["11"] and len(layers["11"]["gate_up"]) == 61
    p = layers["11"]["down"][-1]
    assert p["shape"] == [8192, 2048, 5632]
    a, w, g, sym = weights.parse_scheme(dn[60])
    assert (p["a_bits"], p["w_bits"], p["gsize"], p["sym"]) == (a, w, g, sym)
