"""Re-profile the tile-cost table of the bit-width solver's performance model on this GPU.

The reference's solver reads ``perf/performance_table.json``::

    {scheme: {"1" | "3": {repr(TileConfig): {"first_iter_cost": ms, "inc": ms, "stderr": ms}}}}

and charges a problem ``inc * num_tiles`` (``mxmoe/quant/bits_solver.py:518-542``; it reads sub-key
"1" for weight-only schemes and "3" for weight+activation schemes).  The profiler that produced
the reference table is not part of the reference, so the method here is stated explicitly: for each
scheme the persistent kernel is timed on grouped launches whose tile count sweeps from a fraction
of one wave to many waves at fixed N and K, and ``time = first_iter_cost + inc * tiles`` is fitted
by least squares over the multi-wave points; ``stderr`` is the residual standard deviation.  The key
is the ``repr`` of a dataclass with the reference's field names (``tile_config.py:195-207``), so the
file drops into the solver unchanged; B200 has one tile shape per scheme (up to 176 token rows x 128
output channels, 128 bytes of K per stage: the kernel with swapped operands; w4a4 is profiled with the
layer's expanded int4 activations).

    python -m mxmoe_b200.perf_table [out.json]
"""
from __future__ import annotations

import dataclasses
import json
import os
import sys


# Twins of the reference's dataclasses (tile_config.py:117-207) with the same class names, field names, field order
# and defaults, so that ``repr`` gives the very string the solver uses as a key.
@dataclasses.dataclass
class NO_QUANT:
    T_PACK: str = "half"
    QBITS: int = 16
    GSIZE: int = -1
    SYM: bool = True
    PACK_DIM: str = "PackDim::K"
    USE_FP: bool = False
    T_SCALE: str = "half"


@dataclasses.dataclass
class QConfig:
    T_PACK: str = "half"
    QBITS: int = 16
    GSIZE: int = -1
    SYM: bool = True
    PACK_DIM: str = "PackDim::K"
    USE_FP: bool = False
    T_SCALE: str = "half"


@dataclasses.dataclass
class TileConfig:
    BM: int = 176
    BN: int = 128
    BK: int = 128
    WM: int = 4
    WN: int = 1
    WK: int = 1
    STAGE: int = 5
    SPLITK: int = -1
    MMA: str = "TCGEN05_F16_F32"
    QCFGA: object = dataclasses.field(default_factory=NO_QUANT)
    QCFGB: object = dataclasses.field(default_factory=NO_QUANT)


def b200_tile(scheme: str) -> TileConfig:
    """The tile the sm_100a kernel uses for ``scheme`` (BK in elements of K per pipeline stage)."""
    from .weights import parse_scheme
    a, w, g, sym = parse_scheme(scheme)
    if a >= 16 and w >= 16:
        return TileConfig(BK=64, MMA="TCGEN05_F16_F32")
    if a < 16:
        q = QConfig(QBITS=w, GSIZE=g, SYM=sym, PACK_DIM="PackDim::K")
        qa = QConfig(QBITS=a, GSIZE=g, SYM=sym, PACK_DIM="PackDim::K")
        return TileConfig(BK=128, MMA="TCGEN05_S8_S32", QCFGA=qa, QCFGB=q)
    return TileConfig(BK=64, MMA="TCGEN05_F16_F32",
                      QCFGB=QConfig(QBITS=w, GSIZE=g, SYM=sym, PACK_DIM="PackDim::MN"))


def get_best_tile_configs(batch_range: int, strategy_list: list[str]) -> dict:
    """B200 counterpart of the solver's hard-coded shortlist (bits_solver.py:425-515): the candidate tiles per scheme
    for a batch range.  The sm_100a kernel has one tile per scheme whatever the batch (its token tile adapts to the
    rows an expert has: up to 176, in steps of 16), so every batch range maps to the same single candidate."""
    return {s: [b200_tile(s)] for s in strategy_list}


def subkey(scheme: str) -> str:
    return "1" if "a16" in scheme or scheme == "fp16" else "3"


def _fit(tiles, ms):
    n = len(tiles)
    mx, my = sum(tiles) / n, sum(ms) / n
    sxx = sum((x - mx) ** 2 for x in tiles)
    inc = sum((x - mx) * (y - my) for x, y in zip(tiles, ms)) / sxx
    first = my - inc * mx
    res = [y - (first + inc * x) for x, y in zip(tiles, ms)]
    stderr = (sum(r * r for r in res) / max(1, n - 2)) ** 0.5
    return first, inc, stderr


def profile(schemes=None, shapes=((2816, 2048), (2048, 1408)), iters: int = 20) -> dict:
    import torch
    from . import gg, _lib
    from .weights import parse_scheme, SCHEMES, EXTRA_SCHEMES
    dev = torch.device("cuda", torch.cuda.current_device())
    sms = _lib.lib().mxmoe_device_sm_count()
    table = {}
    for scheme in (schemes or SCHEMES + EXTRA_SCHEMES):
        a_bits, w_bits, g, sym = parse_scheme(scheme)
        entry = {"inc_by_nk": {}}
        for (N, K) in shapes:
            nt = (N + 127) // 128
            pts_t, pts_ms = [], []
            for waves in (0.5, 1, 2, 3, 4, 6, 8, 12, 16):
                m_tiles = max(1, round(waves * sms / nt))
                M = m_tiles * 176
                expanded = a_bits == 4          # the layer's activation format for w4a4: one byte 16*q per code
                A = (torch.randint(-30000, 30000, (M, K * (8 if expanded else a_bits) // 16), dtype=torch.int16, device=dev)
                     if a_bits < 16 else torch.randn(M, K, device=dev).half())
                if w_bits >= 16:
                    B, SB = (torch.randn(N, K, device=dev) * 0.02).half(), None
                elif a_bits >= 16:
                    B = torch.randint(-30000, 30000, (N // 4, K), dtype=torch.int16, device=dev)
                    SB = (torch.rand(K // 128, N, 2, device=dev) * 0.01).half()
                else:
                    B = torch.randint(-30000, 30000, (N, K * w_bits // 16), dtype=torch.int16, device=dev)
                    SB = (torch.rand(N, device=dev) * 0.01).half()
                SA = (torch.rand(M, device=dev) * 0.1).half() if a_bits < 16 else None
                Cc = torch.empty(M, N, dtype=torch.float16, device=dev)
                run = gg.GroupedGemm([gg.Problem(A=A, B=B, C=Cc, M=M, N=N, K=K, qparams=(a_bits, w_bits, g, sym),
                                                 scale_a=SA, scale_b=SB, a_expanded=1 if expanded else 0)])
                for _ in range(3):
                    run.run()
                run.check()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    run.run()
                e1.record()
                torch.cuda.synchronize()
                pts_t.append(m_tiles * nt)
                pts_ms.append(e0.elapsed_time(e1) / iters)
            first, inc, stderr = _fit(pts_t[2:], pts_ms[2:])       # multi-wave points only
            entry["inc_by_nk"][f"{N}x{K}"] = {"first_iter_cost": pts_ms[1], "inc": inc, "stderr": stderr,
                                              "tiles": pts_t, "ms": pts_ms}
        ref = entry["inc_by_nk"][f"{shapes[0][0]}x{shapes[0][1]}"]
        table[scheme] = {subkey(scheme): {repr(b200_tile(scheme)): {
            "first_iter_cost": ref["first_iter_cost"], "inc": ref["inc"], "stderr": ref["stderr"],
            "by_shape": entry["inc_by_nk"]}}}
    return table


def main() -> None:
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "perf",
                                                             "performance_table.json")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    table = profile()
    with open(out, "w") as f:
        json.dump(table, f, indent=1)
    for s, v in table.items():
        for sk, tiles in v.items():
            for k, c in tiles.items():
                print(f"{s:18s} [{sk}] inc={c['inc'] * 1e3:7.3f} us/tile first={c['first_iter_cost'] * 1e3:7.1f} us "
                      f"stderr={c['stderr'] * 1e3:6.2f} us")


if __name__ == "__main__":
    main()
