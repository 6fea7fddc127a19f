"""The file boundary on the GPU: the reference's workload JSON through the bench to its CSV, and the re-profiler of
the solver's tile-cost table."""
import csv

import pytest

from mxmoe_b200 import perf_table, run_gg, workload

pytestmark = pytest.mark.gpu


def test_bench_reads_workload_json_and_writes_reference_csv(cuda_device, tmp_path):
    spec = workload.LayerSpec("tiny", 6, 2, 512, 256, 512, 64, "zipf", 1.2, True, False, "mixed5")
    gu, dn = workload.draw_schemes(spec)
    wpath = tmp_path / "wl.json"
    wpath.write_text(workload.workload_json(spec, [40, 30, 25, 20, 10, 3], gu, dn, layer=7))
    res = run_gg.bench(str(wpath), str(tmp_path / "out" / "bench"), device=cuda_device)
    assert set(res) == {("7", "gate_up"), ("7", "down")}
    for blk in ("gate_up", "down"):
        with open(tmp_path / "out" / f"bench-7-{blk}.csv") as f:
            rows = list(csv.reader(f))
        assert rows[0] == ["kernel_name", "avg_time", "TFLOPS", "speedup"]      # test.cu:858
        assert len(rows) == 3 and rows[1][0] == "gg_swap_kernel[fp16]" and float(rows[1][3]) == 1.0
        assert float(rows[2][1]) > 0 and float(rows[2][2]) > 0


def test_tile_table_profiler(cuda_device):
    table = perf_table.profile(schemes=["w8a8_g-1_sym"], shapes=((512, 256),), iters=3)
    cost = table["w8a8_g-1_sym"]["3"][repr(perf_table.b200_tile("w8a8_g-1_sym"))]
    assert cost["inc"] > 0 and cost["first_iter_cost"] > 0 and cost["stderr"] >= 0
