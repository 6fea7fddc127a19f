"""File boundary of the grouped-GEMM benchmark: the reference's workload JSON and qconfig JSON in, its CSV out.

    python -m mxmoe_b200.run_gg bench --input WORKLOAD.json --output OUT_PREFIX [--layer N]
    python -m mxmoe_b200.run_gg workload --qconfig QCONFIG.json --config qwen15-mixed-8192 --save WORKLOAD.json

``bench`` does what ``./build/test bench --input ... --output ...`` does in the reference
(mxmoe/kernels/src/test.cu:950-983, driven by run_mxmoe_gg.py:112-121) with the kernels prebuilt instead of
generated: it parses the workload JSON (``{"num_tokens": T, "layer-<i>": {"gate_up": [{"shape": [M, N, K], "w_bits",
"a_bits", "gsize", "sym"}, ...], "down": [...]}}``, gen_workload.py:86-101; test.cu:652-674), fills the operands of
every problem with seeded random values (test.cu:877-915: uniform(-1, 1) fp16, here quantised and packed for the
problem's scheme), times one grouped launch per linear block the way ``bench_func`` does (test_utils.h:97-191: up
to 30 warm-ups, 50 timed calls, the median) against an fp16 grouped launch of the same shapes (the role CUTLASS
GemmGrouped has there) and writes ``<OUT_PREFIX>-<layer>-<gate_up|down>.csv`` with the reference's columns
``kernel_name,avg_time,TFLOPS,speedup`` (test.cu:855-865; avg_time in ms, TFLOPS = sum 2MNK / time).

``workload`` writes a workload JSON for one of the synthetic benchmark configurations, taking the scheme of every
(expert, linear block) from a qconfig JSON in the reference's format (``{layer: {"experts": {e: {"gate"|"up"|"down":
QLinearConfig}}}, "LT": ...}``, qconfig.py:66-80; written by bits_solver.py:42-69) the way gen_workload.py:74-84
reads it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import gg, workload
from .weights import prepare_weight, scheme_name


def parse_workload(path: str) -> dict:
    """``{layer_id: {"gate_up": [problem dicts], "down": [...]}}`` from the reference's workload JSON."""
    with open(path) as f:
        js = json.load(f)
    layers = {}
    for key, val in js.items():
        if key.startswith("layer-"):
            for blk in ("gate_up", "down"):
                for p in val[blk]:
                    assert len(p["shape"]) == 3 and {"w_bits", "a_bits", "gsize", "sym"} <= set(p), f"malformed problem {p}"
            layers[key.split("-", 1)[1]] = val
    return layers


def qconfig_schemes(path: str, layer: str, num_experts_incl_shared: int) -> tuple[list[str], list[str]]:
    """Scheme strings ``(gate_up, down)`` of every expert of ``layer`` from a qconfig JSON (qconfig.py:66-80); the
    gate block's entry stands for the fused gate_up GEMM (gen_workload.py:88)."""
    with open(path) as f:
        q = json.load(f)
    q.pop("LT", None)
    experts = q[str(layer)]["experts"]

    def name(c):
        return scheme_name(c["a_bits"], c["w_bits"], c["w_gsize"], c["w_sym"])
    gu = [name(experts[str(e)]["gate"]) for e in range(num_experts_incl_shared)]
    dn = [name(experts[str(e)]["down"]) for e in range(num_experts_incl_shared)]
    return gu, dn


def _problem(p: dict, dev, gen, fp16_baseline: bool) -> gg.Problem:
    m, n, k = p["shape"]
    scheme = "fp16" if fp16_baseline else scheme_name(p["a_bits"], p["w_bits"], p["gsize"], p["sym"])
    a = (torch.rand(m, k, generator=gen, device=dev) * 2 - 1).half()
    w = (torch.rand(n, k, generator=gen, device=dev) * 2 - 1).half()
    pw = prepare_weight(w, scheme)
    a_bits = pw.qparams[0]
    sa = None
    if a_bits < 16:
        from .weights import pack_along_k, quantize_minmax
        codes, s, _ = quantize_minmax(a, a_bits, -1, True)
        a, sa = pack_along_k(codes, a_bits), s.reshape(m).half().contiguous()
    c = torch.empty(m, n, dtype=torch.float16, device=dev)
    return gg.Problem(A=a, B=pw.data, C=c, M=m, N=n, K=k, qparams=pw.qparams, scale_a=sa, scale_b=pw.scale)


def time_launch(g: gg.GroupedGemm, warmup: int = 30, iters: int = 50) -> float:
    """Median milliseconds of one grouped launch (test_utils.h:97-191: warm-ups, then the median of timed calls)."""
    for _ in range(warmup):
        g.run()
    g.check()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.run()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def bench(input_path: str, output_prefix: str | None, layer: str | None = None, device=None) -> dict:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    results = {}
    for lid, blocks in parse_workload(input_path).items():
        if layer is not None and str(layer) != lid:
            continue
        for blk in ("gate_up", "down"):
            probs = [p for p in blocks[blk] if p["shape"][0] > 0]
            flops = sum(2.0 * p["shape"][0] * p["shape"][1] * p["shape"][2] for p in probs)
            rows = []
            base_ms = None
            for kind in ("fp16", "mixed"):
                gen = torch.Generator(device=dev).manual_seed(42)
                g = gg.GroupedGemm([_problem(p, dev, gen, kind == "fp16") for p in probs], device=dev)
                ms = time_launch(g)
                tf = flops / (ms * 1e-3) / 1e12
                base_ms = ms if kind == "fp16" else base_ms
                schemes = sorted({scheme_name(p["a_bits"], p["w_bits"], p["gsize"], p["sym"]) for p in probs})
                name = "gg_swap_kernel[fp16]" if kind == "fp16" else f"gg_swap_kernel[{', '.join(schemes)}]"
                rows.append((name, ms, tf, base_ms / ms))
                del g
            results[(lid, blk)] = rows
            if output_prefix:
                os.makedirs(os.path.dirname(os.path.abspath(output_prefix)), exist_ok=True)
                with open(f"{output_prefix}-{lid}-{blk}.csv", "w") as f:
                    f.write("kernel_name,avg_time,TFLOPS,speedup\n")
                    for name, ms, tf, sp in rows:
                        f.write(f"\"{name}\",{ms:.4f},{tf:.4f},{sp:.3f}\n")
    return results


def write_workload(config: str, qconfig: str | None, save: str, layer: int = 0) -> None:
    spec = workload.CONFIGS[config]
    ids, _ = workload.make_routing(spec)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=spec.num_experts).tolist()
    if qconfig:
        gu, dn = qconfig_schemes(qconfig, str(layer), spec.num_experts + (1 if spec.shared_inter else 0))
    else:
        gu, dn = workload.draw_schemes(spec)
    os.makedirs(os.path.dirname(os.path.abspath(save)), exist_ok=True)
    with open(save, "w") as f:
        f.write(workload.workload_json(spec, counts, gu, dn, layer=layer))


def qconfig_json(spec, gu: list[str], dn: list[str], layer: int = 0) -> str:
    """A qconfig JSON in the reference's format for the schemes of one layer (what bits_solver.py:42-69 writes)."""
    from .weights import parse_scheme

    def lin(s):
        a, w, g, sym = parse_scheme(s)
        return {"w_bits": w, "w_gsize": g, "w_sym": sym, "w_clip": [1.0, 1.0], "a_bits": a, "a_gsize": -1,
                "a_sym": True, "a_clip": [1.0, 1.0]}
    experts = {str(e): {"gate": lin(gu[e]), "up": lin(gu[e]), "down": lin(dn[e])} for e in range(len(gu))}
    return json.dumps({str(layer): {"experts": experts}}, indent=2)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("bench")
    b.add_argument("--input", required=True)
    b.add_argument("--output", default=None)
    b.add_argument("--layer", default=None)
    w = sub.add_parser("workload")
    w.add_argument("--config", default="qwen15-mixed-8192", choices=sorted(workload.CONFIGS))
    w.add_argument("--qconfig", default=None)
    w.add_argument("--save", required=True)
    w.add_argument("--layer", type=int, default=0)
    args = ap.parse_args()
    if args.cmd == "workload":
        write_workload(args.config, args.qconfig, args.save, args.layer)
        print(f"Save generated workloads to `{args.save}`")
        return
    for (lid, blk), rows in bench(args.input, args.output, args.layer).items():
        for name, ms, tf, sp in rows:
            print(f"layer {lid} {blk}: {name}\navg_time: {ms:<8.4f}, TFLOPS: {tf:<9.4f}, speedup: {sp:<.3f}")


if __name__ == "__main__":
    main()
