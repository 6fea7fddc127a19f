#!/usr/bin/env python
"""Benchmark of the mixed-precision MoE layer (routing -> quantise -> grouped GEMM gate_up ->
silu*mul+quantise -> grouped GEMM down -> combine) on synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the layer over one batch.  Prints ONE JSON line (rank 0).
Metric: effective TFLOP/s = sum over problems of 2*M*N*K / step time (the reference's definition,
mxmoe/kernels/src/test.cu:109-116), whole job; tokens/s is reported beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_layer_grouped_gemm_effective_tflops"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["source"] = "fallback"
    return p


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8)),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40)),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20)),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)),
        }
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                if get_reasons:
                    r = get_reasons(self.h)
                    for k, bit in names.items():
                        if r & bit:
                            self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr:
            self._thr.join(timeout=1)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------- CPU arm
def cpu_expert_loop(spec, budget_s: float, threads: int, repeats: int = 1):
    """Time the oracle's restatement of the reference's torch CPU path (fake-quant dequant-then-matmul
    expert loop) on a bounded sample of the workload.  Returns (tflops, seconds, sample description)."""
    from oracle import quant as oq
    from oracle import hadamard as oh
    from mxmoe_b200 import workload
    torch.set_num_threads(threads)
    ids, _ = workload.make_routing(spec)
    gu_s, dn_s = workload.draw_schemes(spec)
    signs = workload.rotation_signs(spec)
    srt, order = torch.sort(ids.reshape(-1).long(), stable=True)
    tok = order // spec.topk
    counts = torch.bincount(srt, minlength=spec.num_experts).tolist()
    hidden = workload.make_hidden(spec)
    x = oh.hadamard_rows(hidden.float() * signs.float()).half() if signs is not None else hidden

    def run_expert(e, rows):
        wgu, wdn = workload.expert_weights_fp16(spec, e)
        if signs is not None:
            wgu = workload.rotate_rows(wgu, signs)
        xe = x[rows]
        t0 = time.perf_counter()
        y1 = oq.fake_quant_expert_loop([xe], [wgu], [gu_s[e]])[0]
        i = wdn.shape[1]
        h = torch.nn.functional.silu(y1[:, :i].float()).half() * y1[:, i:]
        oq.fake_quant_expert_loop([h], [wdn], [dn_s[e]])
        dt = time.perf_counter() - t0
        return dt, 2 * len(rows) * (wgu.numel() + wdn.numel())

    # coldest experts first: many small problems, like the tail of the real workload, then hotter ones
    order_e = sorted(range(spec.num_experts), key=lambda e: counts[e])
    starts = [0]
    for c in counts:
        starts.append(starts[-1] + c)
    total_t, total_f, used, rows_used = 0.0, 0, [], 0
    run_expert(order_e[0], tok[starts[order_e[0]]:starts[order_e[0]] + max(1, counts[order_e[0]])])  # warm-up
    for e in order_e:
        if counts[e] == 0:
            continue
        dt, fl = run_expert(e, tok[starts[e]:starts[e] + counts[e]])
        total_t += dt
        total_f += fl
        used.append(e)
        rows_used += counts[e]
        if total_t >= budget_s:
            break
    desc = (f"{len(used)} of {spec.num_experts} experts ({rows_used} of {sum(counts)} routed rows, coldest first), "
            f"gate_up + silu*mul + down, weights generated outside the timed region")
    return total_f / total_t / 1e12, total_t, desc


def config_of(spec, world: int) -> dict:
    """The workload description both arms print (identical for the same command line)."""
    return {"workload": spec.name, "tokens_per_gpu": spec.tokens, "experts": spec.num_experts, "topk": spec.topk,
            "hidden": spec.hidden, "inter": spec.inter, "shared_inter": spec.shared_inter, "scheme": spec.scheme,
            "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": "operands+outputs per step (>700 MB) exceed the 126 MB L2; no explicit flush"}


def run_reference_arm(args, spec):
    """`--impl reference`: the reference's CPU implementation of the path on the host cores.

    The reference's torch code cannot travel to the GPU box, so the arm runs the oracle's port of it
    (oracle/quant.py: fake-quant dequant-then-matmul expert loop), with all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals = []
    for i in range(args.warmup + args.steps):
        tf, secs, desc = cpu_expert_loop(spec, budget_s=max(1.0, 60.0 / max(1, args.steps + args.warmup)), threads=threads)
        if i >= args.warmup:
            vals.append((tf, secs))
    tf = sum(v[0] for v in vals) / len(vals)
    ms = sum(v[1] for v in vals) / len(vals) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_of(spec, args.gpus),
        "note": "CPU port of the reference torch path (fake-quant dequant-then-matmul expert loop)",
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def ncu_traffic(workload_name: str):
    """DRAM bytes (read + write) per launch of the grouped GEMM, mean of the gate_up and the down launch, from the
    table of ncu captures kept beside the profile summaries (one line per workload and launch); None if the
    workload has no capture."""
    path = os.path.join(ROOT, "profiles", "ncu_dram_traffic.txt")
    vals = []
    if os.path.exists(path):
        with open(path) as f:
            for ln in f:
                parts = ln.split()
                if len(parts) >= 4 and not ln.startswith("#") and parts[0] == workload_name:
                    vals.append(float(parts[3]))
    return sum(vals) / len(vals) if vals else None


def problem_bytes(m: int, n: int, k: int, w, fused_silu: bool = False) -> float:
    """Algorithmic bytes of one problem: A at a_bits per value, the packed weight with its scales, fp16 C and the
    per-token scales (activations of 4-bit schemes count half a byte per code, whatever the layer stores).  A
    gate_up problem with silu(gate) * up in its epilogue writes n / 2 columns."""
    a_bits = w.qparams[0]
    return m * k * a_bits / 8 + w.nbytes() + m * (n // 2 if fused_silu else n) * 2 + (m * 2 if a_bits < 16 else 0)


def class_pass(layer, spec, counts, peaks, reps: int = 10, only: str | None = None):
    """Per-class roofline of the grouped GEMM: every (expert, linear block) problem is classified compute- or
    memory-bound from its algorithmic flops and bytes against the measured peaks, and each class's problem
    subset is launched alone (the other problems' device-side row counts zeroed) and timed with CUDA events."""
    core, E, T = layer._core, spec.num_experts, spec.tokens
    orig = layer.counts.clone()
    has_shared = bool(spec.shared_inter) and hasattr(core, "shared_m")
    bw = peaks["hbm_gbs"] * 1e9
    out = {}
    for cls in ("compute", "memory"):
        out[cls] = {"flops": 0.0, "bytes": 0.0, "ms": 0.0, "problems": 0, "peak_flops_weighted": 0.0}
    try:
        for gg, block, n, k, ns, ks in ((core.gg1, layer.gate_up, 2 * spec.inter, spec.hidden, 2 * spec.shared_inter, spec.hidden),
                                        (core.gg2, layer.down, spec.hidden, spec.inter, spec.hidden, spec.shared_inter)):
            mask = {"compute": [0] * (E + 1), "memory": [0] * (E + 1)}
            for e in range(E + (1 if has_shared else 0)):
                m = T if e == E else counts[e]
                if m == 0:
                    continue
                w = block[e]
                nn, kk = (ns, ks) if e == E else (n, k)
                a_bits = w.qparams[0]
                peak = peaks["bf16_tflops"] * 1e12 * (2.0 if a_bits < 16 else 1.0)
                fl = 2.0 * m * nn * kk
                by = problem_bytes(m, nn, kk, w, gg is core.gg1 and e != E and getattr(core, "fused_silu", False))
                cls = "compute" if fl / peak > by / bw else "memory"
                mask[cls][e] = 1
                out[cls]["flops"] += fl
                out[cls]["bytes"] += by
                out[cls]["problems"] += 1
                out[cls]["peak_flops_weighted"] += fl * peak / 1e12      # flop-weighted peak of a mixed class
            for cls in ("compute", "memory"):
                if not any(mask[cls]) or (only is not None and cls != only):
                    continue
                layer.counts.copy_(orig * torch.tensor(mask[cls][:E], dtype=orig.dtype, device=orig.device))
                if has_shared:
                    core.shared_m.fill_(T if mask[cls][E] else 0)
                for _ in range(2):
                    gg.run()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    gg.run()
                e1.record()
                torch.cuda.synchronize()
                out[cls]["ms"] += e0.elapsed_time(e1) / reps
    finally:
        layer.counts.copy_(orig)
        if has_shared:
            core.shared_m.fill_(T)
    for cls, o in out.items():
        w = o.pop("peak_flops_weighted")
        if o["ms"] > 0:
            o["peak_tflops"] = w / o["flops"] if o["flops"] else None
            o["tflops"] = o["flops"] / (o["ms"] * 1e-3) / 1e12
            o["gbs"] = o["bytes"] / (o["ms"] * 1e-3) / 1e9
            o["frac"] = o["tflops"] / o["peak_tflops"] if cls == "compute" else o["gbs"] / peaks["hbm_gbs"]
    return out


def build_single(spec, dev):
    from mxmoe_b200 import workload
    from mxmoe_b200.layer import MoELayer
    gate_up, down, signs, _ = workload.build_layer_weights(spec, gen_device=dev, device=dev)
    return MoELayer(spec.num_experts, spec.topk, spec.hidden, spec.inter, gate_up, down, spec.tokens,
                    shared_inter=spec.shared_inter, signs=signs, rotate=spec.rotate, device=dev)


def gemm_launch_ms(layer, step_eager, steps: int):
    """CUDA events on the launching stream around the two grouped-GEMM launches of `steps` eager steps."""
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    core = layer._core
    gg1_run, gg2_run = core.gg1.run, core.gg2.run
    state = {"i": 0}

    def timed_gg1():
        e = ev[state["i"]]
        e[0].record(); gg1_run(); e[1].record()

    def timed_gg2():
        e = ev[state["i"]]
        e[2].record(); gg2_run(); e[3].record()
    core.gg1.run, core.gg2.run = timed_gg1, timed_gg2
    try:
        for i in range(steps):
            state["i"] = i
            step_eager()
        torch.cuda.synchronize()
    finally:
        core.gg1.run, core.gg2.run = gg1_run, gg2_run
    d1 = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
    d2 = sum(e[2].elapsed_time(e[3]) for e in ev) / steps
    return d1, d2


def roofline_of(layer, spec, counts, d1, d2, peaks):
    """Roofline entry of the dominant kernel (the persistent grouped GEMM, two launches per step)."""
    flops_launch = spec.flops() / 2
    gemm_ms = (d1 + d2) / 2
    # flop-weighted tensor peak: kind::i8 problems against twice the measured bf16 rate, kind::f16 ones against it
    fl_i8 = fl_all = 0.0
    byts = 0.0
    for block, n, k, ns, ks in ((layer.gate_up, 2 * spec.inter, spec.hidden, 2 * spec.shared_inter, spec.hidden),
                                (layer.down, spec.hidden, spec.inter, spec.hidden, spec.shared_inter)):
        for e, w in block.items():
            m = spec.tokens if e == spec.num_experts else counts[e]
            if m == 0:
                continue
            nn, kk = (ns, ks) if e == spec.num_experts else (n, k)
            fl = 2.0 * m * nn * kk
            fl_all += fl
            if w.qparams[0] < 16:
                fl_i8 += fl
            byts += problem_bytes(m, nn, kk, w, block is layer.gate_up and e != spec.num_experts and
                                  getattr(layer._core, "fused_silu", False))
    share_i8 = fl_i8 / fl_all if fl_all else 0.0
    peak = peaks["bf16_tflops"] * (1.0 + share_i8)
    achieved = flops_launch / (gemm_ms * 1e-3) / 1e12
    bytes_launch = byts / 2
    return {
        "bound": "tensor", "kernel": "gg_swap_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak, "traffic": ncu_traffic(spec.name),
        "peak_source": (f"{peaks['source']} cuBLAS bf16 burst, x2 for the {share_i8:.0%} of the flops that run as "
                        "tcgen05 kind::i8 (twice the bf16 issue rate)"),
        "launch_ms": {"gate_up": d1, "down": d2},
        "algorithmic_flops_per_launch": flops_launch,
        "algorithmic_bytes_per_launch": bytes_launch,
        "hbm_gbs_at_algorithmic_bytes": bytes_launch / (gemm_ms * 1e-3) / 1e9,
        "hbm_peak_gbs": peaks["hbm_gbs"],
    }


def parity_single(layer) -> dict:
    """Correctness of the workload that is about to be timed: the layer's buffers after one step against plain
    torch arithmetic (mxmoe_b200.verify), for the hottest, a median and the coldest expert and the shared expert."""
    from mxmoe_b200 import verify
    rep = verify.check_layer(layer)
    worst = max([p.get("rel_l2", 0.0) for p in rep["problems"]] + [0.0])
    return {"ok": rep["ok"], "checked": len(rep["problems"]),
            "int_accumulators_bit_exact": all(p.get("acc_mismatch", 0) == 0 for p in rep["problems"]),
            "int_outputs_bit_exact": all(p.get("out_mismatch", 0) == 0 for p in rep["problems"]),
            "fp_worst_rel_l2": worst,
            "experts": sorted({p["expert"] for p in rep["problems"]}),
            "against": "torch fp64 product of the codes / fp16 operands found in the layer's device buffers"}


def extra_workload(name: str, dev, peaks, steps: int = 5, warmup: int = 3) -> dict:
    """A few steps of another benchmark configuration on one GPU: step time, GEMM launch times, per-class roofline,
    parity.  The layer is built, measured and freed."""
    from mxmoe_b200 import workload
    spec = workload.CONFIGS[name]
    layer = build_single(spec, dev)
    ids, wts = workload.make_routing(spec)
    hidden = workload.make_hidden(spec).to(dev)
    ids_d, wts_d = ids.to(dev), wts.to(dev)
    for _ in range(warmup):
        layer.forward_graph(hidden, ids_d, wts_d)
    layer.check()
    par = parity_single(layer)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    for _ in range(steps):
        layer.forward_graph(hidden, ids_d, wts_d)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    d1, d2 = gemm_launch_ms(layer, lambda: layer.forward(hidden, ids_d, wts_d), steps)
    counts = layer.counts.cpu().tolist()
    res = {"ms_per_step": ms, "tflops": spec.flops() / (ms * 1e-3) / 1e12,
           "tokens_per_s": spec.tokens / (ms * 1e-3),
           "gemm_only_tflops": spec.flops() / ((d1 + d2) * 1e-3) / 1e12,
           "roofline": roofline_of(layer, spec, counts, d1, d2, peaks), "steps": steps, "parity": par,
           "config": config_of(spec, 1)}
    res["roofline"]["classes"] = class_pass(layer, spec, counts, peaks, reps=5)
    layer.check()
    del layer
    torch.cuda.empty_cache()
    return res


EXTRA_WORKLOADS = ("qwen15-mixed-8192", "ds2lite-w4a16-8192", "ds2lite-w4a16-32", "mixtral-mixed-16384")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="qwen15-w4a4-8192")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work for cpu_baseline")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-extra", action="store_true", help="skip the short runs of the other benchmark configurations")
    ap.add_argument("--no-parity", action="store_true", help="skip the correctness check of the timed workload")
    ap.add_argument("--only-class", choices=["compute", "memory"], default=None,
                    help="after the warm-up, launch the two grouped GEMMs over the compute-bound or the memory-bound "
                         "problems alone a few times and exit (the launches an ncu capture of one class looks at)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from mxmoe_b200 import workload
    spec = workload.CONFIGS[args.workload]
    if args.impl == "reference":
        return run_reference_arm(args, spec)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the kernels)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from mxmoe_b200 import _lib
    _lib.lib()  # fail loudly if the CUDA library is missing
    peaks = load_peaks()

    T = spec.tokens                       # tokens per rank (weak scaling: the global batch is T * world)
    ids, wts = workload.make_routing(spec, seed=2 + rank)
    hidden_host = workload.make_hidden(spec, seed=1 + rank).pin_memory()
    ids_host, wts_host = ids.pin_memory(), wts.pin_memory()
    out_host = torch.empty((T, spec.hidden), dtype=torch.float16).pin_memory()

    if world > 1:
        from mxmoe_b200.ep import EPMoELayer
        layer = EPMoELayer(spec, dev, gen_device=dev)
    else:
        layer = build_single(spec, dev)
    hidden = hidden_host.to(dev, non_blocking=True)
    ids_d, wts_d = ids_host.to(dev, non_blocking=True), wts_host.to(dev, non_blocking=True)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    use_graph = not args.no_graph and hasattr(layer, "forward_graph")

    def step_eager():
        return layer.forward(hidden, ids_d, wts_d)

    def step_resident():
        return layer.forward_graph(hidden, ids_d, wts_d) if use_graph else step_eager()

    # ---- warm-up, correctness of what is about to be timed
    for _ in range(args.warmup):
        step_resident()
    layer.check()
    parity = None
    if not args.no_parity:
        if world == 1:
            parity = parity_single(layer)
        else:
            # every rank: the expert-parallel output for its own tokens must be the bits a single-GPU layer holding
            # ALL experts returns for the same tokens
            import torch.distributed as dist
            out_ep = step_resident().clone()
            full = build_single(spec, dev)
            out_full = full.forward(hidden, ids_d, wts_d)
            full.check()
            same = torch.tensor([1.0 if torch.equal(out_ep, out_full.view_as(out_ep)) else 0.0], device=dev)
            single = parity_single(full)
            ok_local = torch.tensor([1.0 if single["ok"] else 0.0], device=dev)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            dist.all_reduce(ok_local, op=dist.ReduceOp.MIN)
            parity = {"ok": bool(same.item()) and bool(ok_local.item()),
                      "ep_output_bit_equal_to_single_gpu_layer_on_every_rank": bool(same.item()),
                      "single_gpu_layer": single, "replicated_experts": bool(layer.replicated),
                      "virtual_experts": layer.E}
            del full, out_full
            torch.cuda.empty_cache()

    if args.only_class and world == 1:
        counts = layer.counts.cpu().tolist()
        res = class_pass(layer, spec, counts, peaks, reps=3, only=args.only_class)
        print(json.dumps({"only_class": args.only_class, **res[args.only_class]}), flush=True)
        return

    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        step_resident()
    t1.record()
    barrier()
    clocks = sampler.stop()
    ms_total = t0.elapsed_time(t1)
    layer.check()

    # ---- per-launch timing of the dominant kernel (grouped GEMM): the same steps launched eagerly, with
    # CUDA events on the launching stream around the two GEMM launches of every step
    if world == 1:
        d1, d2 = gemm_launch_ms(layer, step_eager, args.steps)

    # ---- end-to-end through the public API with host buffers (H2D of inputs + D2H of the result inside):
    # the public serving loop over host buffers (mxmoe_b200.layer.HostPipeline): per step the host -> device copy of
    # the step's inputs from pinned memory, the layer pass and the device -> host copy of its result; copies of
    # neighbouring steps overlap the compute on their own streams
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(args.steps, 200))
    from mxmoe_b200.layer import HostPipeline
    pipe = HostPipeline(layer, T, spec.hidden, spec.topk, device=dev, use_graph=use_graph,
                        inputs=(hidden, ids_d, wts_d))
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]

    def step_e2e(i):
        pipe.submit(hidden_host, ids_host, wts_host, out_hosts[i & 1])
    for i in range(4):
        step_e2e(i)
    pipe.drain()
    barrier()
    e0.record()
    for i in range(e2e_steps):
        step_e2e(i)
    pipe.drain()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    # ---- aggregate over ranks (max time)
    counts = layer.counts.cpu().tolist() if world == 1 else None
    flops_rank = spec.flops()             # every rank contributes T tokens worth of routed + shared work
    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = times.tolist()
    ms_step = ms_total / args.steps
    value = flops_rank * world / (ms_step * 1e-3) / 1e12
    e2e_value = flops_rank * world / (ms_e2e / e2e_steps * 1e-3) / 1e12

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8" if "a4" in spec.scheme or "a8" in spec.scheme else ("f16" if spec.scheme != "mixed5" else "i8+f16"),
        "data": "synthetic",
        "tokens_per_s": T * world / (ms_step * 1e-3),
        "config": config_of(spec, world),
        "launch": "cuda-graph replay" if use_graph else "eager",
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": hidden_host.numel() * 2 + ids_host.numel() * 4 + wts_host.numel() * 4,
                "d2h_bytes_per_step": out_host.numel() * 2, "steps": e2e_steps, "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": args.steps * layer.launches_per_step,
        "parity": parity,
    }

    if world > 1:
        # where the step goes: CUDA-event times of the phases of a few profiled steps (mean over steps, max and mean
        # over ranks) and the rows every rank's experts received
        import torch.distributed as dist
        if hasattr(layer, "phase_ms"):
            layer.profile, layer.phase_ms = True, {}
            for _ in range(5):
                step_eager()
            layer.profile = False
            names = list(layer.phase_ms)
            mine = torch.tensor([sum(layer.phase_ms[n]) / len(layer.phase_ms[n]) for n in names], dtype=torch.float64, device=dev)
            mx, sm = mine.clone(), mine.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            line["phases_ms"] = {n: {"max": mx[i].item(), "mean": sm[i].item() / world} for i, n in enumerate(names)}
            line["phases_note"] = "eager steps with an event and a host synchronisation per phase"
        if hasattr(layer, "total_recv"):
            rows = torch.zeros(world, dtype=torch.float64, device=dev)
            rows[rank] = float(layer.total_recv[0].item())
            dist.all_reduce(rows)
            r = rows.tolist()
            line["rows_per_rank"] = {"max": max(r), "mean": sum(r) / world, "max_over_mean": max(r) / (sum(r) / world)}

    if world == 1:
        # dominant kernel: the persistent grouped GEMM (2 launches per step)
        line["roofline"] = roofline_of(layer, spec, counts, d1, d2, peaks)
        line["gemm_only_tflops"] = flops_rank / ((d1 + d2) * 1e-3) / 1e12
        # compute-bound and memory-bound problems timed apart (each class's problems launched alone)
        line["roofline"]["classes"] = class_pass(layer, spec, counts, peaks)
        if not args.no_extra:
            del layer, pipe
            torch.cuda.empty_cache()
            line["workloads"] = {}
            for name in EXTRA_WORKLOADS:
                if name != spec.name:
                    line["workloads"][name] = extra_workload(name, dev, peaks)
        if not args.no_cpu and rank == 0:
            threads = os.cpu_count() or 1
            tf, secs, desc = cpu_expert_loop(spec, args.cpu_budget, threads)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc,
                                    "seconds": secs}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
