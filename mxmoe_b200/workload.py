"""Seeded synthetic MoE layers with the shapes, routing skew and value
distributions of the benchmark configurations, plus the reference's workload
JSON format.

Real checkpoints and recorded gate traces are not available offline, so weights
are ``N(0, 0.02)``, activations ``N(0, 1)`` (optionally with 1 % outlier channels
scaled x20) and routing is drawn from a seeded Zipf or biased-softmax
distribution.  The workload JSON written by :func:`workload_json` has the schema
of ``mxmoe/kernels/gen_workload.py:86-101``.
"""
from __future__ import annotations

import dataclasses
import json

import torch

from .weights import PackedWeight, prepare_weight, weight_bits, parse_scheme


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    name: str
    num_experts: int
    topk: int
    hidden: int
    inter: int
    shared_inter: int = 0          # fused intermediate size of the shared expert(s); 0 = none
    tokens: int = 8192
    routing: str = "zipf"          # "zipf" | "softmax_biased"
    zipf_s: float = 1.2
    outliers: bool = False         # 1 % of activation channels scaled x20
    rotate: bool = False           # Hadamard-rotate activations / gate_up weights over the hidden dim
    scheme: str = "w4a4_g-1_sym"   # uniform scheme, or "mixed5" / "mixed_w8w4"

    def flops(self, rows_routed: int | None = None) -> int:
        r = self.tokens * self.topk if rows_routed is None else rows_routed
        f = 2 * r * (2 * self.inter * self.hidden + self.hidden * self.inter)
        if self.shared_inter:
            f += 2 * self.tokens * (2 * self.shared_inter * self.hidden + self.hidden * self.shared_inter)
        return f


# the five benchmark configurations
CONFIGS = {
    "qwen15-w4a4-512": LayerSpec("qwen15-w4a4-512", 60, 4, 2048, 1408, 0, 512, "zipf", 1.2, False, True,
                                 "w4a4_g-1_sym"),
    "qwen15-w4a4-8192": LayerSpec("qwen15-w4a4-8192", 60, 4, 2048, 1408, 0, 8192, "zipf", 1.2, True, True,
                                  "w4a4_g-1_sym"),
    "qwen15-mixed-8192": LayerSpec("qwen15-mixed-8192", 60, 4, 2048, 1408, 5632, 8192, "zipf", 1.2, True, True,
                                   "mixed5"),
    "ds2lite-w4a16-8192": LayerSpec("ds2lite-w4a16-8192", 64, 6, 2048, 1408, 2816, 8192, "zipf", 1.0, False, False,
                                    "w4a16_g128_asym"),
    "ds2lite-w4a16-32": LayerSpec("ds2lite-w4a16-32", 64, 6, 2048, 1408, 2816, 32, "zipf", 1.0, False, False,
                                  "w4a16_g128_asym"),
    "mixtral-mixed-16384": LayerSpec("mixtral-mixed-16384", 8, 2, 4096, 14336, 0, 16384, "softmax_biased", 0.0, True,
                                     True, "mixed_w8w4"),
}


def _gen(seed: int, device="cpu") -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def make_routing(spec: LayerSpec, seed: int = 2, tokens: int | None = None):
    """``(topk_ids int32 [T,k], topk_weights fp32 [T,k])`` drawn on the CPU from a seeded generator."""
    t = spec.tokens if tokens is None else tokens
    g = _gen(seed)
    if spec.routing == "zipf":
        p = torch.arange(1, spec.num_experts + 1, dtype=torch.float64).pow(-spec.zipf_s)
        p = p / p.sum()
        ids = torch.multinomial(p.expand(t, -1), spec.topk, replacement=False, generator=g)
        w = p[ids]
        w = (w / w.sum(dim=-1, keepdim=True)).float()
    elif spec.routing == "softmax_biased":
        logits = torch.randn(t, spec.num_experts, generator=g)
        logits[:, 0] += 1.0
        prob = logits.softmax(dim=-1)
        w, ids = prob.topk(spec.topk, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).float()
    else:
        raise ValueError(spec.routing)
    return ids.to(torch.int32), w


def make_hidden(spec: LayerSpec, seed: int = 1, tokens: int | None = None, device="cpu") -> torch.Tensor:
    t = spec.tokens if tokens is None else tokens
    g = _gen(seed, device)
    x = torch.randn(t, spec.hidden, generator=g, device=device)
    if spec.outliers:
        ch = torch.randperm(spec.hidden, generator=_gen(seed + 100))[: max(1, spec.hidden // 100)]
        x[:, ch.to(x.device)] *= 20.0
    return x.half()


def rotation_signs(spec: LayerSpec, seed: int = 4) -> torch.Tensor | None:
    """+-1 diagonal of the random Hadamard rotation over the hidden dim (int8), or None."""
    if not spec.rotate:
        return None
    s = torch.randint(0, 2, (spec.hidden,), generator=_gen(seed)) * 2 - 1
    return s.to(torch.int8)


def fwht_rows(x: torch.Tensor) -> torch.Tensor:
    """Un-normalised natural-order Walsh-Hadamard transform over the last dim (power of two)."""
    n = x.shape[-1]
    assert n & (n - 1) == 0
    y = x.reshape(-1, n)
    h = 1
    while h < n:
        v = y.reshape(-1, n // (2 * h), 2, h)
        y = torch.stack((v[:, :, 0, :] + v[:, :, 1, :], v[:, :, 0, :] - v[:, :, 1, :]), dim=2).reshape(-1, n)
        h *= 2
    return y.reshape(x.shape)


def rotate_rows(w: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """``W <- W Q`` with ``Q = diag(signs) H / sqrt(n)`` over the last dim, evaluated in fp64
    (the offline weight rotation of rotation.py:353-358), returned as fp16."""
    n = w.shape[-1]
    y = fwht_rows(w.double() * signs.to(w.device).double()) / torch.tensor(n).sqrt().to(w.device)
    return y.half()


def draw_schemes(spec: LayerSpec, seed: int = 3) -> tuple[list[str], list[str]]:
    """Scheme of every (expert, block): ``(gate_up_schemes, down_schemes)``; the shared expert, if any, is last."""
    n_all = spec.num_experts + (1 if spec.shared_inter else 0)
    if spec.scheme == "mixed5":
        # one scheme per (expert, block); parameter-weighted mean of effective weight bits = 5.0 +- 0.02
        blocks = [(e, b) for e in range(n_all) for b in ("gate_up", "down")]
        params = []
        for e, b in blocks:
            i = spec.shared_inter if e == spec.num_experts else spec.inter
            params.append((2 if b == "gate_up" else 1) * i * spec.hidden)
        order = torch.randperm(len(blocks), generator=_gen(seed)).tolist()
        names = ["w4a4_g-1_sym", "w4a16_g128_asym", "w8a8_g-1_sym", "fp16"]
        frac = [0.575, 0.25, 0.145, 0.03]
        total = float(sum(params))
        assign = [None] * len(blocks)
        ci, acc = 0, 0.0
        bounds = [sum(frac[: i + 1]) for i in range(4)]
        for idx in order:
            while ci < 3 and acc / total >= bounds[ci]:
                ci += 1
            assign[idx] = names[ci]
            acc += params[idx]
        # all four schemes must be present: the last three blocks in draw order carry the rare ones if missing
        for j, nm in enumerate(names[1:]):
            if nm not in assign:
                assign[order[-1 - j]] = nm

        def mean_bits():
            return sum(weight_bits(a) * p for a, p in zip(assign, params)) / total
        # greedy repair towards 5.0 by flipping w4a4 <-> w8a8 on the smallest blocks, last drawn first
        for idx in reversed(order):
            m = mean_bits()
            if abs(m - 5.0) <= 0.02:
                break
            if m > 5.0 and assign[idx] == "w8a8_g-1_sym" and assign.count("w8a8_g-1_sym") > 1:
                assign[idx] = "w4a4_g-1_sym"
            elif m < 5.0 and assign[idx] == "w4a4_g-1_sym" and assign.count("w4a4_g-1_sym") > 1:
                assign[idx] = "w8a8_g-1_sym"
                if mean_bits() - 5.0 > 0.02:
                    assign[idx] = "w4a4_g-1_sym"
        gu = [assign[2 * e] for e in range(n_all)]
        dn = [assign[2 * e + 1] for e in range(n_all)]
        return gu, dn
    if spec.scheme == "mixed_w8w4":
        pick = torch.randint(0, 2, (n_all,), generator=_gen(seed)).tolist()
        s = ["w8a8_g-1_sym" if p else "w4a4_g-1_sym" for p in pick]
        if len(set(s)) == 1:
            s[0] = "w8a8_g-1_sym" if s[0] == "w4a4_g-1_sym" else "w4a4_g-1_sym"
        return s, list(s)
    return [spec.scheme] * n_all, [spec.scheme] * n_all


def mean_weight_bits(spec: LayerSpec, gu: list[str], dn: list[str]) -> float:
    tot = bits = 0.0
    for e, (a, b) in enumerate(zip(gu, dn)):
        i = spec.shared_inter if e == spec.num_experts else spec.inter
        bits += weight_bits(a) * 2 * i * spec.hidden + weight_bits(b) * i * spec.hidden
        tot += 3 * i * spec.hidden
    return bits / tot


def expert_weights_fp16(spec: LayerSpec, e: int, seed: int = 1000, device="cpu"):
    """``(W_gate_up [2I, H], W_down [H, I])`` of expert ``e`` (``e == num_experts``: the shared expert)."""
    i = spec.shared_inter if e == spec.num_experts else spec.inter
    g = _gen(seed + e, device)
    wgu = (torch.randn(2 * i, spec.hidden, generator=g, device=device) * 0.02).half()
    wdn = (torch.randn(spec.hidden, i, generator=g, device=device) * 0.02).half()
    return wgu, wdn


def build_layer_weights(spec: LayerSpec, experts=None, seed: int = 1000, scheme_seed: int = 3, sign_seed: int = 4,
                        gen_device="cpu", device="cpu", keep_codes: bool = False, online_had=None):
    """Quantised + packed weights of the layer: ``(gate_up: dict e -> PackedWeight, down: dict, signs, (gu, dn))``.

    ``experts`` restricts the routed experts that are materialised (expert parallelism);
    the shared expert, if the layer has one, is always included under key ``num_experts``.
    With ``spec.rotate`` every gate_up weight is rotated over the hidden dim offline (``W Q``), whatever
    its scheme, and the activation prologue rotates every row (``x Q``), as in a rotated model where
    the residual stream itself is rotated.  ``online_had`` (a K x K Hadamard factor, ``inter = K * m``): the down
    weights of the routed experts are rotated over their input dimension offline, for a layer that rotates the
    down-projection input online (apply_exact_had_to_linear + the hook of rotation.py:403-421).
    """
    gu_s, dn_s = draw_schemes(spec, scheme_seed)
    signs = rotation_signs(spec, sign_seed)
    ids = list(range(spec.num_experts)) if experts is None else list(experts)
    if spec.shared_inter:
        ids.append(spec.num_experts)
    gate_up, down = {}, {}
    for e in ids:
        wgu, wdn = expert_weights_fp16(spec, e, seed, gen_device)
        if signs is not None:
            wgu = rotate_rows(wgu, signs)
        if online_had is not None and e < spec.num_experts:
            from .hadamard import rotate_rows_kron
            wdn = rotate_rows_kron(wdn, online_had)
        gate_up[e] = prepare_weight(wgu, gu_s[e], keep_codes).to(device)
        down[e] = prepare_weight(wdn, dn_s[e], keep_codes).to(device)
    return gate_up, down, signs, (gu_s, dn_s)


def workload_json(spec: LayerSpec, counts: list[int], gu: list[str], dn: list[str], layer: int = 0) -> str:
    """Problem list in the reference's workload format (gen_workload.py:86-101)."""
    def q(name):
        a, w, g, sym = parse_scheme(name)
        return {"w_bits": w, "a_bits": a, "gsize": g, "sym": sym}
    shapes = {"gate_up": [], "down": []}
    for e, m in enumerate(counts):
        shapes["gate_up"].append({"shape": [int(m), spec.inter * 2, spec.hidden], **q(gu[e])})
        shapes["down"].append({"shape": [int(m), spec.hidden, spec.inter], **q(dn[e])})
    if spec.shared_inter:
        e = spec.num_experts
        shapes["gate_up"].append({"shape": [spec.tokens, spec.shared_inter * 2, spec.hidden], **q(gu[e])})
        shapes["down"].append({"shape": [spec.tokens, spec.hidden, spec.shared_inter], **q(dn[e])})
    return json.dumps({"num_tokens": spec.tokens, f"layer-{layer}": shapes}, indent=2)
