"""Child process of the device-oracle tests: runs the reference's own fused GroupGEMM kernel
(oracle/_ref/libref_gg.so, built by `make -C oracle refgg`) on the seeded cases of tests/ref_cases.py
and writes its fp16 outputs to an .npz file.

Runs in a process of its own because the reference's launcher ends the process on any CUDA error
(mxmoe/kernels/src/include/helper.h:186-198).  Operands are packed by the reference's host packers
(quantize.cuh:299-475, exported by the same library).  Every buffer the kernel reads is padded with
zeros to whole 128-row tiles (+ one tile): the reference's per-token scale load has no row guard
(mm_tile.cuh:826-841).

    python tests/ref_gg_worker.py --out OUT.npz [--schemes fp16,w8a8_g-1_sym,...]
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from tests import ref_cases  # noqa: E402

LIB = os.path.join(ROOT, "oracle", "_ref", "libref_gg.so")
PAD = 128


def vp(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def dev_padded(a: np.ndarray, extra_elems: int) -> torch.Tensor:
    """Copy ``a`` (any 16-bit dtype) to the device followed by ``extra_elems`` zero elements."""
    flat = np.ascontiguousarray(a).view(np.int16).reshape(-1)
    t = torch.zeros(flat.size + extra_elems, dtype=torch.int16, device="cuda")
    t[:flat.size] = torch.from_numpy(flat.copy()).cuda()
    return t


def build(lib, c: dict):
    """Device operands of one case in the reference's layouts; returns (A, B, scale_a, scale_b, C tensors)."""
    scheme, m, n, k = c["scheme"], c["m"], c["n"], c["k"]
    a_bits, w_bits, gsize, sym = ref_cases.QPARAMS[scheme]
    sa = sb = None
    if a_bits < 16:
        # weight + activation scheme: both operands packed along K in one call (quantize.cuh:424-475)
        p = 16 // a_bits
        pa = np.zeros((m, k // p), dtype=np.uint16)
        pb = np.zeros((n, k // p), dtype=np.uint16)
        qa = np.ascontiguousarray(c["qa"], dtype=np.int32)
        qb = np.ascontiguousarray(c["qb"], dtype=np.int32)
        rc = lib.ref_gg_pack_wxax(vp(qa), vp(qb), m, n, k, a_bits, vp(pa), vp(pb))
        assert rc == 0, rc
        A = dev_padded(pa, PAD * (k // p))
        B = dev_padded(pb, 0)
        # group-major scales [groups][rows] (permute_scale, quantize.cuh:299-315)
        sa = dev_padded(np.ascontiguousarray(c["sa"].T), 2 * PAD)
        sb = dev_padded(np.ascontiguousarray(c["sb"].T), 2 * PAD)
    else:
        A = dev_padded(c["a"], PAD * k)
        if w_bits == 16:
            B = dev_padded(c["b"], 0)
        else:
            pb = np.zeros((n // 4, k), dtype=np.uint16)
            qb = np.ascontiguousarray(c["qb"], dtype=np.int32)
            rc = lib.ref_gg_permute_pack_weightonly(vp(qb), n, k, w_bits, sym, vp(pb))
            assert rc == 0, rc
            B = dev_padded(pb, 0)
            sz = np.stack((c["sb"].T, c["zb"].T), axis=-1)      # [groups][N][2] (scale, zero)
            sb = dev_padded(np.ascontiguousarray(sz), 4 * PAD)
    Cbuf = torch.full(((m + PAD) * n,), float("nan"), dtype=torch.float16, device="cuda")
    return A, B, sa, sb, Cbuf


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--schemes", default=",".join(ref_cases.QPARAMS))
    args = ap.parse_args()
    lib = C.CDLL(LIB)
    u64p, i32p = C.POINTER(C.c_uint64), C.POINTER(C.c_int32)
    lib.ref_gg_run.argtypes = [u64p, u64p, u64p, u64p, u64p, i32p, i32p, C.c_int]
    lib.ref_gg_run.restype = C.c_int
    out = {}
    for scheme in args.schemes.split(","):
        idxs = [i for i, cs in enumerate(ref_cases.CASES) if cs[0] == scheme]
        cases = [ref_cases.make(i) for i in idxs]
        bufs = [build(lib, c) for c in cases]
        n = len(cases)
        ptr = lambda j: (C.c_uint64 * n)(*[(b[j].data_ptr() if b[j] is not None else 0) for b in bufs])  # noqa: E731
        sizes = (C.c_int32 * (3 * n))(*[v for c in cases for v in (c["m"], c["n"], c["k"])])
        qp = (C.c_int32 * (4 * n))(*[v for c in cases for v in ref_cases.QPARAMS[c["scheme"]]])
        torch.cuda.synchronize()
        rc = lib.ref_gg_run(ptr(0), ptr(1), ptr(2), ptr(3), ptr(4), sizes, qp, n)
        if rc != 0:
            print(f"ref_gg_run({scheme}) returned {rc}", file=sys.stderr)
            sys.exit(3)
        for i, c, b in zip(idxs, cases, bufs):
            full = b[4].cpu().numpy().reshape(c["m"] + PAD, c["n"])
            assert np.isnan(full[c["m"]:].astype(np.float32)).all(), "the reference kernel wrote beyond row M"
            out[f"c{i}"] = full[:c["m"]].copy()
        np.savez(args.out, **out)          # after every scheme: a later failure keeps the earlier results
        print(f"{scheme}: ok", flush=True)


if __name__ == "__main__":
    main()
