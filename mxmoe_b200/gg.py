"""Grouped-GEMM launcher over torch device tensors.

A :class:`Problem` is one ``C[M,N] = A[M,K] x B[N,K]^T`` with its quantisation
scheme; :class:`GroupedGemm` turns a list of them into a prepared workspace
(TMA descriptors encoded once) that can be launched any number of times on the
current CUDA stream.  Torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Sequence

import torch

from . import _lib

OUT_FP16 = 0
OUT_ACC = 1
OUT_SILU = 2   # B = [gate rows; up rows]: C[M, N/2] = fp16(fp16(silu(gate)) * up) of the scaled results


def _ptr(t) -> int | None:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


@dataclasses.dataclass
class Problem:
    """One problem of a grouped launch; tensors are CUDA tensors (or raw device addresses)."""
    A: object
    B: object
    C: object
    M: int
    N: int
    K: int
    qparams: tuple            # (a_bits, w_bits, gsize, sym) as in the reference's QParams
    scale_a: object = None
    scale_b: object = None
    row0: int = 0
    a_rows: int = 0
    ldc: int = 0
    out_mode: int = OUT_FP16
    m_dev: object = None      # int32 device scalar: live row count
    row0_dev: object = None   # int32 device scalar: first row
    lda_bytes: int = 0        # row pitch of A in bytes (0 = dense)
    sa_stride: int = 0        # distance between per-token scales in elements (0 = contiguous)
    a_expanded: int = 0       # w4a4: activations stored as one byte 16*q per code
    c_row0_dev: object = None  # device pointer (int) to the first row of C, when it differs from the rows of A
    c_row_ptrs: object = None  # int64 device table: address of every result row (indexed like the rows of A)

    def fill(self, c: _lib.GGProblem) -> None:
        a_bits, w_bits, gsize, sym = self.qparams
        c.A, c.B, c.C = _ptr(self.A), _ptr(self.B), _ptr(self.C)
        c.scale_a, c.scale_b = _ptr(self.scale_a), _ptr(self.scale_b)
        c.m_dev, c.row0_dev = _ptr(self.m_dev), _ptr(self.row0_dev)
        c.M, c.N, c.K = int(self.M), int(self.N), int(self.K)
        c.a_rows, c.row0, c.ldc = int(self.a_rows), int(self.row0), int(self.ldc)
        c.q.a_bits, c.q.w_bits, c.q.gsize, c.q.sym = int(a_bits), int(w_bits), int(gsize), 1 if sym else 0
        c.out_mode = int(self.out_mode)
        c.lda_bytes = int(self.lda_bytes)
        c.sa_stride = int(self.sa_stride)
        c.a_expanded = int(self.a_expanded)
        c.c_row0_dev = _ptr(self.c_row0_dev)
        c.c_row_ptrs = _ptr(self.c_row_ptrs)

    def flops(self) -> int:
        return 2 * self.M * self.N * self.K


class GroupedGemm:
    """A prepared grouped launch.  ``run()`` enqueues the persistent kernel on the current stream."""

    MAX_PROBLEMS = 256   # problems one launch can walk (kMaxProblems of the kernels)

    def __init__(self, problems: Sequence[Problem], device=None):
        self.problems = list(problems)   # keeps the operand tensors alive
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._parts = None
        if len(self.problems) > self.MAX_PROBLEMS:
            # the reference launcher takes any problem_count (kernel_sketch.py:82-145); a longer list is walked by
            # several launches of at most MAX_PROBLEMS problems each
            m = self.MAX_PROBLEMS
            self._parts = [GroupedGemm(self.problems[i:i + m], device=self.device) for i in range(0, len(self.problems), m)]
            return
        lib = _lib.lib()
        n = len(self.problems)
        self._arr = (_lib.GGProblem * max(n, 1))()
        for i, p in enumerate(self.problems):
            p.fill(self._arr[i])
        nbytes = lib.mxmoe_gg_workspace_bytes(n)
        self.workspace = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
        base = self.workspace.data_ptr()
        self._ws = (base + 255) & ~255
        self._ws_bytes = nbytes
        self._plan = _lib.GGPlan()
        with torch.cuda.device(self.device):
            _lib.check(lib.mxmoe_gg_prepare(C.byref(self._arr), n, self._ws, nbytes, current_stream_ptr(),
                                            C.byref(self._plan)))

    @property
    def kept(self) -> int:
        if self._parts is not None:
            return sum(p.kept for p in self._parts)
        return self._plan.count

    def set_small_tiles(self, on: bool) -> None:
        """Override the library's choice of token-tile geometry (32-row tiles and a deeper ring: for launches whose
        problems hold few rows each, e.g. a decode batch whose row counts only exist on the device)."""
        if self._parts is not None:
            for p in self._parts:
                p.set_small_tiles(on)
            return
        self._plan.flags = (self._plan.flags | 2) if on else (self._plan.flags & ~2)

    def run(self, num_ctas: int = 0, kernel: str | None = None) -> None:
        """Launch; ``kernel`` in KERNELS names the kernel, None leaves the choice to the library."""
        if self._parts is not None:
            for p in self._parts:
                p.run(num_ctas, kernel)
            return
        with torch.cuda.device(self.device):
            if kernel is None:
                _lib.check(_lib.lib().mxmoe_gg_run(self._ws, C.byref(self._plan), num_ctas, current_stream_ptr()))
            else:
                _lib.check(_lib.lib().mxmoe_gg_run_kernel(self._ws, C.byref(self._plan), KERNELS[kernel], num_ctas,
                                                          current_stream_ptr()))

    def check(self) -> None:
        """Synchronise the current stream and raise if the kernel recorded an error."""
        if self._parts is not None:
            for p in self._parts:
                p.check()
            return
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().mxmoe_gg_check(self._ws, current_stream_ptr()))

    def debug(self, timeout_ms: int = 0, skip_stage: int = -1) -> None:
        """Test hook (mxmoe_gg_debug): shorter limit for the device-side waits; leave out one weight load."""
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().mxmoe_gg_debug(self._ws, timeout_ms, skip_stage, current_stream_ptr()))


KERNELS = {"default": 0, "single": 1, "pair": 2, "swap": 3, "swap2": 4}

PROF_NAMES = ("total", "producer_wait", "mma_wait_operands", "mma_wait_accumulator", "mma_issue", "epilogue_wait",
              "epilogue_store", "converter_wait", "converter_work", "tiles", "stages", "mma_gap")


def profile(g: "GroupedGemm") -> dict:
    """Cycle counters CTA 0 recorded during the last launch of ``g`` (see mxmoe_gg_profile)."""
    buf = (C.c_uint64 * 16)()
    with torch.cuda.device(g.device):
        _lib.check(_lib.lib().mxmoe_gg_profile(g._ws, buf, current_stream_ptr()))
    return {n: int(buf[i]) for i, n in enumerate(PROF_NAMES)}


def grouped_gemm(problems: Sequence[Problem], check: bool = True, num_ctas: int = 0) -> GroupedGemm:
    """Prepare, launch once and (by default) check."""
    g = GroupedGemm(problems)
    g.run(num_ctas)
    if check:
        g.check()
    return g
