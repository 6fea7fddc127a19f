"""ctypes binding of ``libmxmoe_b200.so`` (the C ABI declared in ``include/mxmoe_b200.h``).

There is no fallback: if the shared library is missing, or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmxmoe_b200.so")

# every symbol include/mxmoe_b200.h declares
EXPORTS = (
    "mxmoe_last_error", "mxmoe_version", "mxmoe_device_sm_count",
    "mxmoe_gg_workspace_bytes", "mxmoe_gg_prepare", "mxmoe_gg_run", "mxmoe_gg_run_kernel", "mxmoe_ep_plan", "mxmoe_ep_sync", "mxmoe_ep_dispatch_rows", "mxmoe_gate_topk", "mxmoe_gg_launch", "mxmoe_gg_check", "mxmoe_gg_profile", "mxmoe_gg_debug",
    "mxmoe_groupgemm_hz_fused", "mxmoe_quant_act", "mxmoe_quant_tokens", "mxmoe_gather_rows", "mxmoe_quant_tokens_scatter",
    "mxmoe_silu_mul_then_quant", "mxmoe_hadamard_kron",
    "mxmoe_route_workspace_bytes", "mxmoe_route_topk", "mxmoe_route_topk_static", "mxmoe_combine_topk", "mxmoe_fetch_host",
)


class MxMoEError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"mxmoe_b200 status {status}: {message}")
        self.status = status


class QParams(C.Structure):
    _fields_ = [("a_bits", C.c_int32), ("w_bits", C.c_int32), ("gsize", C.c_int32),
                ("sym", C.c_uint8), ("pad_", C.c_uint8 * 3)]


class GGProblem(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("scale_a", C.c_void_p), ("scale_b", C.c_void_p), ("C", C.c_void_p),
        ("m_dev", C.c_void_p), ("row0_dev", C.c_void_p),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("a_rows", C.c_int32), ("row0", C.c_int32), ("ldc", C.c_int32),
        ("q", QParams), ("out_mode", C.c_int32), ("lda_bytes", C.c_int32), ("sa_stride", C.c_int32),
        ("a_expanded", C.c_int32), ("reserved_", C.c_int32), ("c_row0_dev", C.c_void_p), ("c_row_ptrs", C.c_void_p),
    ]


class GGPlan(C.Structure):
    _fields_ = [("count", C.c_int32), ("needs_cvt", C.c_int32), ("flags", C.c_int32), ("kernel", C.c_int32)]


class EpPlanArgs(C.Structure):
    _fields_ = [
        ("counts_all", C.c_void_p), ("range_lo", C.c_void_p),
        ("world", C.c_int32), ("rank", C.c_int32), ("num_experts", C.c_int32), ("experts_local", C.c_int32),
        ("recv_capacity", C.c_int32), ("layout", C.c_int32),
        ("seg_m", C.c_void_p), ("seg_row0", C.c_void_p), ("seg_src_row0", C.c_void_p), ("recv_row_expert", C.c_void_p),
        ("total_recv", C.c_void_p), ("dst_row0", C.c_void_p), ("exp_owner", C.c_void_p),
        ("exp_m", C.c_void_p), ("exp_row0", C.c_void_p), ("row_dst", C.c_void_p), ("peer_ret", C.c_void_p),
        ("ret_row_bytes", C.c_int32), ("reserved_", C.c_int32),
    ]


class EpSyncArgs(C.Structure):
    _fields_ = [("peer_sync", C.c_void_p), ("local_sync", C.c_void_p), ("payload", C.c_void_p),
                ("world", C.c_int32), ("rank", C.c_int32), ("payload_len", C.c_int32), ("payload_cap", C.c_int32),
                ("timeout_ms", C.c_int32), ("reserved_", C.c_int32)]


class EpDispatchArgs(C.Structure):
    _fields_ = [
        ("peer_base", C.c_void_p), ("row_expert", C.c_void_p), ("row_token", C.c_void_p), ("exp_row_start", C.c_void_p),
        ("exp_qtag", C.c_void_p), ("dst_row0", C.c_void_p), ("exp_owner", C.c_void_p),
        ("rows", C.c_int32), ("k", C.c_int32), ("rec_bytes", C.c_int32), ("scale_off_bytes", C.c_int32),
        ("recv_capacity", C.c_int32), ("reserved_", C.c_int32),
    ]


class ActArgs(C.Structure):
    _fields_ = [
        ("inp", C.c_void_p), ("in_shared", C.c_void_p), ("q_store", C.c_void_p), ("s_store", C.c_void_p),
        ("row_expert", C.c_void_p), ("row_token", C.c_void_p),
        ("exp_qtag", C.c_void_p), ("exp_row_start", C.c_void_p), ("exp_q_off", C.c_void_p), ("exp_s_off", C.c_void_p),
        ("signs", C.c_void_p),
        ("k", C.c_int32), ("k_shared", C.c_int32), ("rows_routed", C.c_int32), ("rows_total", C.c_int32),
        ("num_experts", C.c_int32), ("rotate", C.c_int32), ("rec_stride", C.c_int32), ("rec_scale_off", C.c_int32),
        ("rows_dev", C.c_void_p),
    ]


class TokenQuantArgs(C.Structure):
    _fields_ = [
        ("inp", C.c_void_p), ("f16", C.c_void_p), ("q8", C.c_void_p), ("s8", C.c_void_p), ("q4", C.c_void_p),
        ("s4", C.c_void_p), ("q4x", C.c_void_p), ("signs", C.c_void_p),
        ("k", C.c_int32), ("num_tokens", C.c_int32), ("rotate", C.c_int32), ("reserved_", C.c_int32),
    ]


class RouteArgs(C.Structure):
    _fields_ = [
        ("topk_ids", C.c_void_p), ("counts", C.c_void_p), ("row_start", C.c_void_p), ("row_expert", C.c_void_p),
        ("row_token", C.c_void_p), ("slot_row", C.c_void_p), ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("num_tokens", C.c_int32), ("topk", C.c_int32), ("num_experts", C.c_int32), ("num_ids", C.c_int32),
        ("id_map", C.c_void_p), ("rep_base", C.c_void_p), ("rep_count", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m mxmoe_b200.build` "
                "(there is no CPU or PyTorch fallback for the grouped GEMM)")
        l = C.CDLL(LIB_PATH)
        l.mxmoe_last_error.restype = C.c_char_p
        l.mxmoe_gg_workspace_bytes.restype = C.c_size_t
        l.mxmoe_gg_workspace_bytes.argtypes = [C.c_int]
        l.mxmoe_gg_prepare.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
        l.mxmoe_gg_run.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        l.mxmoe_gg_run_kernel.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        l.mxmoe_gg_launch.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        l.mxmoe_gg_check.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_gg_profile.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        l.mxmoe_gg_debug.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        l.mxmoe_groupgemm_hz_fused.argtypes = [C.c_void_p] * 14 + [C.c_int]
        l.mxmoe_quant_act.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_silu_mul_then_quant.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_quant_tokens.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_gather_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        l.mxmoe_quant_tokens_scatter.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        l.mxmoe_hadamard_kron.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
        l.mxmoe_ep_plan.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_ep_sync.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_gate_topk.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        l.mxmoe_ep_dispatch_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        l.mxmoe_route_workspace_bytes.restype = C.c_size_t
        l.mxmoe_route_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
        l.mxmoe_route_topk.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_route_topk_static.argtypes = [C.c_void_p, C.c_void_p]
        l.mxmoe_combine_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int, C.c_int, C.c_int, C.c_void_p]
        l.mxmoe_fetch_host.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        _lib = l
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise MxMoEError(status, lib().mxmoe_last_error().decode("utf-8", "replace"))
