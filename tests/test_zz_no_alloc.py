"""Routing through the entry point that owns its scratch memory (``mxmoe_route_topk_static``).

Who needs it: callers that may not allocate device memory at the point where tokens are routed -
for instance a serving loop whose memory pool was sized once at start-up, or a plug-in that is
given input and output buffers by its host and nothing more.  They cannot supply the workspace
``mxmoe_route_topk`` asks for, so this variant keeps the per-block histograms in a fixed array
inside the library.

The test calls it through the C ABI twice in a row with different routings (the second call finds
the first call's histograms still in the shared array) and requires the same integers as the
workspace-taking entry point and as ``torch.sort(stable=True)`` / ``bincount``.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from mxmoe_b200 import _lib
from mxmoe_b200.gg import current_stream_ptr

pytestmark = pytest.mark.gpu


def _route(fn_name, ids, e, dev, with_workspace):
    t, k = ids.shape
    n = t * k
    out = {
        "counts": torch.full((e,), -1, dtype=torch.int32, device=dev),
        "row_start": torch.full((e + 1,), -1, dtype=torch.int32, device=dev),
        "row_expert": torch.full((n,), -1, dtype=torch.int32, device=dev),
        "row_token": torch.full((n,), -1, dtype=torch.int64, device=dev),
        "slot_row": torch.full((n,), -7, dtype=torch.int32, device=dev),
    }
    a = _lib.RouteArgs()
    a.topk_ids = ids.data_ptr()
    for name, tns in out.items():
        setattr(a, name, tns.data_ptr())
    ws = None
    if with_workspace:
        nbytes = _lib.lib().mxmoe_route_workspace_bytes(t, k, e)
        ws = torch.zeros(nbytes // 4 + 1, dtype=torch.int32, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    a.num_tokens, a.topk, a.num_experts = t, k, e
    _lib.check(getattr(_lib.lib(), fn_name)(C.byref(a), current_stream_ptr()))
    torch.cuda.synchronize()
    return {k_: v.cpu() for k_, v in out.items()}


def test_static_scratch_routing_matches_workspace_routing(cuda_device):
    rng = np.random.default_rng(123)
    # two calls in a row: a large routing first, then a smaller one with other experts
    for t, e, k in ((8192, 60, 4), (777, 64, 6)):
        ids = np.stack([rng.choice(e, k, replace=False) for _ in range(t)]).astype(np.int32)
        ids[5, 1] = e + 3                      # an out-of-range expert id is skipped by both
        ids_d = torch.from_numpy(ids).to(cuda_device)
        want = _route("mxmoe_route_topk", ids_d, e, cuda_device, True)
        got = _route("mxmoe_route_topk_static", ids_d, e, cuda_device, False)
        valid = int(want["row_start"][e])
        assert valid == t * k - 1
        for name in ("counts", "row_start", "slot_row"):
            assert torch.equal(got[name], want[name]), name
        for name in ("row_expert", "row_token"):
            assert torch.equal(got[name][:valid], want[name][:valid]), name
        # and against torch itself: stable sort of the (token, slot) pairs by expert, bincount of the experts
        flat = torch.from_numpy(ids.reshape(-1).astype(np.int64))
        ok = flat < e
        srt, order = torch.sort(flat[ok], stable=True)
        pairs = torch.nonzero(ok).reshape(-1)[order]
        assert torch.equal(got["counts"].long(), torch.bincount(srt, minlength=e))
        assert torch.equal(got["row_expert"][:valid].long(), srt)
        assert torch.equal(got["row_token"][:valid], pairs // k)
        inv = torch.full((t * k,), -1, dtype=torch.int64)
        inv[pairs] = torch.arange(valid)
        assert torch.equal(got["slot_row"].long(), inv)


def test_static_scratch_routing_allocates_nothing(cuda_device):
    """After the first call on the device (which looks up the address of the built-in array), a call leaves the
    amount of free device memory unchanged: nothing is allocated behind the caller's back."""
    rng = np.random.default_rng(5)
    t, e, k = 4096, 60, 4
    ids = torch.from_numpy(np.stack([rng.choice(e, k, replace=False) for _ in range(t)]).astype(np.int32)).to(cuda_device)
    n = t * k
    bufs = [torch.zeros(e, dtype=torch.int32, device=cuda_device), torch.zeros(e + 1, dtype=torch.int32, device=cuda_device),
            torch.zeros(n, dtype=torch.int32, device=cuda_device), torch.zeros(n, dtype=torch.int64, device=cuda_device),
            torch.zeros(n, dtype=torch.int32, device=cuda_device)]
    a = _lib.RouteArgs()
    a.topk_ids = ids.data_ptr()
    a.counts, a.row_start, a.row_expert, a.row_token, a.slot_row = [b.data_ptr() for b in bufs]
    a.num_tokens, a.topk, a.num_experts = t, k, e
    stream = current_stream_ptr()
    _lib.check(_lib.lib().mxmoe_route_topk_static(C.byref(a), stream))     # first call: set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        _lib.check(_lib.lib().mxmoe_route_topk_static(C.byref(a), stream))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


def test_static_scratch_limit_is_reported(cuda_device):
    t, k, e = 300000, 8, 512                   # ceil(2.4M / 1024) * 512 words > 65536
    a = _lib.RouteArgs()
    dummy = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    a.topk_ids = a.counts = a.row_start = a.row_expert = a.row_token = a.slot_row = dummy.data_ptr()
    a.num_tokens, a.topk, a.num_experts = t, k, e
    rc = _lib.lib().mxmoe_route_topk_static(C.byref(a), current_stream_ptr())
    assert rc == 4
    assert b"built-in scratch" in _lib.lib().mxmoe_last_error()
