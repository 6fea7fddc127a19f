"""Expert-parallel layer on GPUs: world size 1 in-process, world size 2 under torchrun (needs 2 GPUs)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
CASES = ["tiny-ep", "tiny-ep-w4a4", "tiny-ep-w8w4"]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(nproc):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "ep_worker.py")] + CASES
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


def test_expert_parallel_world1_matches_single_gpu(cuda_device):
    _torchrun(1)


def test_expert_parallel_world2_matches_single_gpu(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _torchrun(2)


def test_barrier_wait_runs_out_when_a_peer_never_arrives(cuda_device):
    """The stream-ordered barrier of the expert-parallel step on one GPU, as rank 0 of a world of two whose second
    rank does not exist: the second sync block is a plain local buffer that nobody signals from, so rank 0's wait
    for flag 1 is a wait for a flag nothing sets.  It must give up after its limit, name the missing rank in the
    error word and return; the payload must still have been delivered to both blocks."""
    import ctypes as C
    import time
    from mxmoe_b200 import _lib
    from mxmoe_b200.gg import current_stream_ptr
    e = 6
    blocks = [torch.zeros(128 + 2 * e, dtype=torch.int32, device=cuda_device) for _ in range(2)]
    peers = torch.tensor([b.data_ptr() for b in blocks], dtype=torch.int64, device=cuda_device)
    counts = torch.arange(1, e + 1, dtype=torch.int32, device=cuda_device)
    a = _lib.EpSyncArgs()
    a.peer_sync, a.local_sync, a.payload = peers.data_ptr(), blocks[0].data_ptr(), counts.data_ptr()
    a.world, a.rank, a.payload_len, a.payload_cap, a.timeout_ms = 2, 0, e, e, 50
    t0 = time.time()
    _lib.check(_lib.lib().mxmoe_ep_sync(C.byref(a), current_stream_ptr()))
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    b0, b1 = blocks[0].cpu(), blocks[1].cpu()
    assert b0[64].item() == 2                      # 1 + the rank that did not arrive
    assert b0[65].item() == 1                      # the epoch advanced: the next barrier is well-formed
    assert b0[0].item() == 1 and b1[0].item() == 1 and b0[1].item() == 0
    assert torch.equal(b0[128:128 + e], counts.cpu()) and torch.equal(b1[128:128 + e], counts.cpu())
    # a world of one never waits
    a.world = 1
    blocks[0].zero_()
    _lib.check(_lib.lib().mxmoe_ep_sync(C.byref(a), current_stream_ptr()))
    torch.cuda.synchronize()
    assert blocks[0][64].item() == 0
