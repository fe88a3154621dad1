"""`b2_w4a16_gather` on one GPU: the push of a column slice into a second buffer and the flag
exchange, with the peer played by the test (both buffers and both flag blocks are local memory, and
the "peer's" epoch flag is written by the host before the launch - a kernel never waits for another
kernel here).  The give-up path: a flag that nothing sets and a short wait limit; the kernel must
return with bit 2 of the status word set.  The real multi-rank exchange is checked by
multi_gpu_gather_check.py (run under torchrun on 2+ GPUs).
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from dandan_ops_b200 import _native

pytestmark = pytest.mark.gpu
WORDS = _native.GATHER_FLAG_BYTES // 4


def _setup(m, n):
    bufs = [torch.full((m, n), float(r + 1), dtype=torch.float16, device="cuda") for r in range(2)]
    flags = [torch.zeros(WORDS, dtype=torch.int32, device="cuda") for _ in range(2)]
    return bufs, flags


@pytest.mark.parametrize("m,n,col0,cols", [(1, 1024, 0, 512), (8, 4096, 2048, 2048), (5, 1000, 504, 496), (3, 77, 13, 31),
                                           (300, 12288, 6144, 6144)])
def test_push_and_flag_exchange_with_a_host_played_peer(m, n, col0, cols):
    bufs, flags = _setup(m, n)
    g = torch.Generator().manual_seed(m + n)
    bufs[0][:, col0:col0 + cols] = torch.randn(m, cols, generator=g).half().cuda()
    want = bufs[1].clone()
    want[:, col0:col0 + cols] = bufs[0][:, col0:col0 + cols]
    for call in range(1, 4):                                  # epochs 1, 2, 3 on the same flag blocks
        flags[0][1] = call                                    # the peer's slice "has arrived"
        _native.gather([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], 0, m, n, col0, cols)
        torch.cuda.synchronize()
        assert torch.equal(bufs[1], want)                     # slice pushed, nothing else touched
        assert int(flags[1][0]) == call                       # my epoch published in the peer's block
        assert int(flags[0][16]) == call and int(flags[0][17]) == 0 and int(flags[0][18]) == 0
    assert _native.gather_status(flags[0].data_ptr()) == 0


def test_a_peer_that_never_arrives_gives_a_status_not_a_hang():
    bufs, flags = _setup(4, 256)
    _native.gather_wait_limit(2000)       # 2 ms
    try:
        _native.gather([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], 0, 4, 256, 0, 128)
        torch.cuda.synchronize()                               # returns although flags[0][1] stays 0
    finally:
        _native.gather_wait_limit(0)
    assert _native.gather_status(flags[0].data_ptr()) & 4
    assert int(flags[0][16]) == 1 and int(flags[0][17]) == 0   # epoch advanced, ticket reset: the block is reusable
    assert torch.equal(bufs[1][:, :128], bufs[0][:, :128])


def test_gather_argument_checks():
    lib = _native.load()
    bufs, flags = _setup(2, 64)
    with pytest.raises(RuntimeError, match="slice outside the row"):
        _native.gather([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], 0, 2, 64, 32, 64)
    with pytest.raises(RuntimeError, match="rank / world"):
        _native.gather([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], 2, 2, 64, 0, 32)
    assert lib.b2_w4a16_noop(None) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_exchange_under_torchrun():
    """Two processes, one GPU each: sharded projection + peer-store gather against the unsharded layer."""
    root = Path(__file__).resolve().parent
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", "29731", str(root / "multi_gpu_gather_check.py")],
                          capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "gather check ok" in proc.stdout
