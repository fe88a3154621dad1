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
MAILBOX = 1 << 16            # bytes of one slice that may travel as packets in these tests


def _setup(m, n, mailbox=0):
    bufs = [torch.full((m, n), float(r + 1), dtype=torch.float16, device="cuda") for r in range(2)]
    words = _native.gather_block_bytes(2, mailbox) // 4
    flags = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(2)]
    return bufs, flags


def _call(bufs, flags, mailbox, m, n_total, slice_cols):
    _native.gather([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], mailbox, 0, m, bufs[0].shape[1], n_total, slice_cols)


@pytest.mark.parametrize("m,n,slice_cols", [(1, 1024, 512), (8, 4096, 2048), (5, 992, 496), (3, 62, 31), (300, 12288, 6144)])
def test_push_and_flag_exchange_with_a_host_played_peer(m, n, slice_cols):
    """Large-slice form (no mailbox): rank 0's columns [0, slice_cols) are pushed into the peer's buffer."""
    bufs, flags = _setup(m, n)
    g = torch.Generator().manual_seed(m + n)
    bufs[0][:, :slice_cols] = torch.randn(m, slice_cols, generator=g).half().cuda()
    want = bufs[1].clone()
    want[:, :slice_cols] = bufs[0][:, :slice_cols]
    for call in range(1, 4):                                  # epochs 1, 2, 3 on the same flag blocks
        flags[0][1] = call                                    # the peer's slice "has arrived"
        _call(bufs, flags, 0, m, n, slice_cols)
        torch.cuda.synchronize()
        assert torch.equal(bufs[1], want)                     # slice pushed, nothing else touched
        assert int(flags[1][0]) == call                       # my epoch published in the peer's block
        assert int(flags[0][16]) == call and int(flags[0][17]) == 0 and int(flags[0][18]) == 0
    assert _native.gather_status(flags[0].data_ptr()) == 0


def _mailbox_view(flag_block, parity, sender):
    slots = MAILBOX // 4
    box = flag_block[32:].view(2, 2, slots, 2)                # [parity][sender][slot]{word, epoch}
    return box[parity, sender]


@pytest.mark.parametrize("m,n,slice_cols", [(1, 1024, 512), (8, 4096, 2048), (16, 1000, 504), (5, 62, 32)])
def test_mailbox_form_with_a_host_played_peer(m, n, slice_cols):
    """Small-slice form: my words go out as {word, epoch} packets into the peer's mailbox, and the peer's
    packets - written here by the host before the launch - are polled and copied into my buffer."""
    bufs, flags = _setup(m, n, MAILBOX)
    g = torch.Generator().manual_seed(3 * m + n)
    cols1 = n - slice_cols
    for call in range(1, 4):
        mine = torch.randn(m, slice_cols, generator=g).half().cuda()
        theirs = torch.randn(m, cols1, generator=g).half().cuda()
        bufs[0][:, :slice_cols] = mine
        packets = _mailbox_view(flags[0], call & 1, 1)
        packets[:m * cols1 // 2, 0] = theirs.contiguous().view(torch.int32).reshape(-1)
        packets[:m * cols1 // 2, 1] = call
        _call(bufs, flags, MAILBOX, m, n, slice_cols)
        torch.cuda.synchronize()
        assert torch.equal(bufs[0][:, slice_cols:], theirs) and torch.equal(bufs[0][:, :slice_cols], mine)
        sent = _mailbox_view(flags[1], call & 1, 0)[:m * slice_cols // 2]
        assert torch.equal(sent[:, 0], mine.contiguous().view(torch.int32).reshape(-1)) and bool((sent[:, 1] == call).all())
        assert int(flags[0][16]) == call and int(flags[0][17]) == 0 and int(flags[0][18]) == 0
    assert _native.gather_status(flags[0].data_ptr()) == 0


@pytest.mark.parametrize("mailbox", [0, MAILBOX])
def test_a_peer_that_never_arrives_gives_a_status_not_a_hang(mailbox):
    bufs, flags = _setup(4, 256, mailbox)
    _native.gather_wait_limit(2000)       # 2 ms
    try:
        _call(bufs, flags, mailbox, 4, 256, 128)
        torch.cuda.synchronize()                               # returns although nothing of the peer ever arrives
    finally:
        _native.gather_wait_limit(0)
    assert _native.gather_status(flags[0].data_ptr()) & 4
    assert int(flags[0][16]) == 1 and int(flags[0][17]) == 0   # epoch advanced, ticket reset: the block is reusable
    if mailbox == 0:
        assert torch.equal(bufs[1][:, :128], bufs[0][:, :128])


def test_gather_argument_checks():
    lib = _native.load()
    bufs, flags = _setup(2, 64)
    with pytest.raises(RuntimeError, match="slices do not cover"):
        _native.gather([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], 0, 0, 2, 64, 64, 16)
    with pytest.raises(RuntimeError, match="rank / world"):
        _native.gather([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], 0, 2, 2, 64, 64, 32)
    assert lib.b2_w4a16_noop(None) == 0
    assert _native.gather_block_bytes(8, 1 << 20) == 128 + 2 * 8 * (1 << 20) * 2


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
