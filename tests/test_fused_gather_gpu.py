"""`b2_w4a16_linear_gather` on one GPU: the column-sharded projection and the all-gather as ONE launch
(w4a16_stream_gather_kernel, w4a16_tile_gather_kernel), with the peers played by the test.  All buffers and flag blocks are local
memory; the "peers'" packets are written into this rank's mailbox by the host before the launch, so the
kernel never waits for another kernel.  Checked: the gathered `[M, N]` (own slice bit-equal to the plain
projection and within the reference's tolerance of the CPU oracle, peers' slices as sent), the packets this
rank sent into every peer's mailbox, the flag block after the call, the number of launches, the two-launch
fallback, CUDA-graph replay, and the give-up path (packets that never arrive and a short wait limit: status
bit 2, nothing hangs).  The exchange between real ranks is checked by multi_gpu_gather_check.py.
"""
import numpy as np
import pytest
import torch

from dandan_ops_b200 import _native
from dandan_ops_b200.quantized_linear import QuantizedLinear
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu
MAILBOX = 1 << 16            # bytes of one slice that may travel as packets in these tests


class Peers:
    """`world` full-size buffers and flag blocks on this GPU; rank `rank` is the one the kernel runs as."""

    def __init__(self, world, rank, m, n_total, slice_cols):
        self.world, self.rank, self.m, self.n_total, self.slice_cols = world, rank, m, n_total, slice_cols
        self.bufs = [torch.full((m, n_total), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
        words = _native.gather_block_bytes(world, MAILBOX) // 4
        self.flags = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]

    def cols(self, q):
        lo = min(self.n_total, q * self.slice_cols)
        return lo, min(self.n_total, lo + self.slice_cols)

    def box(self, owner, parity, sender):
        slots = MAILBOX // 4
        return self.flags[owner][32:].view(2, self.world, slots, 2)[parity, sender]      # [slot]{word, epoch}

    def play_peers(self, epoch, generator):
        """Write every peer's slice for call `epoch` into this rank's mailbox; returns {q: slice}."""
        sent = {}
        for q in range(self.world):
            lo, hi = self.cols(q)
            if q == self.rank or hi == lo:
                continue
            theirs = torch.randn(self.m, hi - lo, generator=generator).half().cuda()
            packets = self.box(self.rank, epoch & 1, q)
            count = self.m * (hi - lo) // 2
            packets[:count, 0] = theirs.contiguous().view(torch.int32).reshape(-1)
            packets[:count, 1] = epoch
            sent[q] = theirs
        return sent

    def ptrs(self):
        return [b.data_ptr() for b in self.bufs], [f.data_ptr() for f in self.flags]


def _layer(cols, k, seed, with_bias, fp16_steps=False):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(cols, k, generator=g) * 0.02
    bias = torch.randn(cols, generator=g) if with_bias else None
    layer = QuantizedLinear.from_float(w.cuda(), None if bias is None else bias.cuda())
    if fp16_steps:
        layer = QuantizedLinear(layer.packed_weight, layer.scales.half().float(), layer.zeros, in_features=k,
                                bias=layer.bias)
        assert layer._image_flags & _native.FLAG_FP16_STEPS
    return layer


def _run(peers, layer, x, k):
    ys, fs = peers.ptrs()
    _native.linear_gather(x, layer._native_image(), k, ys, fs, MAILBOX, peers.rank, peers.n_total, peers.n_total,
                          peers.slice_cols, bias=layer._bias_fp16(), flags=layer._image_flags)


CASES = [  # world, rank, m, n_total, slice_cols, k, bias, fp16 steps, launches
    (2, 0, 1, 2048, 1024, 28672, False, False, 1),      # streaming kernel, 16-warp CTAs
    (2, 1, 8, 1990, 1008, 28672, True, False, 1),       # short last slice, ragged last tile
    (4, 2, 16, 1024, 256, 28680, True, False, 1),       # 4-warp CTAs, two row tiles of x, ragged K
    (4, 3, 5, 4096, 1024, 28672, False, True, 1),       # FP16-step chain
    (8, 5, 13, 2048, 256, 28672, False, False, 1),
    # layers of the tile kernel (one CTA per row tile, or a cluster of 2 or 4 that splits K): one launch while the
    # last CTA can collect the peers' packets in a single round, else projection + gather kernel
    (2, 0, 1, 2048, 1024, 2048, False, False, 1),
    (2, 1, 2, 1990, 1008, 1024, True, False, 1),
    (4, 2, 1, 1024, 256, 2048, True, False, 1),
    (8, 5, 1, 2048, 256, 1032, False, False, 1),
    (4, 0, 1, 4096, 1024, 4096, True, True, 1),
    (2, 1, 6, 96, 48, 3072, True, False, 1),
    (4, 2, 16, 1024, 256, 2048, True, False, 2),
    (2, 1, 8, 1990, 1008, 1024, True, False, 2),
]


@pytest.mark.parametrize("world,rank,m,n_total,slice_cols,k,with_bias,h16,launches", CASES)
def test_one_call_computes_sends_and_collects(world, rank, m, n_total, slice_cols, k, with_bias, h16, launches):
    peers = Peers(world, rank, m, n_total, slice_cols)
    lo, hi = peers.cols(rank)
    layer = _layer(hi - lo, k, 11 * world + rank + m, with_bias, h16)
    assert _native.linear_gather_launches(m, n_total, slice_cols, k, rank, world, MAILBOX) == launches
    g = torch.Generator().manual_seed(1000 + m)
    mine_flag = peers.flags[rank]
    for epoch in range(1, 4):
        x = torch.randn(m, k, generator=g).half().cuda()
        want_own = layer(x)                                    # the plain projection of the same slice
        theirs = peers.play_peers(epoch, g)
        before = _native.load().b2_w4a16_launch_count()
        _run(peers, layer, x, k)
        assert _native.load().b2_w4a16_launch_count() - before == launches
        torch.cuda.synchronize()
        full = peers.bufs[rank]
        assert torch.equal(full[:, lo:hi], want_own)
        for q, data in theirs.items():
            qlo, qhi = peers.cols(q)
            assert torch.equal(full[:, qlo:qhi], data)
        words = want_own.contiguous().view(torch.int32).reshape(-1)
        for q in range(world):
            if q == rank:
                continue
            sent = peers.box(q, epoch & 1, rank)[:words.numel()]
            assert torch.equal(sent[:, 0], words) and bool((sent[:, 1] == epoch).all())
            assert torch.isnan(peers.bufs[q]).all()            # a peer's buffer is never written, only its mailbox
        assert int(mine_flag[16]) == epoch and int(mine_flag[17]) == 0 and int(mine_flag[18]) == 0
        if epoch == 1:                                         # reference's rule against the CPU oracle
            ref = oracle.linear(x.cpu().numpy(), layer.packed_weight.cpu().numpy(), layer.scales.cpu().numpy(),
                                layer.zeros.cpu().numpy(), k, bias=None if layer.bias is None else layer.bias.cpu().numpy())
            got = want_own.cpu().numpy().astype(np.float64)
            assert (np.abs(got - ref) <= 2e-3 + 2e-3 * np.abs(ref.astype(np.float64))).all()
    assert _native.gather_status(mine_flag.data_ptr()) == 0 and _native.status() == 0


def test_unaligned_x_takes_two_launches_with_the_same_result():
    world, rank, m, n_total, slice_cols, k = 2, 0, 8, 2048, 1024, 2048
    peers = Peers(world, rank, m, n_total, slice_cols)
    layer = _layer(slice_cols, k, 5, True)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(m, k + 8, generator=g).half().cuda()[:, 1:k + 1]       # rows start 2 bytes off a 16-byte boundary
    assert x.data_ptr() % 16 != 0 and x.stride(0) == k + 8
    theirs = peers.play_peers(1, g)
    before = _native.load().b2_w4a16_launch_count()
    _run(peers, layer, x, k)
    assert _native.load().b2_w4a16_launch_count() - before == 2
    torch.cuda.synchronize()
    assert torch.equal(peers.bufs[0][:, :slice_cols], layer(x)) and torch.equal(peers.bufs[0][:, slice_cols:], theirs[1])
    # slices that do not fit the mailbox, or more than 16 rows: two launches as well
    assert _native.linear_gather_launches(17, 2048, 1024, 28672, 0, 2, MAILBOX) == 2
    assert _native.linear_gather_launches(16, 8192, 4096, 28672, 0, 2, MAILBOX) == 2
    assert _native.linear_gather_launches(0, 8192, 4096, 28672, 0, 2, MAILBOX) == 0


def test_graph_replay_of_the_fused_call():
    """Two captured calls (epochs of both parities); the host plays the peers for every replay."""
    world, rank, m, n_total, slice_cols, k = 2, 1, 4, 2048, 1024, 28672
    peers = Peers(world, rank, m, n_total, slice_cols)
    layer = _layer(slice_cols, k, 21, False)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(m, k, generator=g).half().cuda()
    want = layer(x)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        peers.play_peers(1, g)
        _run(peers, layer, x, k)                               # warm-up outside the graph (epoch 1)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with _native.private_workspace(), torch.cuda.graph(graph, stream=stream):
            _run(peers, layer, x, k)
            _run(peers, layer, x, k)
        epoch = 1
        for _ in range(3):
            first, second = peers.play_peers(epoch + 1, g), peers.play_peers(epoch + 2, g)
            peers.bufs[rank].fill_(float("nan"))
            graph.replay()
            stream.synchronize()
            epoch += 2
            assert torch.equal(peers.bufs[rank][:, slice_cols:], want)
            assert torch.equal(peers.bufs[rank][:, :slice_cols], second[0]) and first[0].shape == second[0].shape
            assert int(peers.flags[rank][16]) == epoch
    assert _native.gather_status(peers.flags[rank].data_ptr()) == 0


def test_packets_that_never_arrive_give_a_status_not_a_hang():
    world, rank, m, n_total, slice_cols, k = 2, 0, 8, 2048, 1024, 28672
    peers = Peers(world, rank, m, n_total, slice_cols)
    layer = _layer(slice_cols, k, 31, False)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(1)).half().cuda()
    _native.gather_wait_limit(2000)       # 2 ms
    try:
        _run(peers, layer, x, k)
        torch.cuda.synchronize()                               # returns although no packet of the peer ever arrives
    finally:
        _native.gather_wait_limit(0)
    flag = peers.flags[rank]
    assert _native.gather_status(flag.data_ptr()) & 4
    assert int(flag[16]) == 1 and int(flag[17]) == 0           # epoch advanced, ticket reset: the block is reusable
    assert torch.equal(peers.bufs[0][:, :slice_cols], layer(x))          # this rank's own slice is complete
    assert _native.status() == 0                               # the projection itself saw no timeout
    # the block works again once the peer's packets are there
    theirs = peers.play_peers(2, torch.Generator().manual_seed(2))
    _run(peers, layer, x, k)
    torch.cuda.synchronize()
    assert torch.equal(peers.bufs[0][:, slice_cols:], theirs[1]) and int(flag[16]) == 2


def test_argument_checks_of_the_fused_call():
    peers = Peers(2, 0, 2, 64, 32)
    layer = _layer(32, 64, 1, False)
    x = torch.zeros(2, 64, dtype=torch.float16, device="cuda")
    ys, fs = peers.ptrs()
    with pytest.raises(RuntimeError, match="slices do not cover"):
        _native.linear_gather(x, layer._native_image(), 64, ys, fs, MAILBOX, 0, 64, 64, 16)
    with pytest.raises(RuntimeError, match="unknown flag"):
        _native.linear_gather(x, layer._native_image(), 64, ys, fs, MAILBOX, 0, 64, 64, 32, flags=8)
