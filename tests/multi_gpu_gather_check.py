"""Run under torchrun on 2+ GPUs of one node (one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=N --master-addr 127.0.0.1 tests/multi_gpu_gather_check.py

Every rank builds its row slice of a seeded layer (ColumnShardedLinear), attaches a PeerArena and runs
forward(gather=True) - b2_w4a16_linear_gather: one launch that computes, sends and collects at decode
sizes on layers the streaming kernel takes, else the projection into the symmetric buffer + one
b2_w4a16_gather launch - for decode and prefill batch sizes, with and without the one-launch form.
The gathered [M, N] must equal, bit for bit, the NCCL all-gather of the same local slices on every rank, must satisfy |y - y_ref| <= 2e-3 + 2e-3|y_ref| against the CPU oracle on
rank 0, and a CUDA-graph capture of the gathered forward must replay to the same bits.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from dandan_ops_b200.sharded import ColumnShardedLinear, PeerArena  # noqa: E402
from oracle import w4a16_oracle as oracle  # noqa: E402


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    arena = PeerArena(64 << 20)
    worst = 0.0
    fused_seen = 0
    for n, k, with_bias in ((4096, 2048, False), (1000, 1032, True), (8192, 4096, False), (2048, 28672, True)):
        g = torch.Generator().manual_seed(n + k)
        w = (torch.randn(n, k, generator=g) * (0.02 if k <= 8192 else 0.004)).half()   # outputs of order one at every K
        bias = torch.randn(n, generator=g) if with_bias else None
        layer = ColumnShardedLinear.from_float(w, bias, rank=rank, world_size=world, device=device).attach_arena(arena)
        # CPU oracle first (rank 0), so that the ranks reach every gather together
        xs = {m: torch.randn(m, k, generator=g).half() for m in (1, 8, 16, 40, 300)}
        refs = {}
        if rank == 0:
            codes, step, zero = oracle.quantize(w.numpy())
            words = oracle.pack(codes)
            refs = {m: oracle.linear(x.numpy(), words, step, zero, k, bias=None if bias is None else bias.numpy())
                    for m, x in xs.items()}
        dist.barrier()
        for m, x in xs.items():
            xg = x.to(device)
            full = layer(xg, gather=True).clone()
            nccl = layer.gather(layer(xg))
            if k == 28672 and m <= 16 and world == 2:           # (narrower slices may take the tile kernel: two launches)
                assert layer.gather_launches(m) == 1, "expected the one-launch form here"
            fused_seen += layer.gather_launches(m) == 1
            layer.fuse_gather = False                          # the same through projection + gather kernel
            two = layer(xg, gather=True).clone()
            layer.fuse_gather = True
            assert torch.equal(two, full), f"one-launch and two-launch forms differ (rank {rank}, {n}x{k}, M={m})"
            if not torch.equal(full, nccl):
                start, stop = layer.rows
                bad = (full != nccl)
                own = int(bad[:, start:stop].sum())
                raise AssertionError(f"peer gather != NCCL gather (rank {rank}, {n}x{k}, M={m}): {int(bad.sum())} elements differ, "
                                     f"{own} of them in this rank's own columns; largest difference "
                                     f"{float((full.float() - nccl.float()).abs().max()):.3e}")
            if rank == 0:
                ref = refs[m]
                ratio = np.abs(full.cpu().numpy().astype(np.float64) - ref) / (2e-3 + 2e-3 * np.abs(ref.astype(np.float64)))
                worst = max(worst, float(ratio.max()))
                assert ratio.max() <= 1.0, f"outside the tolerance: {n}x{k} M={m}"
        # capture two gathered calls (two buffers in turn) and replay
        xg = torch.randn(8, k, generator=g).half().to(device)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            want = layer(xg, gather=True).clone()
            layer(xg, gather=True)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                a = layer(xg, gather=True)
                b = layer(xg, gather=True)
            for _ in range(5):
                graph.replay()
            stream.synchronize()
            assert torch.equal(a, want) and torch.equal(b, want), "graph replay of the gathered forward differs"
    assert arena.status() == 0
    dist.barrier()
    if rank == 0:
        print(f"gather check ok: world {world}, worst bound ratio {worst:.3f}, one-launch calls seen: {fused_seen}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
