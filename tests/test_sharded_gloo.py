"""Column sharding over ranks, checked with two (and three) CPU ranks on the gloo backend.

The exchange logic (row ranges, padding of short shards, all-gather layout for M = 1 and
M > 1, a rank with an empty shard) needs no GPU.  The local product is supplied by the CPU
oracle through the `compute` hook; the shipped layer itself still refuses CPU tensors.
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, k, m, fail_rank, result_dir):
    for p in (str(ROOT), str(ROOT / "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import cases
    import dandan_ops_b200 as ops
    from oracle import w4a16_oracle as oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        w, x = cases.gaussian_case(n, k, m, 99)
        bias = torch.linspace(-1, 1, n)
        sharded = ops.ColumnShardedLinear.from_float(w, bias, rank=rank, world_size=world)
        start, stop = sharded.rows
        assert (start, stop) == ops.shard_rows(n, world, rank)
        full = ops.QuantizedLinear.from_float(w, bias)
        if sharded.local is not None:        # the shard's state is the row slice of the full layer's state
            assert torch.equal(sharded.local.packed_weight, full.packed_weight[start:stop])
            assert torch.equal(sharded.local.scales, full.scales[start:stop])
            assert torch.equal(sharded.local.zeros, full.zeros[start:stop])
            with pytest.raises(ValueError, match="CUDA FP16"):
                sharded(x)                    # no CPU compute path in the product
        if rank == fail_rank:
            raise RuntimeError("injected host failure before the collective")

        def local_product(xx):
            if stop == start:
                return xx.new_empty((xx.shape[0], 0))
            l = sharded.local
            y = oracle.linear(xx.numpy(), l.packed_weight.numpy(), l.scales.numpy(), l.zeros.numpy(), k,
                              bias=l.bias.numpy())
            return torch.from_numpy(y)

        y_local = sharded(x, compute=local_product)
        assert y_local.shape == (m, stop - start)
        y_full = sharded(x, gather=True, compute=local_product)
        want = torch.from_numpy(oracle.linear(x.numpy(), full.packed_weight.numpy(), full.scales.numpy(),
                                              full.zeros.numpy(), k, bias=bias.numpy()))
        assert y_full.shape == (m, n)
        assert torch.equal(y_full[:, start:stop], y_local)
        assert oracle.within_tolerance(y_full.numpy(), want.numpy())
        np.save(os.path.join(result_dir, f"rank{rank}.npy"), y_full.numpy())
    finally:
        dist.destroy_process_group()


def _spawn(world, n, k, m, tmp_path, fail_rank=-1):
    ctx = mp.spawn(_worker, args=(world, _free_port(), n, k, m, fail_rank, str(tmp_path)), nprocs=world, join=False)
    return ctx


@pytest.mark.parametrize("world,n,m", [(2, 96, 1), (2, 100, 5), (3, 40, 3), (2, 16, 2)])
def test_sharded_gather_matches_full_layer(world, n, m, tmp_path):
    ctx = _spawn(world, n, 72, m, tmp_path)
    while not ctx.join(timeout=120):
        pass
    outs = [np.load(tmp_path / f"rank{r}.npy") for r in range(world)]
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])          # every rank holds the same gathered output


def test_rank_failure_before_collective_surfaces_on_the_host(tmp_path):
    """A rank that raises before the all-gather must not leave the others hanging: the
    process group's timeout (or the peer's closed connection) ends their collective."""
    ctx = _spawn(2, 64, 72, 2, tmp_path, fail_rank=1)
    with pytest.raises(Exception):
        while not ctx.join(timeout=120):
            pass
    assert not (tmp_path / "rank1.npy").exists()


def test_shard_rows_cover_and_align():
    import dandan_ops_b200 as ops

    for n in (1, 15, 16, 17, 1000, 8192, 57344, 12289):
        for world in (1, 2, 3, 4, 8):
            spans = [ops.shard_rows(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(s % 16 == 0 for s, _ in spans if s < n)
    assert ops.shard_rows(57344, 8, 3) == (3 * 7168, 4 * 7168)
    with pytest.raises(ValueError):
        ops.shard_rows(10, 2, 2)
