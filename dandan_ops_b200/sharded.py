"""Column-sharded (output-row-sharded) execution of one quantized layer over several GPUs.

Output column n of `y = x @ W^T` depends only on row n of the packed weight and on all of
x, so a layer splits along N with no exchange on the data path: every rank streams its
own slice of the weight image from its own HBM and produces `y[:, n0:n1]`.  A following
row-parallel layer consumes that slice directly.  Only when the caller asks for the full
output are the slices gathered - one NCCL all-gather over NVLink on the compute stream.

The reference is single-GPU; this module is the multi-GPU form of its QuantizedLinear.
One process per GPU, `torch.distributed` already initialised by the caller.
"""
import torch
import torch.distributed as dist

from .quantized_linear import QuantizedLinear

ROW_ALIGN = 16   # native tile height: shards start on tile boundaries


def shard_rows(out_features, world_size, rank, align=ROW_ALIGN):
    """Half-open row range [start, stop) owned by `rank`; every rank but the last gets the
    same, `align`-multiple number of rows, trailing ranks may be short or empty."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must satisfy 0 <= rank < world_size")
    tiles = -(-out_features // align)
    per_rank = -(-tiles // world_size) * align
    start = min(out_features, rank * per_rank)
    stop = min(out_features, start + per_rank)
    return start, stop


class ColumnShardedLinear(torch.nn.Module):
    """This rank's row slice of a QuantizedLinear plus the optional gather of outputs."""

    def __init__(self, local, *, out_features, rank, world_size, process_group=None):
        super().__init__()
        start, stop = shard_rows(out_features, world_size, rank)
        if local is not None and local.out_features != stop - start:
            raise ValueError("local layer does not match this rank's row range")
        self.local = local
        self.out_features = out_features
        self.rank, self.world_size = rank, world_size
        self.process_group = process_group
        self.rows = (start, stop)
        self.rows_per_rank = shard_rows(out_features, world_size, 0)[1]

    @classmethod
    def from_float(cls, weight, bias=None, *, rank, world_size, process_group=None, group_size=64,
                   device=None):
        """Quantize only this rank's rows of the full [N, K] weight.  Quantization is
        independent per row, so the result equals the row slice of the full layer's state."""
        start, stop = shard_rows(weight.shape[0], world_size, rank)
        local = None
        if stop > start:
            w = weight[start:stop]
            b = None if bias is None else bias[start:stop]
            if device is not None:
                w = w.to(device)
                b = None if b is None else b.to(device)
            local = QuantizedLinear.from_float(w, b, group_size=group_size)
        return cls(local, out_features=weight.shape[0], rank=rank, world_size=world_size,
                   process_group=process_group)

    @classmethod
    def from_state(cls, packed_weight, scales, zeros, *, in_features, rank, world_size, bias=None,
                   process_group=None, device=None):
        """Slice an existing full-layer state (reference layout) by rows."""
        start, stop = shard_rows(packed_weight.shape[0], world_size, rank)
        local = None
        if stop > start:
            parts = [t[start:stop] for t in (packed_weight, scales, zeros)]
            b = None if bias is None else bias[start:stop]
            if device is not None:
                parts = [t.to(device) for t in parts]
                b = None if b is None else b.to(device)
            local = QuantizedLinear(*parts, in_features=in_features, bias=b)
        return cls(local, out_features=packed_weight.shape[0], rank=rank, world_size=world_size,
                   process_group=process_group)

    def forward(self, x, gather=False, compute=None):
        """Local slice `[M, n_local]`, or the full `[M, N]` on every rank when `gather`.
        `compute` replaces the local layer's forward (tests of the exchange logic)."""
        run = compute if compute is not None else self.local
        if run is None:
            y = x.new_empty((x.shape[0], 0))
        else:
            y = run(x)
        return self.gather(y) if gather else y

    def gather(self, y_local):
        """All-gather of the per-rank slices into `[M, N]` (same result on every rank)."""
        if self.world_size == 1:
            return y_local
        m = y_local.shape[0]
        pad = self.rows_per_rank - y_local.shape[1]
        piece = y_local if pad == 0 else torch.nn.functional.pad(y_local, (0, pad))
        piece = piece.contiguous()
        out = piece.new_empty((self.world_size * m, self.rows_per_rank))     # rank-major concatenation
        dist.all_gather_into_tensor(out, piece, group=self.process_group)
        out = out.view(self.world_size, m, self.rows_per_rank)
        if m == 1:
            full = out.view(1, self.world_size * self.rows_per_rank)
        else:
            full = out.permute(1, 0, 2).reshape(m, self.world_size * self.rows_per_rank)
        return full[:, :self.out_features]
