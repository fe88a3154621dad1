"""Column-sharded (output-row-sharded) execution of one quantized layer over several GPUs.

Output column n of `y = x @ W^T` depends only on row n of the packed weight and on all of
x, so a layer splits along N with no exchange on the data path: every rank streams its
own slice of the weight image from its own HBM and produces `y[:, n0:n1]`.  A following
row-parallel layer consumes that slice directly.  Only when the caller asks for the full
output are the slices gathered - one NCCL all-gather over NVLink on the compute stream.

Two forms of that gather exist.  `PeerArena` + `ColumnShardedLinear.attach_arena()`: the full
`[M, N]` output lives in memory that every rank maps (torch's symmetric memory: one allocation per
rank, peer-mapped over NVLink), the projection kernel stores its slice straight into the local
copy, and ONE more launch (`b2_w4a16_gather`) pushes the slice into every peer's copy with plain
stores and exchanges epoch flags with a bounded wait - no NCCL call, no padding or permute pass,
capturable into a CUDA graph.  Without an arena the slices go through NCCL's
`all_gather_into_tensor` (also what the CPU/gloo tests of the host logic run).

The reference is single-GPU; this module is the multi-GPU form of its QuantizedLinear.
One process per GPU, `torch.distributed` already initialised by the caller.
"""
import warnings

import torch
import torch.distributed as dist

from . import _native
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


class PeerArena:
    """Memory that every rank of `group` can write: one symmetric allocation per rank holding the
    flag block of the gather kernel and, behind it, the gathered output buffers.  Construction is
    a collective call (every rank, same `nbytes`).  Buffers are carved out in call order, so all
    ranks must request them in the same order (they do: the model code is the same everywhere)."""

    ALIGN = 256

    def __init__(self, nbytes, group=None, device=None, mailbox_slice_bytes=1 << 20):
        """`nbytes`: room for the gathered outputs.  `mailbox_slice_bytes`: largest slice (bytes of one
        rank's columns of one output) that travels as polled packets instead of push + flags (costs
        4 * world * mailbox_slice_bytes of the arena; 0 = never)."""
        import torch.distributed._symmetric_memory as symm

        group = dist.group.WORLD if group is None else group
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            try:
                symm.set_backend("CUDA")
            except Exception:          # already fixed by an earlier allocation
                pass
            symm.enable_symm_mem_for_group(group.group_name)
        self.group = group
        world = dist.get_world_size(group)
        self.mailbox_slice_bytes = int(mailbox_slice_bytes)
        self.head = -(-_native.gather_block_bytes(world, self.mailbox_slice_bytes) // self.ALIGN) * self.ALIGN
        self.bytes = int(nbytes) + self.head
        self.storage = symm.empty(self.bytes, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.storage, group)
        self.rank, self.world = int(self.handle.rank), int(self.handle.world_size)
        if self.world > 16:
            raise ValueError("the gather kernel takes at most 16 ranks")
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.storage.zero_()                       # flag block: epochs, ticket and status start at zero
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                  # nobody signals into a block that is not zeroed yet
        self.used = self.head
        self.buffers = {}

    @property
    def flag_ptrs(self):
        return self.ptrs

    def output(self, key, m, n):
        """The `[m, n]` FP16 buffer registered under `key` (allocated on first use): its local
        tensor and the per-rank device addresses."""
        hit = self.buffers.get((key, m, n))
        if hit is not None:
            return hit
        size = -(-(m * n * 2) // self.ALIGN) * self.ALIGN
        if self.used + size > self.bytes:
            raise RuntimeError(f"PeerArena of {self.bytes} bytes is full ({self.used} used, {size} more requested)")
        local = self.storage[self.used:self.used + m * n * 2].view(torch.float16).view(m, n)
        entry = (local, [p + self.used for p in self.ptrs])
        self.used += size
        self.buffers[(key, m, n)] = entry
        return entry

    def status(self):
        """Sticky status word of this rank's flag block (synchronizes; bit 2 = a peer's flag did
        not arrive within the wait limit)."""
        return _native.gather_status(self.ptrs[self.rank])


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
        self.arena = None
        self.fuse_gather = True      # one launch for projection + gather where the library has it; False = always two
        self._calls = 0

    def attach_arena(self, arena):
        """Gather through peer stores into `arena` (a PeerArena of the same ranks) from now on."""
        if arena.world != self.world_size or arena.rank != self.rank:
            raise ValueError("arena belongs to another group")
        self.arena = arena
        return self

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
        if gather and self.arena is not None and compute is None and self.world_size > 1:
            return self._forward_peer_gather(x)
        run = compute if compute is not None else self.local
        if run is None:
            y = x.new_empty((x.shape[0], 0))
        else:
            y = run(x)
        return self.gather(y) if gather else y

    def _forward_peer_gather(self, x):
        """`b2_w4a16_linear_gather`: at decode sizes ONE launch that streams this rank's weights, sends every
        finished tile to the peers' mailboxes and collects theirs; otherwise the projection into this rank's
        columns of the symmetric `[M, N]` buffer followed by one `b2_w4a16_gather` launch.
        Two buffers per batch size are used in turn, so a peer that runs
        ahead writes the next call's slice into the other buffer while this rank still reads this one
        (a captured graph replays the buffer it was captured with: see include/b2_w4a16.h)."""
        m = x.shape[0]
        full, ptrs = self.arena.output((id(self), self._calls & 1), m, self.out_features)
        self._calls += 1
        if m == 0:
            return full
        local = self.local
        if local is not None and not self.fuse_gather:
            start, stop = self.rows
            local.forward_into(x, full[:, start:stop])
            local = None                                   # the call below is then the gather alone
        if local is None:
            _native.linear_gather(x, None, 0, ptrs, self.arena.flag_ptrs, self.arena.mailbox_slice_bytes, self.rank,
                                  self.out_features, self.out_features, self.rows_per_rank)
            return full
        x = local.check_input(x)
        _native.linear_gather(x, local._native_image(), local.in_features, ptrs, self.arena.flag_ptrs,
                              self.arena.mailbox_slice_bytes, self.rank, self.out_features, self.out_features,
                              self.rows_per_rank, bias=local._bias_fp16(), flags=local._image_flags)
        return full

    def gather_launches(self, m):
        """Kernels one gathered forward of `m` rows launches on this rank (1 = projection and gather fused)."""
        if self.arena is None or self.world_size == 1:
            return None
        if self.local is None:
            return 1
        if not self.fuse_gather:
            return 2
        return _native.linear_gather_launches(m, self.out_features, self.rows_per_rank, self.local.in_features, self.rank,
                                              self.world_size, self.arena.mailbox_slice_bytes)

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
