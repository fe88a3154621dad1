"""Projection sets that share an input, run as one N-concatenated launch.

The reference keeps q/k/v and gate/up as separate layers and refuses to combine its INT4
path with the engine's projection fusion (dandan_ops/integrations/myvllm.py:96-97), while its
benchmarks time the fused shapes (`qkv_fused`, `gate_up_fused`,
benchmarks/bench_qwen3_gemm.py:50-57).  Output column n of a W4A16 linear depends only on row n
of the quantized state, so stacking the rows of several layers gives exactly the layers'
columns side by side: one weight stream, one launch, no change to any value of the state.
"""
import torch
from torch import nn

from . import _native
from .quantized_linear import QuantizedLinear


def concat_layers(layers, backend=None):
    """One QuantizedLinear whose rows are the rows of `layers` in order (same in_features,
    group size and device).  A missing bias counts as zeros when any layer has one."""
    layers = list(layers)
    if not layers or not all(isinstance(l, QuantizedLinear) for l in layers):
        raise TypeError("concat_layers takes a non-empty sequence of QuantizedLinear layers")
    first = layers[0]
    for layer in layers[1:]:
        if layer.in_features != first.in_features or layer.group_size != first.group_size:
            raise ValueError("fused projections must share in_features and group_size")
        if layer.packed_weight.device != first.packed_weight.device:
            raise ValueError("fused projections must share a device")
    bias = None
    if any(l.bias is not None for l in layers):
        dtype = next(l.bias.dtype for l in layers if l.bias is not None)
        bias = torch.cat([l.bias.to(dtype) if l.bias is not None
                          else torch.zeros(l.out_features, dtype=dtype, device=first.packed_weight.device)
                          for l in layers])
    return QuantizedLinear(torch.cat([l.packed_weight for l in layers]), torch.cat([l.scales for l in layers]),
                           torch.cat([l.zeros for l in layers]), in_features=first.in_features,
                           group_size=first.group_size, bias=bias, backend=backend or first.backend)


class FusedProjections(nn.Module):
    """`forward(x)` returns one output per original layer (views of one [M, sum N_i] result).

    `unfuse()` gives the original layers back, state bit-identical, e.g. to save a checkpoint
    in the per-projection format."""

    def __init__(self, layers, names=None):
        super().__init__()
        layers = list(layers)
        self.op = concat_layers(layers)
        self.split_sizes = [l.out_features for l in layers]
        self.names = list(names) if names is not None else [str(i) for i in range(len(layers))]
        if len(self.names) != len(layers):
            raise ValueError("one name per fused layer")
        self._had_bias = [l.bias is not None for l in layers]
        self.in_features, self.out_features = self.op.in_features, self.op.out_features
        self.eval()

    @property
    def storage_bytes(self):
        return self.op.storage_bytes

    def execution_info(self, x):
        return self.op.execution_info(x)

    def forward(self, x):
        y = self.op(x)
        return y.split(self.split_sizes, dim=1)

    def unfuse(self):
        out, row = [], 0
        for rows, had_bias in zip(self.split_sizes, self._had_bias):
            sl = slice(row, row + rows)
            out.append(QuantizedLinear(self.op.packed_weight[sl].clone(), self.op.scales[sl].clone(),
                                       self.op.zeros[sl].clone(), in_features=self.in_features,
                                       group_size=self.op.group_size,
                                       bias=self.op.bias[sl].clone() if had_bias else None,
                                       backend=self.op.backend))
            row += rows
        return out


def pair_order(rows, device=None):
    """Row permutation of a [gate; up] stack of 2 x `rows` rows into pair order: every 16-row tile
    holds 8 gate rows followed by the 8 up rows of the same output columns."""
    if rows % 8:
        raise ValueError("the fused gate/up epilogue needs a multiple of 8 output columns")
    j = torch.arange(rows, device=device).view(-1, 8)
    return torch.cat([j, j + rows], dim=1).reshape(-1)


class GateUpSilu(nn.Module):
    """SiLU(gate(x)) * up(x) of a gated MLP as ONE launch.

    The reference runs the fused `gate_up` projection and then a separate `silu_and_mul` kernel
    (dandan_ops/elementwise.py:168-173).  Here the rows of the two layers are interleaved in
    groups of eight so that a thread of the decode kernels ends up with the gate and the up sum
    of the same output column, and the activation is applied before anything is written: the
    [M, 2I] intermediate never exists for M <= 64.  Rounding follows the reference: both sums to
    FP16 (plus FP16 bias), SiLU rounded to FP16, product rounded to FP16."""

    def __init__(self, gate, up):
        super().__init__()
        if gate.out_features != up.out_features:
            raise ValueError("gate and up projections must have the same number of rows")
        stacked = concat_layers([gate, up])
        order = pair_order(gate.out_features, stacked.packed_weight.device)
        self.op = QuantizedLinear(stacked.packed_weight[order], stacked.scales[order], stacked.zeros[order],
                                  in_features=stacked.in_features, group_size=stacked.group_size,
                                  bias=None if stacked.bias is None else stacked.bias[order], backend=stacked.backend)
        self.in_features, self.out_features = gate.in_features, gate.out_features
        self._had_bias = (gate.bias is not None, up.bias is not None)
        self.eval()

    @property
    def storage_bytes(self):
        return self.op.storage_bytes

    def forward(self, x):
        if not isinstance(x, torch.Tensor) or x.ndim != 2 or x.shape[1] != self.in_features:
            raise ValueError("x must have shape [M, in_features]")
        if x.dtype != torch.float16 or not x.is_cuda or x.device != self.op.packed_weight.device:
            raise ValueError("the fused gate/up projection requires CUDA FP16 input on the layer's device")
        if x.stride(1) != 1:
            x = x.contiguous()
        image = self.op._native_image()
        return _native.linear_silu_mul(x, image, self.op.out_features, self.in_features, bias=self.op._bias_fp16(),
                                       flags=self.op._image_flags & _native.FLAG_OVERLAP_LAUNCH)

    def unfuse(self):
        """The original (gate, up) layers, state bit-identical."""
        inverse = torch.empty_like(pair_order(self.out_features, self.op.packed_weight.device))
        inverse[pair_order(self.out_features, inverse.device)] = torch.arange(2 * self.out_features, device=inverse.device)
        out = []
        for part, had_bias in zip((0, 1), self._had_bias):
            rows = inverse[part * self.out_features:(part + 1) * self.out_features]
            out.append(QuantizedLinear(self.op.packed_weight[rows].clone(), self.op.scales[rows].clone(),
                                       self.op.zeros[rows].clone(), in_features=self.in_features,
                                       group_size=self.op.group_size,
                                       bias=self.op.bias[rows].clone() if had_bias else None, backend=self.op.backend))
        return tuple(out)


class RmsNormLinear(nn.Module):
    """`forward(x, residual=None) -> (y, summed)`: residual add + RMSNorm + projection.

    The step in front of the qkv projection of a decoder layer, with the rounding order of the
    reference's `residual_rms_norm` (dandan_ops/elementwise.py:156-165): one norm kernel (a CTA per
    row, fixed summation order) and the projection, both on the current stream."""

    def __init__(self, norm_weight, layer, eps=1e-5):
        super().__init__()
        if not isinstance(layer, QuantizedLinear):
            raise TypeError("layer must be a QuantizedLinear")
        if norm_weight.ndim != 1 or norm_weight.shape[0] != layer.in_features:
            raise ValueError("norm weight must have in_features elements")
        if layer.in_features % 8:
            raise ValueError("the RMSNorm prologue needs in_features to be a multiple of 8")
        eps = float(eps)
        if not (eps >= 0.0) or eps == float("inf"):
            raise ValueError("eps must be finite, nonnegative and representable as FP32")
        self.op = layer
        self.eps = eps
        self.register_buffer("norm_weight", norm_weight.detach().to(torch.float16).contiguous())
        self.in_features, self.out_features = layer.in_features, layer.out_features
        self.eval()

    def forward(self, x, residual=None):
        for t in (x, residual):
            if t is None:
                continue
            if not isinstance(t, torch.Tensor) or t.ndim != 2 or t.shape[1] != self.in_features:
                raise ValueError("x and residual must have shape [M, in_features]")
            if t.dtype != torch.float16 or t.device != self.op.packed_weight.device or not t.is_cuda:
                raise ValueError("the RMSNorm prologue requires CUDA FP16 inputs on the layer's device")
        if residual is not None and residual.shape != x.shape:
            raise ValueError("x and residual must have the same shape")
        x = x.contiguous()
        residual = None if residual is None else residual.contiguous()
        return _native.rmsnorm_linear(x, residual, self.norm_weight, self.eps, self.op._native_image(),
                                      self.out_features, self.in_features, bias=self.op._bias_fp16())


def fuse_named_projections(parent, names, fused_name=None):
    """Replace the child modules `names` of `parent` (QuantizedLinear layers or adapters that
    hold one in `.op`) by one FusedProjections child called `fused_name` (default: the names
    joined by '_').  The caller changes its forward to use the fused child's tuple output.
    Returns the new module."""
    children = [getattr(parent, n) for n in names]
    layers = [c if isinstance(c, QuantizedLinear) else getattr(c, "op", None) for c in children]
    if not all(isinstance(l, QuantizedLinear) for l in layers):
        raise TypeError("every fused child must be a QuantizedLinear or hold one in .op")
    fused = FusedProjections(layers, names)
    for n in names:
        delattr(parent, n)
    setattr(parent, fused_name or "_".join(names), fused)
    return fused
