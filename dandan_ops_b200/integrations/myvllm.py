"""Bridge from an engine's signed-INT4 / group-128 weights to the operator's format.

Counterpart of the reference's `dandan_ops/integrations/myvllm.py`: the engine stores
symmetric two's-complement INT4 (two codes per byte, low nibble first, K padded to whole
groups of 128, one FP32 scale per group); the operator wants unsigned codes with a zero
point, groups of 64.  The conversion is lossless: `code_unsigned = code_signed + 8` (which
is the nibble XOR 8), zero point 8 everywhere, each scale used for two consecutive groups.

The engine itself (`mini_engine`) is not part of this repository, so the adapters take the
engine's packed tensors - or any callable that produces them from an `nn.Linear` - instead of
importing its quantizer.
"""
import torch
from torch import nn

from ..quantization import pack_int4
from ..quantized_linear import QuantizedLinear

SOURCE_GROUP = 128


def convert_signed_int4(weight, scales, in_features, source_group_size=SOURCE_GROUP):
    """(packed uint8 [N, padded_K/2], FP32 scales [N, ceil(K/128)]) -> (words, steps, zeros)
    in the operator's layout (reference: dandan_ops/integrations/myvllm.py:15-46).
    Values are checked here, once; nothing of this runs per token."""
    if source_group_size != SOURCE_GROUP:
        raise ValueError("myvllm bridge requires source_group_size=128")
    if not isinstance(in_features, int) or isinstance(in_features, bool) or in_features <= 0:
        raise ValueError("in_features must be a positive integer")
    if not isinstance(weight, torch.Tensor) or weight.dtype != torch.uint8:
        raise TypeError("source packed weight must be uint8")
    if weight.ndim != 2 or 0 in weight.shape or weight.device.type not in ("cpu", "cuda"):
        raise ValueError("source packed weight must be non-empty [N, padded_K/2] on CPU/CUDA")
    if not isinstance(scales, torch.Tensor) or scales.dtype != torch.float32:
        raise TypeError("source scales must be FP32")
    groups = -(-in_features // SOURCE_GROUP)
    if weight.shape[1] != groups * (SOURCE_GROUP // 2) or tuple(scales.shape) != (weight.shape[0], groups):
        raise ValueError("invalid source packed weight or scales shape")
    if weight.device != scales.device:
        raise ValueError("source packed weight and scales must share a device")
    if not bool(torch.logical_and(torch.isfinite(scales), scales > 0).all()):
        raise ValueError("source scales must be finite and strictly positive")
    with torch.no_grad():
        rows = weight.shape[0]
        codes = torch.empty((rows, weight.shape[1] * 2), dtype=torch.uint8, device=weight.device)
        codes[:, 0::2] = weight & 0xF          # low nibble first
        codes[:, 1::2] = weight >> 4
        unsigned = (codes[:, :in_features] ^ 8).contiguous()      # two's complement + 8
        words = pack_int4(unsigned)
        steps = scales.repeat_interleave(2, dim=1)[:, :-(-in_features // 64)].contiguous()
        zeros = torch.full(steps.shape, 8, dtype=torch.int32, device=steps.device)
    return words, steps, zeros


def _validate_config(config):
    """The engine configuration the bridge accepts (dandan_ops/integrations/myvllm.py:48-51)."""
    if (config.canonical_weight_dtype != "int4" or config.activation_dtype != "fp16"
            or config.group_size != SOURCE_GROUP or not config.symmetric):
        raise ValueError("myvllm dandan adapter requires symmetric INT4, FP16 activation, group_size=128")


def _is_config(obj):
    return all(hasattr(obj, a) for a in ("canonical_weight_dtype", "activation_dtype", "group_size", "symmetric"))


def engine_packer():
    """The engine's own signed-INT4 group-128 packer as `linear -> (packed uint8, FP32 scales)`.  The engine
    (`mini_engine`) is an external checkout; it is imported only here, on demand, as the reference does."""
    try:
        from mini_engine.quantization.backends import Int4WeightOnlyBackend
    except ImportError as exc:
        raise ImportError("the (model, config) form needs the engine's quantizer (mini_engine) on the path; "
                          "pass pack_linear=... to use another packer") from exc
    backend = Int4WeightOnlyBackend(SOURCE_GROUP)

    def pack(linear):
        source = backend.pack(linear.weight)
        return source.weight, source.scale
    return pack


class EngineQuantLinear(nn.Module):
    """Projection adapter: any leading dimensions in, same leading dimensions out.

    Two call shapes: `EngineQuantLinear(packed_weight, scales, in_features, out_features, bias=None)` from the
    engine's packed tensors, or the reference's `EngineQuantLinear(linear, config)` (an `nn.Linear` on CUDA in
    FP16 plus the engine's quantization config; needs the engine's packer, see `engine_packer`)."""

    def __init__(self, packed_weight, scales, in_features=None, out_features=None, bias=None, pack_linear=None):
        if isinstance(packed_weight, nn.Linear):
            linear, config = packed_weight, scales
            _validate_config(config)
            if linear.weight.device.type != "cuda" or linear.weight.dtype != torch.float16:
                raise ValueError("source model must be CUDA FP16")
            packed_weight, scales = (pack_linear or engine_packer())(linear)
            in_features, out_features, bias = linear.in_features, linear.out_features, linear.bias
        elif _is_config(scales):
            raise TypeError("source projection must be nn.Linear")
        super().__init__()
        words, steps, zeros = convert_signed_int4(packed_weight, scales, in_features)
        if words.shape[0] != out_features:
            raise ValueError("source packed weight does not have out_features rows")
        self.op = QuantizedLinear(words, steps, zeros, in_features=in_features, group_size=64, bias=bias,
                                  backend="cuda")
        self.in_features, self.out_features = in_features, out_features
        self.eval()

    @property
    def storage_bytes(self):
        return self.op.storage_bytes

    def dequantize(self):
        return self.op.dequantize()

    def forward(self, x):
        if x.ndim < 1 or x.shape[-1] != self.in_features:
            raise ValueError("input feature dimension mismatch")
        y = self.op(x.reshape(-1, self.in_features))      # raises on BF16 / CPU / training, as the reference
        return y.reshape(*x.shape[:-1], self.out_features)


def install_int4_projections(model, pack_linear, prefix="model.layers.", *, packer=None):
    """Replace every `nn.Linear` under `prefix` by an EngineQuantLinear.

    The second argument is either `pack_linear(linear) -> (packed uint8, FP32 scales)`, the engine's
    signed-INT4 group-128 packer, or - the reference's call shape, `install_int4_projections(model, config)` -
    the engine's quantization config, which is validated as the reference validates it and then uses
    `packer` or the engine's own packer (`engine_packer()`).  All replacements are prepared before the model
    is touched, so a failure leaves it unchanged.  Returns the report the reference attaches to the model
    (dandan_ops/integrations/myvllm.py:87-119)."""
    if _is_config(pack_linear):
        _validate_config(pack_linear)
        pack_linear = packer
    elif not callable(pack_linear):
        raise TypeError("the second argument is the engine's quantization config or a packer callable")
    if getattr(model, "quantization_report", None) is not None:
        raise ValueError("model is already quantized; reload floating weights")
    if getattr(model, "projection_fusion_enabled", False):
        raise ValueError("projection fusion and dandan quantization are not combined yet")
    selected = [(name, mod) for name, mod in model.named_modules()
                if name.startswith(prefix) and isinstance(mod, nn.Linear)]
    if not selected:
        raise ValueError("no decoder projections found")
    prepared = []
    for name, linear in selected:
        if linear.weight.device.type != "cuda" or linear.weight.dtype != torch.float16:
            raise ValueError("source model must be CUDA FP16")
        if pack_linear is None:
            pack_linear = engine_packer()
        packed, scales = pack_linear(linear)
        prepared.append((name, EngineQuantLinear(packed, scales, linear.in_features, linear.out_features,
                                                 bias=linear.bias)))
    original = sum(m.weight.numel() * m.weight.element_size() for _, m in selected)
    packed_bytes = sum(m.storage_bytes for _, m in prepared)
    for name, replacement in prepared:
        parent, _, child = name.rpartition(".")
        setattr(model.get_submodule(parent) if parent else model, child, replacement)
    report = {
        "weight_format": "int4", "activation_dtype": "fp16", "format_version": 2,
        "compute_backend": "b200_w4a16_tile_stream_or_tcgen05", "reference_only": False,
        "accelerated_quant_gemm": True, "source_group_size": SOURCE_GROUP, "storage_group_size": 64,
        "replaced_layers": [name for name, _ in prepared],
        "original_projection_weight_bytes": original,
        "packed_projection_weight_and_scale_bytes": packed_bytes,
        "projection_storage_ratio": original / packed_bytes,
        "high_precision_modules": ["embedding", "all_norms", "residual", "lm_head", "kv_cache"],
    }
    model.quantization_report = report
    return report
