"""B200-native W4A16 quantized-linear engine behind the dandan-ops operator API.

    import dandan_ops_b200 as ops
    layer = ops.QuantizedLinear.from_float(weight, group_size=64)   # weight on a CUDA device
    y = layer(x)                                                    # x: CUDA FP16 [M, K]

The public names are those of the reference package's quantized-linear path; the
compute path is a C-ABI CUDA library for sm_100a (see include/b2_w4a16.h).
"""
from .quantization import (dequantize_int4, pack_int4, quantize_int4, unpack_int4,
                           validate_int4_state)
from .quantized_linear import BACKENDS, FORMAT_VERSION, QuantizedLinear, quantized_linear
from .sharded import ColumnShardedLinear, shard_rows
from .fused import FusedProjections, GateUpSilu, RmsNormLinear, concat_layers, fuse_named_projections
from . import checkpoint
from . import ops as _ops

__all__ = ["quantize_int4", "dequantize_int4", "pack_int4", "unpack_int4", "validate_int4_state",
           "QuantizedLinear", "quantized_linear", "BACKENDS", "FORMAT_VERSION",
           "ColumnShardedLinear", "shard_rows", "FusedProjections", "GateUpSilu", "RmsNormLinear", "concat_layers",
           "fuse_named_projections", "checkpoint"]

try:
    _ops.register()
except RuntimeError:      # the names are already defined (reference extension loaded first)
    pass
