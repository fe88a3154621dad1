"""`QuantizedLinear` and `quantized_linear`: the operator API of the W4A16 path.

Drop-in for the reference's `dandan_ops/quantized_linear.py`: same constructor and
factories, buffers (`packed_weight` int32, `scales` float32, `zeros` int32, `bias`),
versioned `extra_state`, load-time validation, dtype pinning, `execution_info` keys and
error messages.  Behind it sits one engine instead of four kernels plus a CPU route:

  * every CUDA FP16 call runs the native library (weight-streaming kernel for small
    batches, tensor-memory GEMM for large ones); the regime is chosen by M, not by a
    backend string or an offline route table;
  * the backend names of the reference are still accepted: "auto", "cuda",
    "tensorcore" and "naive" mean "the engine", "gemv" and "small" keep their M==1 /
    M<=8 argument checks;
  * there is no CPU, BF16, FP32 or training path: what the reference would route to
    its CPU "reference" implementation raises ValueError here, with the reference's own
    wording.

The module keeps the reference-layout tensors (they are the checkpoint format) and a
derived device-native image of them that the kernels read.  The image is rebuilt when
the tensors are replaced or modified in place (load_state_dict, .to()).
"""
import weakref

import torch

from . import _native
from . import ops as _ops_module
from .quantization import CUDA_ONLY, pack_int4, quantize_int4, validate_int4_state

BACKENDS = ("auto", "cuda", "gemv", "small", "tensorcore", "naive", "reference")
FORMAT_VERSION = 2


def _check_bias(bias, rows, device):
    ok = bias is None or (isinstance(bias, torch.Tensor) and bias.ndim == 1 and bias.numel() == rows
                          and bias.device == device and bias.is_floating_point())
    if not ok:
        raise ValueError("bias must be a floating tensor [N] on the input device")


def _resolve(x, scales, group_size, backend):
    """Backend string -> (implementation, reason).  Mirrors the argument checks of
    dandan_ops/quantized_linear.py:17-53; raises where the reference would leave the GPU."""
    if backend not in BACKENDS:
        raise ValueError(f"backend must be one of {BACKENDS}")
    training = torch.is_grad_enabled() and (x.requires_grad or scales.requires_grad)
    if backend == "reference":
        raise ValueError("backend 'reference' does not exist here: this package " + CUDA_ONLY)
    if not (x.is_cuda and x.dtype == torch.float16 and group_size == 64
                                      and not training):
        raise ValueError(CUDA_ONLY)
    if backend == "gemv" and x.shape[0] != 1:
        raise ValueError("gemv requires M=1")
    if backend == "small" and x.shape[0] > 8:
        raise ValueError("small requires M<=8")
    _native.load()
    return None


# ------------------------------------------------------------------------------------------
# Native images for callers that hold only reference-layout tensors (the functional form
# and the torch.ops entry points).  Keyed by tensor identity and version counter; entries
# die with their tensors.
# ------------------------------------------------------------------------------------------
_images = {}


def _state_key(packed, scales, zeros):
    return (packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
            packed._version, scales._version, zeros._version, tuple(packed.shape), tuple(scales.shape))


def _image_for(packed, scales, zeros, in_features):
    ident = id(packed)
    entry = _images.get(ident)
    key = _state_key(packed, scales, zeros)
    if entry is not None and entry[0] == key and entry[1]() is packed:
        return entry[2]
    image = _native.repack(packed, scales, zeros, in_features)
    ref = weakref.ref(packed, lambda _r, i=ident: _images.pop(i, None))
    _images[ident] = (key, ref, image)
    return image


def _engine(x, image, rows, in_features, bias16, flags=0):
    """`bias16`: the bias already converted to FP16 (or None); `flags`: layer flags of the C ABI.  The kernels round the product to
    FP16 first and add the FP16 bias afterwards, as the reference's `y + bias.to(y.dtype)` does."""
    if x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) < in_features):
        x = x.contiguous()
    if _ops_module.SHIM_LOADED:       # C++ operator library: output, workspace and launch without a ctypes round trip
        return torch.ops.dandan_ops.w4a16_linear_image(x, image, rows, in_features, bias16, 0, flags)
    return _native.linear(x, image, rows, in_features, bias=bias16, flags=flags)


def quantized_linear(x, packed_weight, scales, zeros, *, in_features, group_size=64, bias=None,
                     backend="auto"):
    """y = fp16(x @ W^T) (+ bias) with W = fp16((code - zero) * step), FP32 accumulation
    (dandan_ops/quantized_linear.py:56-81).  CUDA FP16 activations only."""
    validate_int4_state(packed_weight, scales, zeros, in_features, group_size)
    if not isinstance(x, torch.Tensor) or x.ndim != 2 or x.shape[1] != in_features:
        raise ValueError("x must have shape [M, in_features]")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("x must be float16, bfloat16, or float32")
    if x.device != packed_weight.device:
        raise ValueError("x and quantized weight must share a device")
    _check_bias(bias, packed_weight.shape[0], x.device)
    _resolve(x, scales, group_size, backend)
    image = _image_for(packed_weight.contiguous(), scales.contiguous(), zeros.contiguous(), in_features)
    bias16 = None if bias is None else bias.to(torch.float16).contiguous()
    return _engine(x, image, packed_weight.shape[0], in_features, bias16)


class QuantizedLinear(torch.nn.Module):
    """Packed INT4 linear layer (inference only).

    Values are validated when the layer is built or a checkpoint is loaded (that
    synchronizes); `forward` checks metadata only and never reads tensor values on the
    host, so it can be captured into a CUDA graph and replayed.
    """

    def __init__(self, packed_weight, scales, zeros, *, in_features, group_size=64, bias=None,
                 backend="auto", defer_image=False):
        """`defer_image=True` (an addition to the reference's signature) skips the eager build of the
        device-native image: for loaders that attach a prebuilt one (`checkpoint.ImageCache.load_layer`)."""
        super().__init__()
        if backend not in BACKENDS:
            raise ValueError("invalid quantized backend")
        validate_int4_state(packed_weight, scales, zeros, in_features, group_size, values=True)
        _check_bias(bias, packed_weight.shape[0], packed_weight.device)
        self.in_features = in_features
        self.out_features = packed_weight.shape[0]
        self.group_size = group_size
        self.backend = backend
        self.register_buffer("packed_weight", packed_weight.detach().contiguous())
        self.register_buffer("scales", scales.detach().contiguous())
        self.register_buffer("zeros", zeros.detach().contiguous())
        self.register_buffer("bias", None if bias is None else bias.detach().clone().contiguous())
        self._image = None
        self._image_key = None
        self._image_flags = 0
        self._bias16 = None
        self._bias16_key = None
        self._checked_key = None
        self._checked_device = None
        self.eval()
        if self.packed_weight.is_cuda and group_size == 64 and not defer_image:
            self._native_image()

    # -- construction ----------------------------------------------------------------------
    @classmethod
    def from_float(cls, weight, bias=None, *, bits=4, group_size=64, backend="auto"):
        """Quantize a floating-point [N, K] weight (dandan_ops/quantized_linear.py:158-165)."""
        if not isinstance(bits, int) or isinstance(bits, bool) or bits != 4:
            raise ValueError("only bits=4 is supported")
        with torch.no_grad():
            codes, steps, zero_points = quantize_int4(weight, group_size)
        return cls(pack_int4(codes), steps, zero_points, in_features=weight.shape[1],
                   group_size=group_size, bias=bias, backend=backend)

    @classmethod
    def from_state_dict(cls, state, *, backend="auto"):
        meta = state.get("_extra_state")
        if not isinstance(meta, dict) or meta.get("format_version") != FORMAT_VERSION:
            raise ValueError("missing or unsupported INT4 format_version")
        shape = meta.get("original_shape")
        if not isinstance(shape, (tuple, list)) or len(shape) != 2:
            raise ValueError("invalid original_shape metadata")
        layer = cls(state["packed_weight"], state["scales"], state["zeros"], in_features=shape[1],
                    group_size=meta["group_size"], bias=state.get("bias"), backend=backend)
        layer.load_state_dict(state)
        return layer

    # -- checkpoint format -----------------------------------------------------------------
    def get_extra_state(self):
        return {"format_version": FORMAT_VERSION, "bits": 4, "scheme": "affine_unsigned",
                "packing": "int32_low_nibble_first",
                "original_shape": [self.out_features, self.in_features],
                "group_size": self.group_size, "fp16_weight_rounding": "fp16_before_multiply"}

    def set_extra_state(self, state):
        mine = self.get_extra_state()
        if not isinstance(state, dict) or any(state.get(k) != v for k, v in mine.items()):
            raise ValueError("incompatible INT4 checkpoint metadata/version/shape/group_size")

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        # Validate everything before anything is copied: a bad checkpoint must leave the
        # layer untouched (dandan_ops/quantized_linear.py:115-130).
        names = [prefix + n for n in ("packed_weight", "scales", "zeros")]
        try:
            self.set_extra_state(state_dict.get(prefix + "_extra_state"))
            if all(n in state_dict for n in names):
                validate_int4_state(state_dict[names[0]], state_dict[names[1]], state_dict[names[2]],
                                    self.in_features, self.group_size, values=True)
                if state_dict[names[0]].shape[0] != self.out_features:
                    raise ValueError("incompatible output dimension")
            bias = state_dict.get(prefix + "bias")
            if bias is not None:
                _check_bias(bias, self.out_features, state_dict[names[0]].device)
        except (ValueError, TypeError, KeyError) as exc:
            error_msgs.append(f"{prefix}invalid INT4 state: {exc}")
            return
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)

    def _apply(self, fn, recurse=True):
        # .half()/.bfloat16()/.to(dtype) must not touch the quantized state: keep the
        # original tensors and only follow the device (dandan_ops/quantized_linear.py:148-156).
        words, steps, zero_points = self.packed_weight, self.scales, self.zeros
        super()._apply(fn, recurse=recurse)
        device = self.packed_weight.device
        self.packed_weight = words.to(device=device, dtype=torch.int32)
        self.scales = steps.to(device=device, dtype=torch.float32)
        self.zeros = zero_points.to(device=device, dtype=torch.int32)
        return self

    # -- native image ----------------------------------------------------------------------
    def _native_image(self):
        key = (self.packed_weight.data_ptr(), self.scales.data_ptr(), self.zeros.data_ptr(),
               self.packed_weight._version, self.scales._version, self.zeros._version)
        if self._image is None or self._image_key != key:
            self._image = _native.repack(self.packed_weight, self.scales, self.zeros, self.in_features)
            self._image_key = key
            self._image_flags = self._layer_flags()
        return self._image

    def _layer_flags(self):
        """Flags of the C ABI for this state.  FLAG_FP16_STEPS when every step is exactly representable in
        FP16 (checkpoints with FP16 scales): the decode kernels then use the FP16-only dequantization, which
        is bit-identical for such steps; FLAG_OVERLAP_LAUNCH unless switched off (B2_W4A16_OVERLAP=0).  Reads the steps once (a host sync), only when an image is (re)built -
        never on the per-token path - and not while a stream is being captured."""
        if not self.scales.is_cuda or torch.cuda.is_current_stream_capturing():
            return 0
        flags = _native.FLAG_FP16_STEPS if bool((self.scales.half().float() == self.scales).all()) else 0
        # The read above has synchronized the stream, so the image is complete in memory from here on: the
        # decode kernel may start under the tail of whatever kernel precedes it (FLAG_OVERLAP_LAUNCH).
        return flags | (_native.FLAG_OVERLAP_LAUNCH if _native.OVERLAP_LAUNCH else 0)

    def attach_native_image(self, image):
        """Use a prebuilt device image of THIS layer's state (e.g. from `checkpoint.ImageCache`)
        instead of repacking.  The image is dropped again if the state tensors change."""
        if image.dtype != torch.uint8 or image.device != self.packed_weight.device or \
                image.numel() != _native.native_bytes(self.out_features, self.in_features):
            raise ValueError("not a native image of this layer")
        self._image = image
        self._image_key = (self.packed_weight.data_ptr(), self.scales.data_ptr(), self.zeros.data_ptr(),
                           self.packed_weight._version, self.scales._version, self.zeros._version)
        self._image_flags = self._layer_flags()

    def _bias_fp16(self):
        """FP16 copy of the bias for the fused epilogue (derived, rebuilt when the bias changes)."""
        if self.bias is None:
            return None
        key = (self.bias.data_ptr(), self.bias._version, self.bias.dtype)
        if self._bias16 is None or self._bias16_key != key:
            self._bias16 = self.bias.detach().to(torch.float16).contiguous()
            self._bias16_key = key
        return self._bias16

    # -- introspection ---------------------------------------------------------------------
    def execution_info(self, x):
        """What `forward(x)` would run, without running it (same keys as the reference;
        `kernel_plan` is an addition)."""
        try:
            _resolve(x, self.scales, self.group_size, self.backend)
        except ValueError as exc:
            return {"requested_backend": self.backend, "implementation": "unavailable",
                    "fallback_reason": str(exc), "reason": str(exc), "input_copies": [],
                    "format_version": FORMAT_VERSION, "activation_dtype": str(x.dtype),
                    "group_size": self.group_size, "kernel_plan": None}
        plan = _native.plan(x.shape[0], self.out_features, self.in_features)
        return {"requested_backend": self.backend, "implementation": plan["route"],
                "fallback_reason": None, "reason": "selected packed inference backend",
                "input_copies": [i for i, t in enumerate((x, self.packed_weight, self.scales, self.zeros))
                                 if not t.is_contiguous()],
                "format_version": FORMAT_VERSION, "activation_dtype": str(x.dtype),
                "group_size": self.group_size, "kernel_plan": plan}

    @property
    def storage_bytes(self):
        """Bytes of the checkpoint-format state, as the reference counts them."""
        return sum(t.numel() * t.element_size() for t in (self.packed_weight, self.scales, self.zeros))

    @property
    def native_bytes(self):
        """Bytes of the device image the kernels stream (0.5703 B/weight for full tiles)."""
        return _native.native_bytes(self.out_features, self.in_features)

    def dequantize(self):
        """FP32 [N, K] weights, bit-identical to the reference's dequantize_int4."""
        if not self.packed_weight.is_cuda or self.group_size != 64:
            raise ValueError("dequantize " + CUDA_ONLY.replace(" FP16", ""))
        return _native.dequantize(self._native_image(), self.out_features, self.in_features)

    def _forward_key(self):
        bias = self.bias
        return (self.packed_weight.data_ptr(), self.scales.data_ptr(), self.zeros.data_ptr(),
                self.packed_weight._version, self.scales._version, self.zeros._version,
                id(self.packed_weight), id(self.scales), id(self.zeros),
                self.in_features, self.group_size, self.backend,
                None if bias is None else (bias.data_ptr(), bias._version, bias.dtype))

    def forward(self, x):
        # Per-token fast path: the metadata checks below depend only on the layer's state, so they
        # are repeated only when a state tensor was replaced or written (data pointer / version
        # counter), an attribute was reassigned, or x is not the plain CUDA FP16 case.
        key = self._forward_key()
        if (key == self._checked_key and type(x) is torch.Tensor and x.dtype is torch.float16 and x.ndim == 2
                and x.shape[1] == self.in_features and x.device == self._checked_device
                and not (x.requires_grad and torch.is_grad_enabled())):
            return _engine(x, self._image, self.out_features, self.in_features, self._bias_fp16(), self._image_flags)
        y = self._forward_checked(x)
        if self.backend in ("auto", "cuda", "tensorcore", "naive") and not self.scales.requires_grad \
                and self._image is not None:
            self._checked_key, self._checked_device = self._forward_key(), self.packed_weight.device
        return y

    def check_input(self, x):
        """Metadata checks of the raw-kernel entry points (`forward_into`, the sharded layer's fused call):
        CUDA FP16 `[M, in_features]`; returns x with unit inner stride."""
        if type(x) is not torch.Tensor or x.dtype is not torch.float16 or x.ndim != 2 or x.shape[1] != self.in_features:
            raise ValueError("x must be a CUDA FP16 tensor [M, in_features]")
        _resolve(x, self.scales, self.group_size, self.backend)
        if x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) < self.in_features):
            x = x.contiguous()
        return x

    def forward_into(self, x, out):
        """`forward(x)` written into `out`, an FP16 `[M, N]` CUDA tensor or a column slice of a wider one
        (unit inner stride; the row stride is passed to the kernel).  Used by the column-sharded layer,
        whose slice of the gathered output lives in memory shared with the other ranks."""
        if (out.dtype != torch.float16 or out.ndim != 2 or tuple(out.shape) != (x.shape[0], self.out_features)
                or out.stride(1) != 1 or out.device != x.device):
            raise ValueError("out must be an FP16 [M, N] tensor with unit inner stride on the input device")
        x = self.check_input(x)
        image = self._native_image()
        return _native.linear(x, image, self.out_features, self.in_features, out=out, bias=self._bias_fp16(),
                              flags=self._image_flags)

    def _forward_checked(self, x):
        validate_int4_state(self.packed_weight, self.scales, self.zeros, self.in_features, self.group_size)
        if not isinstance(x, torch.Tensor) or x.ndim != 2 or x.shape[1] != self.in_features:
            raise ValueError("x must have shape [M, in_features]")
        if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            raise TypeError("x must be float16, bfloat16, or float32")
        if x.device != self.packed_weight.device:
            raise ValueError("x and quantized weight must share a device")
        _check_bias(self.bias, self.out_features, x.device)
        _resolve(x, self.scales, self.group_size, self.backend)
        image = self._native_image()
        return _engine(x, image, self.out_features, self.in_features, self._bias_fp16(), self._image_flags)
