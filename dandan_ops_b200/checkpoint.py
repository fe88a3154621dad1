"""Checkpoint tooling around the packed INT4 format (format version 2).

* `int4_prefixes` / `load_int4_layers` / `export_int4_layers`: whole-model state dicts in the
  reference's per-layer format (`<prefix>packed_weight`, `<prefix>scales`, `<prefix>zeros`,
  optional `<prefix>bias`, `<prefix>_extra_state`; dandan_ops/quantized_linear.py:105-146) go
  straight into engine layers and come back unchanged, tensor for tensor.
* `ImageCache`: the device-native weight image of a layer (what `b2_w4a16_repack` builds) kept on
  disk under a key that is a hash of the layer's state.  `ImageCache.load_layer(state)` is the restart
  path: it hashes the checkpoint tensors while they are still on the host, builds the layer without
  repacking, reads the image file (header with a CRC-32 of the image bytes, verified) and copies it to
  the device; only a miss repacks.  `attach(layer)` serves layers that already exist on the device (it
  has to copy their state back to hash it, so it saves nothing over the repack kernel and exists for
  filling the cache).
"""
import hashlib
import os
import struct
import zlib

import numpy as np
import torch

from . import _native
from .quantized_linear import FORMAT_VERSION, QuantizedLinear

_STATE_KEYS = ("packed_weight", "scales", "zeros")


def int4_prefixes(state_dict):
    """Prefixes (with trailing dot, '' for a bare layer) that hold a complete packed INT4 layer."""
    found = []
    for key in state_dict:
        if key.endswith("packed_weight"):
            prefix = key[: -len("packed_weight")]
            if all(prefix + k in state_dict for k in _STATE_KEYS) and prefix + "_extra_state" in state_dict:
                found.append(prefix)
    return sorted(found)


def load_int4_layers(state_dict, device="cuda", backend="auto"):
    """{prefix: QuantizedLinear on `device`} for every packed layer of a state dict.  Metadata and
    values are validated exactly as `QuantizedLinear.from_state_dict` does."""
    layers = {}
    for prefix in int4_prefixes(state_dict):
        local = {k: state_dict[prefix + k] for k in _STATE_KEYS}
        if isinstance(device, (str, torch.device)):
            local = {k: v.to(device) for k, v in local.items()}
        local["_extra_state"] = state_dict[prefix + "_extra_state"]
        if prefix + "bias" in state_dict:
            local["bias"] = state_dict[prefix + "bias"].to(device)
        layers[prefix] = QuantizedLinear.from_state_dict(local, backend=backend)
    return layers


def export_int4_layers(layers):
    """Inverse of `load_int4_layers`: a flat state dict (CPU tensors) in the reference's format."""
    out = {}
    for prefix, layer in layers.items():
        for key, value in layer.state_dict().items():
            out[prefix + key] = value.cpu() if isinstance(value, torch.Tensor) else value
    return out


# ---------------------------------------------------------------------------------------------
# native image cache
# ---------------------------------------------------------------------------------------------
IMAGE_MAGIC = b"B2W4IMG1"
IMAGE_LAYOUT = 1            # 16 x 256 blocks of 2336 bytes: codes, FP32 steps, 4-bit zero points
_HEADER = struct.Struct("<8sIIqqqI20x")       # magic, layout, format version, N, K, image bytes, CRC-32 of the image; 64 bytes


def state_digest(packed_weight, scales, zeros, in_features):
    """Hex SHA-256 over the layer's checkpoint-format state and shape (the cache key)."""
    h = hashlib.sha256()
    h.update(struct.pack("<IIqq", IMAGE_LAYOUT, FORMAT_VERSION, packed_weight.shape[0], in_features))
    for t in (packed_weight, scales, zeros):
        h.update(np.ascontiguousarray(t.detach().cpu().numpy()).tobytes())
    return h.hexdigest()


def write_image_file(path, image_bytes, n, k):
    """`image_bytes`: a bytes-like object or uint8 numpy array holding the native image."""
    data = bytes(image_bytes) if not isinstance(image_bytes, np.ndarray) else image_bytes.tobytes()
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(_HEADER.pack(IMAGE_MAGIC, IMAGE_LAYOUT, FORMAT_VERSION, n, k, len(data), zlib.crc32(data)))
        f.write(data)
    os.replace(tmp, path)          # readers never see a partial file


def read_image_file(path, n, k, expected_bytes):
    """uint8 numpy array of the image, or None when the file does not describe this layer."""
    try:
        with open(path, "rb") as f:
            head = f.read(_HEADER.size)
            if len(head) != _HEADER.size:
                return None
            magic, layout, version, fn, fk, nbytes, crc = _HEADER.unpack(head)
            if (magic, layout, version, fn, fk, nbytes) != (IMAGE_MAGIC, IMAGE_LAYOUT, FORMAT_VERSION, n, k,
                                                            expected_bytes):
                return None
            data = np.fromfile(f, dtype=np.uint8, count=nbytes)
    except OSError:
        return None
    if data.size != expected_bytes or zlib.crc32(data.tobytes()) != crc:      # truncated or damaged file: a miss
        return None
    return data


class ImageCache:
    """Directory of native weight images keyed by `state_digest`."""

    def __init__(self, directory):
        self.directory = str(directory)
        os.makedirs(self.directory, exist_ok=True)
        self.hits = 0
        self.misses = 0

    def path_for(self, layer):
        return os.path.join(self.directory, state_digest(layer.packed_weight, layer.scales, layer.zeros,
                                                         layer.in_features) + ".b2img")

    def store(self, layer):
        """Write the layer's image (built on its CUDA device) and return the file path."""
        path = self.path_for(layer)
        image = layer._native_image()
        write_image_file(path, image.cpu().numpy(), layer.out_features, layer.in_features)
        return path

    def load_layer(self, state, device="cuda", backend="auto"):
        """(layer on `device`, hit) from a per-layer state dict in the reference's format whose tensors
        are on the HOST: the restart path.  The key is hashed from the host tensors, the layer is built
        without its image (`defer_image=True`), and on a hit the image comes from the file - no repack
        kernel, no device-to-host copy.  On a miss the image is built on the device and stored."""
        meta = state.get("_extra_state")
        if not isinstance(meta, dict) or meta.get("format_version") != FORMAT_VERSION:
            raise ValueError("missing or unsupported INT4 format_version")
        n, k = (int(v) for v in meta["original_shape"])
        path = os.path.join(self.directory, state_digest(state["packed_weight"], state["scales"], state["zeros"], k) + ".b2img")
        bias = state.get("bias")
        layer = QuantizedLinear(state["packed_weight"].to(device), state["scales"].to(device), state["zeros"].to(device),
                                in_features=k, group_size=meta["group_size"], bias=None if bias is None else bias.to(device),
                                backend=backend, defer_image=True)
        layer.set_extra_state(meta)
        data = read_image_file(path, n, k, _native.native_bytes(n, k))
        if data is None:
            self.misses += 1
            write_image_file(path, layer._native_image().cpu().numpy(), n, k)
            return layer, False
        self.hits += 1
        layer.attach_native_image(_native.image_from_host(torch.from_numpy(data), layer.packed_weight.device))
        return layer, True

    def attach(self, layer):
        """Give a CUDA layer its image from the cache (True) or build and store it (False)."""
        if not layer.packed_weight.is_cuda:
            raise ValueError("the native image lives on a CUDA device")
        path = self.path_for(layer)
        nbytes = _native.native_bytes(layer.out_features, layer.in_features)
        data = read_image_file(path, layer.out_features, layer.in_features, nbytes)
        if data is None:
            self.misses += 1
            self.store(layer)
            return False
        self.hits += 1
        layer.attach_native_image(_native.image_from_host(torch.from_numpy(data), layer.packed_weight.device))
        return True
