"""Writes safetensors images for the loader tests (the published layout: u64 header length, JSON
header, tensor bytes)."""
import json
import struct

import numpy as np

from boat_b200 import rng


def to_bytes(a, dtype):
    a = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == "F32":
        return a.tobytes()
    if dtype == "BF16":
        return rng.to_bf16_bits(a).tobytes()
    if dtype == "F16":
        return a.astype(np.float16).tobytes()
    raise ValueError(dtype)


def image(tensors, dtype="F32", metadata=None, pad_header=True):
    """tensors: ordered dict name -> float array (stored as `dtype`) or (array, dtype_tag, raw_bytes)."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, a in tensors.items():
        if isinstance(a, tuple):
            arr, tag, raw = a
        else:
            arr, tag, raw = a, dtype, to_bytes(a, dtype)
        header[name] = {"dtype": tag, "shape": list(np.shape(arr)), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header, separators=(",", ":"))
    if pad_header:
        text += " " * (-len(text) % 8)
    return struct.pack("<Q", len(text)) + text.encode() + b"".join(blobs)


def bert_style(H, seed=11, prefix="encoder.layer.0.", dtype="F32", with_bias=True, extra=True):
    """Checkpoint-style tensors ([out, in] weights) and the Boat-layout parameters they give."""
    names = ("attention.self.query", "attention.self.key", "attention.self.value", "attention.output.dense")
    tensors, want = {}, {}
    if extra:
        tensors["embeddings.word_embeddings.weight"] = rng.normal(seed, 90, (7, H))
    for i, (n, p) in enumerate(zip(names, "qkvo")):
        w = rng.normal(seed, i, (H, H), 0.1)               # [out, in]
        tensors[prefix + n + ".weight"] = w
        want["weight_" + p] = w.T
        if with_bias:
            b = rng.normal(seed, 10 + i, (H,), 0.1)
            tensors[prefix + n + ".bias"] = b
            want["bias_" + p] = b
    if extra:
        tensors[prefix + "attention.output.LayerNorm.weight"] = np.ones(H, np.float32)
        tensors[prefix + "attention.output.LayerNorm.bias"] = np.zeros(H, np.float32)
        tensors[prefix + "intermediate.dense.weight"] = rng.normal(seed, 91, (4 * H, H))
    return tensors, want
