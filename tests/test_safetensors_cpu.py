"""safetensors loader, the part that needs no GPU: header parsing and every refusal happen
before the first device call."""
import struct

import numpy as np
import pytest

import safetensors_util as st
from boat_b200.host import Attention

H = 16


@pytest.fixture()
def layer(lib):
    a = Attention(H, 4)
    yield a
    a.free()


def test_null_arguments_and_short_images(lib, layer):
    assert lib.boat_attention_load_safetensors(None, None, 0, None) == 1
    assert layer.load_safetensors(b"") == 2
    assert layer.load_safetensors(b"\x01\x02\x03") == 2
    assert layer.load_safetensors("/nonexistent/file.safetensors") == 1


@pytest.mark.parametrize("mutate", ["header_longer_than_file", "not_json", "truncated_json", "offset_past_end",
                                    "begin_after_end", "missing_offsets", "deep_nesting"])
def test_malformed_images_are_refused(layer, mutate):
    tensors, _ = st.bert_style(H)
    img = bytearray(st.image(tensors))
    n = struct.unpack("<Q", img[:8])[0]
    if mutate == "header_longer_than_file":
        img[:8] = struct.pack("<Q", len(img))
    elif mutate == "not_json":
        img[8:12] = b"@@@@"
    elif mutate == "truncated_json":
        img = img[:8] + img[8:8 + n - 9] + b" " * 9 + img[8 + n:]
    elif mutate == "offset_past_end":
        img = bytearray(st.image(tensors)[:-64])
    elif mutate == "begin_after_end":
        text = img[8:8 + n].decode().replace('"data_offsets":[0,', '"data_offsets":[99999999,', 1)
        text = text[:n] if len(text) >= n else text + " " * (n - len(text))
        img = bytearray(struct.pack("<Q", len(text)) + text.encode() + bytes(img[8 + n:]))
    elif mutate == "missing_offsets":
        text = img[8:8 + n].decode().replace('"data_offsets"', '"data_offsetz"', 1)
        img = bytearray(struct.pack("<Q", len(text)) + text.encode() + bytes(img[8 + n:]))
    elif mutate == "deep_nesting":
        img = bytearray(st.image(tensors, metadata={"a": eval("[" * 40 + "]" * 40)}))
    assert layer.load_safetensors(bytes(img)) == 2


def test_missing_projection_wrong_shape_wrong_type_and_ambiguity(layer):
    tensors, _ = st.bert_style(H)
    partial = {k: v for k, v in tensors.items() if "value.weight" not in k}
    assert layer.load_safetensors(st.image(partial)) == 3
    wrong, _ = st.bert_style(H + 8)
    assert layer.load_safetensors(st.image(wrong)) == 4
    ints = dict(tensors)
    key = "encoder.layer.0.attention.self.query.weight"
    ints[key] = (tensors[key], "I32", np.zeros((H, H), np.int32).tobytes())
    assert layer.load_safetensors(st.image(ints)) == 4
    two_layers = dict(tensors)
    two_layers.update(st.bert_style(H, prefix="encoder.layer.1.", extra=False)[0])
    assert layer.load_safetensors(st.image(two_layers)) == 4            # ambiguous without a prefix
    assert layer.load_safetensors(st.image(two_layers), prefix="decoder.") == 3   # nothing matches that prefix
