"""Darknet .weights round trip and the reference's length check (CPU only)."""
import struct

import numpy as np
import pytest

from pixienn_b200 import graph, presets, weights
from pixienn_b200.runner import synth_weights


def test_round_trip_and_layout(tmp_path):
    model = graph.parse_model(presets.yolov3_tiny(96, 96))
    w = synth_weights(model, 3, head_bias=-1.0)
    path = str(tmp_path / "tiny.weights")
    n = weights.save(path, model, w, seen=1234)
    params = sum(v.size for d in w.values() for v in d.values())
    assert n == 16 + 4 * params                      # version 0.1: 3 ints + 4-byte seen
    back, hdr = weights.load(path, model)
    assert hdr == {"major": 0, "minor": 1, "revision": 0, "seen": 1234}
    for i, d in w.items():
        for k, v in d.items():
            assert np.array_equal(back[i][k], v), (i, k)
    # first conv block: biases, scales, mean, var, then weights
    raw = open(path, "rb").read()
    first = np.frombuffer(raw, "<f4", 16, 16)
    assert np.array_equal(first, w[0]["biases"])
    assert np.array_equal(np.frombuffer(raw, "<f4", 16, 16 + 64), w[0]["scales"])


def test_eight_byte_seen_for_version_0_2(tmp_path):
    model = graph.parse_model(presets.yolov3_tiny(96, 96))
    w = synth_weights(model, 4)
    path = str(tmp_path / "v02.weights")
    n = weights.save(path, model, w, seen=2 ** 33 + 5, version=(0, 2, 0))
    assert struct.unpack_from("<3i", open(path, "rb").read(), 0) == (0, 2, 0)
    back, hdr = weights.load(path, model)
    assert hdr["seen"] == 2 ** 33 + 5 and n == 20 + 4 * sum(v.size for d in w.values() for v in d.values())
    assert np.array_equal(back[12]["weights"], w[12]["weights"])


def test_wrong_length_is_an_error(tmp_path):
    model = graph.parse_model(presets.yolov3_tiny(96, 96))
    w = synth_weights(model, 5)
    path = str(tmp_path / "t.weights")
    weights.save(path, model, w)
    blob = open(path, "rb").read()
    open(path, "wb").write(blob + b"\0\0\0\0")
    with pytest.raises(ValueError, match="did not fully read"):
        weights.load(path, model)
    open(path, "wb").write(blob[:-8])
    with pytest.raises(ValueError, match="file ends inside"):
        weights.load(path, model)


def test_connected_layer_blocks(tmp_path):
    """A connected layer's block is biases, weights, then (with batch normalisation) scales, mean, variance
    (include/ConnLayer.h:119-135); a convolution behind it starts where the reference's reader would be."""
    doc = {"model": {"channels": 3, "height": 8, "width": 8, "layers": [
        {"type": "conv", "filters": 4, "kernel": 3, "stride": 2, "pad": True, "batch_normalize": True, "activation": "leaky"},
        {"type": "connected", "output": 10, "activation": "leaky", "batch_normalize": True},
        {"type": "connected", "output": 6, "activation": "linear"},
        {"type": "softmax"},
    ]}}
    model = graph.parse_model(doc)
    w = synth_weights(model, 6)
    path = str(tmp_path / "conn.weights")
    n = weights.save(path, model, w)
    conv = 4 * 4 + 4 * 3 * 9
    conn1 = 10 + 10 * 64 + 3 * 10
    conn2 = 6 + 6 * 10
    assert n == 16 + 4 * (conv + conn1 + conn2)
    raw = open(path, "rb").read()
    base = 16 + 4 * conv
    assert np.array_equal(np.frombuffer(raw, "<f4", 10, base), w[1]["biases"])
    assert np.array_equal(np.frombuffer(raw, "<f4", 640, base + 40).reshape(10, 64), w[1]["weights"])
    assert np.array_equal(np.frombuffer(raw, "<f4", 10, base + 40 + 2560), w[1]["scales"])
    back, _ = weights.load(path, model)
    for i, d in w.items():
        assert set(back[i]) == set(d)
        for k, v in d.items():
            assert np.array_equal(back[i][k], v), (i, k)
