"""Darknet-format ``.weights`` files, as PixieNN reads and writes them.

Layout (Model::loadWeights / saveWeights, include/Model.h:1246-1296, 1965-1985):
``int32 major, minor, revision``, then ``seen`` -- 8 bytes when ``major*10 + minor >= 2`` (and both
< 1000), else 4 -- then every layer's block in layer order.  A convolution stores
(ConvLayer::loadWeights, include/ConvLayer.h:131-150): ``biases[F]``, and with batch
normalisation ``scales[F]``, ``rollingMean[F]``, ``rollingVar[F]``, then
``weights[F * C/groups * k * k]``, all float32.  The reference writes ``seen`` as 4 bytes whatever
the version (Model.h:1979); files it saves carry version 0.1, for which 4 bytes is also what it
reads back.

A connected layer stores (ConnLayer::loadWeights, include/ConnLayer.h:119-135): ``biases[out]``,
``weights[out * in]``, and with batch normalisation ``scales[out]``, ``rollingMean[out]``,
``rollingVar[out]`` -- note the weights come before the normalisation parameters here, unlike a
convolution.  Every other layer type this package plans carries no weights.  A file with bytes left
over, or too short, is an error exactly as in the reference ("Did not fully read weights file").
"""
from __future__ import annotations

import struct
from typing import Dict, Tuple

import numpy as np

from . import graph


def _seen_bytes(major: int, minor: int) -> int:
    return 8 if (major * 10 + minor) >= 2 and major < 1000 and minor < 1000 else 4


_NO_WEIGHTS = ("maxpool", "upsample", "route", "shortcut", "yolo", "centernet", "region", "softmax", "avgpool",
               "dropout", "detection")


def _block(l: graph.Layer):
    """The arrays of one layer's block, in file order, as (name, shape) pairs."""
    norm = [("scales", (l.filters,)), ("rolling_mean", (l.filters,)), ("rolling_var", (l.filters,))]
    if l.type == "conv":
        cin = l.in_shape[0] // l.groups
        return [("biases", (l.filters,))] + (norm if l.batch_norm else []) + \
               [("weights", (l.filters, cin, l.kernel, l.kernel))]
    if l.type in ("connected", "conn"):
        inputs = l.in_shape[0] * l.in_shape[1] * l.in_shape[2]
        return [("biases", (l.filters,)), ("weights", (l.filters, inputs))] + (norm if l.batch_norm else [])
    if l.type in _NO_WEIGHTS:
        return []
    raise ValueError(f"layer {l.index}: no weights-file layout known for layer type {l.type!r}")


def load(path: str, model: graph.Model) -> Tuple[Dict[int, Dict[str, np.ndarray]], dict]:
    """Returns (weights by layer index -- the dictionary Runner and the CPU walker take --, header)."""
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < 16:
        raise ValueError(f"{path}: too short for a weights header")
    major, minor, revision = struct.unpack_from("<3i", data, 0)
    nseen = _seen_bytes(major, minor)
    seen = int.from_bytes(data[12:12 + nseen], "little")
    pos = 12 + nseen
    out: Dict[int, Dict[str, np.ndarray]] = {}

    def take(n: int) -> np.ndarray:
        nonlocal pos
        end = pos + 4 * n
        if end > len(data):
            raise ValueError(f"{path}: file ends inside layer data (need {end} bytes, have {len(data)})")
        a = np.frombuffer(data, "<f4", n, pos).copy()
        pos = end
        return a

    for l in model.layers:
        for k, shape in _block(l):
            out.setdefault(l.index, {})[k] = take(int(np.prod(shape))).reshape(shape)
    if pos != len(data):
        raise ValueError(f"{path}: did not fully read weights file; read {pos} bytes, file has {len(data)}")
    return out, {"major": major, "minor": minor, "revision": revision, "seen": seen}


def save(path: str, model: graph.Model, weights: Dict[int, Dict[str, np.ndarray]], seen: int = 0,
         version: Tuple[int, int, int] = (0, 1, 0)) -> int:
    """Writes the file the reference's saveWeights would; returns the byte count."""
    major, minor, revision = version
    chunks = [struct.pack("<3i", major, minor, revision),
              int(seen).to_bytes(_seen_bytes(major, minor), "little")]
    for l in model.layers:
        for k, shape in _block(l):
            a = np.ascontiguousarray(weights[l.index][k], "<f4")
            want = int(np.prod(shape))
            if a.size != want:
                raise ValueError(f"layer {l.index}: {k} has {a.size} values, expected {want}")
            chunks.append(a.tobytes())
    blob = b"".join(chunks)
    with open(path, "wb") as f:
        f.write(blob)
    return len(blob)
