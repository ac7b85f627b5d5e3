"""Model graphs of the benchmark configurations, generated in the reference's YAML schema.

The reference ships these graphs as YAML files (resources/models/yolov3-tiny.yml, yolov3.yml,
yolov7.yml, centernet-tiny-voc.yml); its files load unchanged through ``graph.load_yaml``.  The
builders below write the same architectures (Darknet-53 / YOLOv3, YOLOv3-tiny, the YOLOv7 E-ELAN
graph, the tiny CenterNet) from their block structure, so the benchmarks run where no checkout
of the reference exists.  ``tests/test_presets.py`` checks them layer by layer against the
reference's files when those are available.
"""
from __future__ import annotations

from typing import List


def _conv(filters, kernel, stride=1, act="leaky", bn=True, pad=True):
    d = {"type": "conv", "filters": filters, "kernel": kernel, "stride": stride, "pad": pad, "activation": act}
    if bn:
        d["batch_normalize"] = True
    return d


def _yolo(mask, anchors, num):
    return {"type": "yolo", "mask": list(mask), "anchors": list(anchors), "num": num}


def _doc(layers: List[dict], height: int, width: int) -> dict:
    return {"model": {"batch": 1, "subdivisions": 1, "channels": 3, "height": height, "width": width, "layers": layers}}


V3_TINY_ANCHORS = [10, 14, 23, 27, 37, 58, 81, 82, 135, 169, 344, 319]
V3_ANCHORS = [10, 13, 16, 30, 33, 23, 30, 61, 62, 45, 59, 119, 116, 90, 156, 198, 373, 326]
V7_ANCHORS = [8, 10, 12, 23, 26, 18, 23, 49, 49, 36, 47, 95, 92, 72, 125, 158, 298, 261]


def yolov3_tiny(height: int = 416, width: int = 416, classes: int = 80) -> dict:
    head = 3 * (classes + 5)
    L: List[dict] = []
    for i, f in enumerate([16, 32, 64, 128, 256, 512]):
        L.append(_conv(f, 3))
        L.append({"type": "maxpool", "kernel": 2, "stride": 2 if i < 5 else 1})
    L += [_conv(1024, 3), _conv(256, 1), _conv(512, 3), _conv(head, 1, act="linear", bn=False),
          _yolo([3, 4, 5], V3_TINY_ANCHORS, 6),
          {"type": "route", "layers": [-4]}, _conv(128, 1), {"type": "upsample", "stride": 2},
          {"type": "route", "layers": [-1, 8]}, _conv(256, 3), _conv(head, 1, act="linear", bn=False),
          _yolo([0, 1, 2], V3_TINY_ANCHORS, 6)]
    return _doc(L, height, width)


def yolov3(height: int = 416, width: int = 416, classes: int = 80) -> dict:
    """Darknet-53 backbone (52 convolutions, 23 residual shortcuts) + 3-scale FPN head."""
    head = 3 * (classes + 5)
    L: List[dict] = [_conv(32, 3)]
    for filters, blocks in [(64, 1), (128, 2), (256, 8), (512, 8), (1024, 4)]:
        L.append(_conv(filters, 3, 2))
        for _ in range(blocks):
            L += [_conv(filters // 2, 1), _conv(filters, 3), {"type": "shortcut", "from": -3, "activation": "linear"}]
    for scale, (filters, mask, lateral) in enumerate([(512, [6, 7, 8], None), (256, [3, 4, 5], 61), (128, [0, 1, 2], 36)]):
        if lateral is not None:
            L += [{"type": "route", "layers": [-4]}, _conv(filters, 1), {"type": "upsample", "stride": 2},
                  {"type": "route", "layers": [-1, lateral]}]
        for _ in range(3):
            L += [_conv(filters, 1), _conv(filters * 2, 3)]
        L += [_conv(head, 1, act="linear", bn=False), _yolo(mask, V3_ANCHORS, 9)]
    return _doc(L, height, width)


def yolov7(height: int = 416, width: int = 416, classes: int = 80) -> dict:
    head = 3 * (classes + 5)
    c = lambda f, k, s=1: _conv(f, k, s, act="swish")
    route = lambda *ls: {"type": "route", "layers": list(ls)}
    mp = lambda k, s: {"type": "maxpool", "kernel": k, "stride": s}
    L: List[dict] = [c(32, 3), c(64, 3, 2), c(64, 3), c(128, 3, 2)]

    def elan(width_, out):
        L.extend([c(width_, 1), route(-2), c(width_, 1), c(width_, 3), c(width_, 3), c(width_, 3), c(width_, 3),
                  route(-1, -3, -5, -7), c(out, 1)])

    def transition(width_):
        L.extend([mp(2, 2), c(width_, 1), route(-3), c(width_, 1), c(width_, 3, 2), route(-1, -4)])

    elan(64, 256)
    transition(128)
    elan(128, 512)
    transition(256)
    elan(256, 1024)
    transition(512)
    elan(256, 1024)
    # SPPCSPC
    L.extend([c(512, 1), route(-2), c(512, 1), c(512, 3), c(512, 1), mp(5, 1), route(-2), mp(9, 1), route(-4),
              mp(13, 1), route(-6, -5, -3, -1), c(512, 1), c(512, 3), route(-1, -13), c(512, 1)])

    def elan_w(width_, out):
        half = width_ // 2
        L.extend([c(width_, 1), route(-2), c(width_, 1), c(half, 3), c(half, 3), c(half, 3), c(half, 3),
                  route(-1, -2, -3, -4, -5, -7), c(out, 1)])

    L.extend([c(256, 1), {"type": "upsample", "stride": 2}, route(42), c(256, 1), route(-1, -3)])
    elan_w(256, 256)
    L.extend([c(128, 1), {"type": "upsample", "stride": 2}, route(27), c(128, 1), route(-1, -3)])
    elan_w(128, 128)

    def down(width_, lateral):
        L.extend([mp(2, 2), c(width_, 1), route(-3), c(width_, 1), c(width_, 3, 2), route(-1, -4, lateral)])

    down(128, 86)
    elan_w(256, 256)
    down(256, 72)
    elan_w(512, 512)
    for src, filters, mask in [(100, 256, [0, 1, 2]), (115, 512, [3, 4, 5]), (130, 1024, [6, 7, 8])]:
        L.extend([route(src), c(filters, 3), _conv(head, 1, act="linear", bn=False), _yolo(mask, V7_ANCHORS, 9)])
    return _doc(L, height, width)


def centernet_tiny(height: int = 320, width: int = 320, classes: int = 20) -> dict:
    c = lambda f, k, s=1: _conv(f, k, s, act="mish", pad=(k == 3))
    L: List[dict] = [c(32, 3, 2), c(64, 3, 2), c(128, 3, 2), c(128, 3), c(256, 3, 2), c(256, 3), c(384, 3, 2), c(384, 3)]
    for filters, lateral in [(256, 5), (128, 3), (64, 1)]:
        L += [c(filters, 1), {"type": "upsample", "stride": 2}, {"type": "route", "layers": [-1, lateral]},
              c(max(128, filters), 3)]
    L += [c(64, 3), _conv(classes + 4, 1, act="linear", bn=False, pad=False),
          {"type": "centernet", "heatmap_bias": -2.19, "max_detections": 100}]
    return _doc(L, height, width)


PRESETS = {"yolov3-tiny": yolov3_tiny, "yolov3": yolov3, "yolov7": yolov7, "centernet-tiny": centernet_tiny}
