"""Graph builders, shape propagation and the fusion plan (CPU only)."""
import os

import pytest
import yaml

from oracle.pxoracle import reference_root
from pixienn_b200 import graph, presets

# the reference's model files, where its tree is present ($PXE_REFERENCE_ROOT, or a checkout beside this repository)
REF_MODELS = os.path.join(reference_root() or "", "resources", "models")
KEYS = ["type", "activation", "batch_normalize", "filters", "kernel", "pad", "stride", "layers", "from", "mask",
        "anchors", "num", "padding", "dilation", "groups", "heatmap_bias", "max_detections"]


def essential(ld, t):
    d = {k: ld[k] for k in KEYS if k in ld}
    if t == "conv":
        d.setdefault("batch_normalize", False)
        d.setdefault("dilation", 1)
    return d


@pytest.mark.parametrize("name,file", [("yolov3-tiny", "yolov3-tiny.yml"), ("yolov3", "yolov3.yml"),
                                       ("yolov7", "yolov7.yml"), ("centernet-tiny", "centernet-tiny-voc.yml")])
def test_builders_equal_reference_graphs(name, file):
    path = os.path.join(REF_MODELS, file)
    if not os.path.exists(path):
        pytest.skip("no reference checkout")
    ref = yaml.safe_load(open(path))["model"]
    mine = presets.PRESETS[name](ref["height"], ref["width"])["model"]
    assert len(mine["layers"]) == len(ref["layers"])
    for i, (a, b) in enumerate(zip(mine["layers"], ref["layers"])):
        assert essential(a, a["type"]) == essential(b, b["type"]), f"layer {i}"


def test_shapes_yolov3_608():
    m = graph.parse_model(presets.yolov3(608, 608))
    assert len(m.layers) == 107 and m.classes == 80
    heads = [l for l in m.layers if l.type == "yolo"]
    assert [l.in_shape for l in heads] == [(255, 19, 19), (255, 38, 38), (255, 76, 76)]
    assert m.layers[86].out_shape == (768, 38, 38) and m.layers[98].out_shape == (384, 76, 76)
    assert sum(1 for l in m.layers if l.type == "conv") == 75 and sum(1 for l in m.layers if l.type == "shortcut") == 23


def test_shapes_tiny_416_and_v7_640():
    m = graph.parse_model(presets.yolov3_tiny())
    assert m.layers[11].out_shape == (512, 13, 13)            # maxpool k2 s1 keeps 13x13
    assert m.layers[9].out_shape == (256, 13, 13) and m.layers[20].out_shape == (384, 26, 26)
    m7 = graph.parse_model(presets.yolov7(640, 640))
    assert len(m7.layers) == 143
    assert [l.in_shape[1] for l in m7.layers if l.type == "yolo"] == [80, 40, 20]
    assert m7.layers[68].out_shape == (2048, 20, 20)
    m7b = graph.parse_model(presets.yolov7())                 # 416: odd extents 13, 26, 52
    assert m7b.layers[68].out_shape == (2048, 13, 13)


def test_plan_yolov3_fuses_every_shortcut_and_eliminates_routes():
    p = graph.plan(graph.parse_model(presets.yolov3(608, 608)))
    assert p.stats["fused_shortcut"] == 23 and p.stats["raw_heads"] == 3
    assert p.stats["routes_aliased"] == 2 and p.stats["routes_eliminated"] == 2 and p.stats["concat_copies"] == 0
    ops = [s.op for s in p.steps]
    assert ops.count("conv") == 75 and "shortcut" not in ops and "concat" not in ops
    # layer 61 (a fused conv+shortcut) feeds the next conv AND the 768-channel route: two stores
    st = [s for s in p.steps if 61 in s.produces][0]
    assert [d.kind for d in st.dests] == ["dense", "slot"] and st.dests[1].route == 86 and st.dests[1].offset == 256
    up = [s for s in p.steps if s.op == "upsample"][0]
    assert [d.kind for d in up.dests] == ["slot"] and up.dests[0].offset == 0


def test_plan_tiny_folds_pools():
    p = graph.plan(graph.parse_model(presets.yolov3_tiny()))
    assert p.stats["fused_pool"] == 5
    st8 = [s for s in p.steps if s.op == "conv" and s.layer == 8][0]
    assert st8.fused_pool == 9 and st8.keep_full and [d.kind for d in st8.dests] == ["slot"]
    st0 = [s for s in p.steps if s.op == "conv" and s.layer == 0][0]
    assert st0.fused_pool == 1 and not st0.keep_full and st0.dests == []
    assert [s.op for s in p.steps if s.layer == 11] == ["maxpool"]      # k2/s1 stays a separate launch


def test_plan_yolov7_spp_and_routes():
    p = graph.plan(graph.parse_model(presets.yolov7(640, 640)))
    assert p.stats["spp_blocks"] == 1 and p.stats["concat_copies"] == 0
    spp = [s for s in p.steps if s.op == "spp"][0]
    assert spp.spp_layers == [63, 65, 67] and spp.inputs == [62]
    assert p.stats["routes_aliased"] + p.stats["routes_eliminated"] == 38
    unfused = graph.plan(graph.parse_model(presets.yolov7(640, 640)), fuse=False)
    assert unfused.stats["concat_copies"] == 38 and len(unfused.steps) == 143
