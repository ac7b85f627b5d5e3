"""Pins the CPU oracle against the known-answer cases the reference's own unit tests hold for this
path.  Expected values are derived here in float64 / closed form.

Reference cases covered (paths inside trieck/pixienn):
  tests/src/activations.cpp  apply() on {1,-2,3,-4} for all nine activations
  tests/src/maxpool.cpp      3x3, kernel 2, stride 1, padding 1
  tests/src/blas.cpp         addBias, scaleBias
  tests/src/math.cpp         softmax, sigmoid
  tests/src/yolo_cuda.cpp    1x1 head decode, yoloActivate values
  tests/src/centernet.cpp    4x4 heatmap decode (prob 0.982014, box 0.125/0.375/0.5/0.25)
  tests/src/box.cpp          five NMS cases
"""
import math

import numpy as np
import pytest

X = np.array([1.0, -2.0, 3.0, -4.0], np.float32)


def f64_act(kind, x):
    x = np.asarray(x, np.float64)
    sig = lambda t: 1.0 / (1.0 + np.exp(-t))
    sp = lambda t: np.where(t > 20, t, np.where(t < -20, np.exp(t), np.log1p(np.exp(t))))
    return {
        "leaky": np.where(x > 0, x, 0.1 * x), "linear": x, "loggy": 2.0 * sig(x) - 1.0, "logistic": sig(x),
        "mish": x * np.tanh(sp(x)), "relu": np.maximum(x, 0), "softplus": sp(x), "swish": x * sig(x),
        "tanh": np.tanh(x),
    }[kind]


@pytest.mark.parametrize("kind", ["leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"])
def test_activation_known_answers(oracle, kind):
    got = oracle.activate(kind, X)
    np.testing.assert_allclose(got, f64_act(kind, X), rtol=4 * 1.2e-7, atol=1e-7)
    if kind == "mish":       # the two values the reference test spells out
        assert abs(got[0] - 0.865098) < 1e-5 and abs(got[1] + 0.252502) < 1e-5


def test_activation_softplus_branches(oracle):
    x = np.array([20.5, -20.5, 19.5, -19.5], np.float32)
    got = oracle.activate("softplus", x)
    assert got[0] == x[0]
    assert got[1] == np.float32(math.exp(-20.5))
    np.testing.assert_allclose(got[2:], np.log1p(np.exp(x[2:].astype(np.float64))), rtol=1e-6, atol=1e-7)


def test_maxpool_known_answer(oracle):
    x = np.arange(1, 10, dtype=np.float32).reshape(1, 1, 3, 3)
    v, i = oracle.maxpool(x, 2, 1, 1)
    assert v.ravel().tolist() == [5, 6, 6, 8, 9, 9, 8, 9, 9]
    assert i.ravel().tolist() == [4, 5, 5, 7, 8, 8, 7, 8, 8]


def test_maxpool_geometry_defaults(oracle):
    # padding defaults to kernel-1; origin -padding/2 truncates toward zero
    assert oracle.maxpool_out_dim(416, 2, 2, 1) == 208
    assert oracle.maxpool_out_dim(13, 2, 2, 1) == 7
    assert oracle.maxpool_out_dim(13, 2, 1, 1) == 13
    assert oracle.maxpool_out_dim(20, 13, 1, 12) == 20
    x = np.arange(25, dtype=np.float32).reshape(1, 1, 5, 5)
    v, _ = oracle.maxpool(x, 3, 1)            # 'same' pooling, origin -1
    assert v[0, 0, 0, 0] == 6 and v[0, 0, 4, 4] == 24 and v[0, 0, 2, 2] == 18


def test_add_bias_and_scale_bias(oracle):
    out = np.arange(12, dtype=np.float32).reshape(1, 3, 2, 2)
    bias = np.array([1.0, 2.0, 3.0], np.float32)
    got = oracle.conv_epilogue(out, bias=bias, act="linear")
    assert np.array_equal(got, out + bias.reshape(1, 3, 1, 1))
    y = out.copy()
    oracle.lib().pxo_scale_bias(y.ctypes.data_as(oracle._f), bias.ctypes.data_as(oracle._f), 1, 3, 4)
    assert np.array_equal(y, out * bias.reshape(1, 3, 1, 1))


def test_batchnorm_inference_formulas(oracle):
    x = np.array([[[[0.5, -1.5]], [[2.0, 4.0]]]], np.float32)
    g, b = np.array([1.5, 0.5], np.float32), np.array([0.1, -0.2], np.float32)
    m, v = np.array([0.25, 1.0], np.float32), np.array([4.0, 0.25], np.float32)
    x64, g64, b64, m64, v64 = (t.astype(np.float64) for t in (x, g, b, m, v))
    sh = (1, 2, 1, 1)
    cudnn = g64.reshape(sh) * (x64 - m64.reshape(sh)) / np.sqrt(v64.reshape(sh) + 1e-5) + b64.reshape(sh)
    cpu = g64.reshape(sh) * (x64 - m64.reshape(sh)) / (np.sqrt(v64.reshape(sh)) + 1e-5) + b64.reshape(sh)
    np.testing.assert_allclose(oracle.conv_epilogue(x, g, b, m, v, eps_mode=0), cudnn, rtol=1e-6)
    np.testing.assert_allclose(oracle.conv_epilogue(x, g, b, m, v, eps_mode=1), cpu, rtol=1e-6)
    assert np.abs(cudnn - cpu).max() > 0       # the two placements of epsilon really differ


def test_softmax_and_sigmoid(oracle):
    x = np.array([1.0, 2.0, 3.0], np.float32)
    e = np.exp(x.astype(np.float64) - 3.0)
    np.testing.assert_allclose(oracle.softmax_one(x), e / e.sum(), rtol=1e-6)
    np.testing.assert_allclose(oracle.softmax_one(x, 2.0), np.exp(x / 2.0) / np.exp(x / 2.0).sum(), rtol=1e-6)
    assert abs(oracle.softmax_one(x).sum() - 1.0) < 1e-6
    big = np.array([1000.0, 1000.0], np.float32)                 # max-subtraction keeps it finite
    assert np.array_equal(oracle.softmax_one(big), np.array([0.5, 0.5], np.float32))
    assert oracle.activate("logistic", np.array([0.0], np.float32))[0] == 0.5


def test_yolo_activate_values(oracle):
    raw = np.array([0, 0, 0, 0, 0, -1, 1], np.float32).reshape(1, 7, 1, 1)
    out = oracle.yolo_activate(raw, 1, 2).ravel()
    assert out[:5].tolist() == [0.5, 0.5, 0.0, 0.0, 0.5]
    assert abs(out[5] - 1 / (1 + math.e)) < 1e-6 and abs(out[6] - 1 / (1 + 1 / math.e)) < 1e-6


def test_yolo_decode_1x1(oracle):
    raw = np.array([0.2, -0.4, 0.1, -0.2, 2.0, 1.5], np.float32).reshape(1, 6, 1, 1)
    act = oracle.yolo_activate(raw, 1, 1)
    dets, total = oracle.yolo_decode(act, [0], [1, 1], 1, 1, 1, 0.1)
    assert total == 1
    sig = lambda t: 1 / (1 + math.exp(-t))
    d = dets[0]
    w, h = math.exp(0.1), math.exp(-0.2)
    assert abs(d["prob"] - sig(2.0) * sig(1.5)) < 1e-6
    assert abs(d["w"] - w) < 1e-6 and abs(d["h"] - h) < 1e-6
    assert abs(d["x"] - (sig(0.2) - w / 2)) < 1e-6 and abs(d["y"] - (sig(-0.4) - h / 2)) < 1e-6


def test_yolo_decode_order_threshold_rules(oracle):
    """Emission order cell -> mask slot -> class; skip on obj < thr; emit on obj*cls >= thr."""
    masks, classes, H, W = 2, 2, 1, 2
    pred = np.zeros((1, masks * (classes + 5), H, W), np.float32)
    v = pred.reshape(masks, classes + 5, H * W)
    v[:, 4, :] = [[0.9, 0.5], [0.19, 1.0]]        # objectness [mask][cell]
    v[:, 5, :] = 0.5
    v[:, 6, :] = [[0.1, 0.4], [1.0, 0.2]]
    dets, total = oracle.yolo_decode(pred, [0, 1], [10, 10, 20, 20], classes, 100, 100, 0.2)
    got = [(int(d["source"]), int(d["class_id"]), round(float(d["prob"]), 4)) for d in dets]
    # cell0: slot0 obj .9 -> cls0 .45; cls1 .09 no.  slot1 obj .19 < thr skipped entirely.
    # cell1: slot0 obj .5 -> cls0 .25, cls1 .2 (== thr, kept); slot1 obj 1 -> cls0 .5, cls1 .2
    assert got == [(0, 0, 0.45), (2, 0, 0.25), (2, 1, 0.2), (3, 0, 0.5), (3, 1, 0.2)]
    assert total == 5


def test_centernet_known_answer(oracle):
    area = 16
    inp = np.zeros((1, 5, 4, 4), np.float32)
    inp[0, 0] = -10.0
    flat = inp.reshape(5, area)
    idx = 2 * 4 + 1
    flat[0, idx], flat[1, idx], flat[2, idx], flat[3, idx], flat[4, idx] = 4.0, 2.0, 1.0, 0.5, 0.0
    act = oracle.centernet_activate(inp, 1, 0.0)
    dets, ncand = oracle.centernet_decode(act[:, :1], act[:, 1:3], act[:, 3:], 0.5, 10)
    d = dets[0]
    assert len(d) == 1 and ncand == [1] and d["class_id"][0] == 0
    assert abs(d["prob"][0] - 0.982014) < 1e-5
    assert abs(d["x"][0] - 0.125) < 1e-6 and abs(d["y"][0] - 0.375) < 1e-6
    assert abs(d["w"][0] - 0.5) < 1e-6 and abs(d["h"][0] - 0.25) < 1e-6


def D(oracle, x, y, w, h, batch, cls, prob, source=0):
    return oracle.make_det(x, y, w, h, batch, cls, prob, source)


def test_nms_reference_cases(oracle):
    cat = np.concatenate
    # same class: duplicate suppressed, distant box kept
    r = oracle.nms(cat([D(oracle, 100, 100, 50, 50, 0, 1, .9), D(oracle, 100, 100, 50, 50, 0, 1, .8),
                        D(oracle, 200, 200, 50, 50, 0, 1, .7)]), 0.5)
    assert len(r) == 2 and r["x"].tolist() == [100, 200]
    # no suppression across images
    r = oracle.nms(cat([D(oracle, 100, 100, 50, 50, 0, 1, .9), D(oracle, 100, 100, 50, 50, 1, 1, .8)]), 0.5)
    assert len(r) == 2
    # near-identical boxes of different classes: the stronger one survives
    r = oracle.nms(cat([D(oracle, 100, 100, 50, 50, 0, 16, .9), D(oracle, 100, 100, 50, 50, 0, 15, .8)]), 0.3)
    assert len(r) == 1 and r["class_id"][0] == 16 and r["prob"][0] == np.float32(0.9)
    # ordinary overlap of different classes is kept (IoU 45*45/(2*2500-2025) = 0.68 < 0.9)
    r = oracle.nms(cat([D(oracle, 100, 100, 50, 50, 0, 16, .9), D(oracle, 105, 105, 50, 50, 0, 15, .8)]), 0.3)
    assert len(r) == 2
    # a suppressed box must not suppress others: IoU(a,b)=.6, IoU(b,c)=.6, IoU(a,c)=1/3
    r = oracle.nms(cat([D(oracle, 0, 0, 100, 100, 0, 1, .9), D(oracle, 25, 0, 100, 100, 0, 1, .8),
                        D(oracle, 50, 0, 100, 100, 0, 1, .7)]), 0.5)
    assert len(r) == 2 and r["x"].tolist() == [0, 50]


def test_box_iou(oracle):
    a, b = D(oracle, 0, 0, 2, 2, 0, 0, 1), D(oracle, 1, 1, 2, 2, 0, 0, 1)
    assert abs(oracle.box_iou(a, b) - 1 / 7) < 1e-6
    assert oracle.box_iou(a, D(oracle, 5, 5, 1, 1, 0, 0, 1)) == 0.0
    assert oracle.box_iou(a, D(oracle, 0, 0, 0, 0, 0, 0, 1)) == 0.0      # 0/0 -> 0
    assert abs(oracle.box_iou(D(oracle, 2, 2, -2, -2, 0, 0, 1), a) - 1.0) < 1e-6   # negative extents normalised


def test_upsample_shortcut_route_semantics(oracle):
    x = np.arange(8, dtype=np.float32).reshape(1, 2, 2, 2)
    up = oracle.upsample(x, 2, 0.5)
    assert up.shape == (1, 2, 4, 4) and np.array_equal(up[0, 1, 2:, :2], np.full((2, 2), 3.0, np.float32))
    a, b = np.ones((2, 2, 2, 2), np.float32), np.full((2, 2, 2, 2), 2.0, np.float32)
    assert np.array_equal(oracle.shortcut(a, b, 1.0, 1.0, "linear"), np.full_like(a, 3.0))
    assert np.array_equal(oracle.shortcut(-a, -b, 1.0, 1.0, "leaky"), np.full_like(a, np.float32(0.1) * np.float32(-3.0)))
    s0 = np.arange(2 * 1 * 2, dtype=np.float32).reshape(2, 1, 1, 2)
    s1 = 10 + np.arange(2 * 2 * 2, dtype=np.float32).reshape(2, 2, 1, 2)
    assert np.array_equal(oracle.route([s0, s1]), np.concatenate([s0, s1], 1))


def test_region_forward_layout(oracle):
    B, num, coords, classes, H, W = 1, 2, 4, 3, 2, 2
    size = coords + 1 + classes
    x = np.arange(B * num * size * H * W, dtype=np.float32).reshape(B, num * size, H, W) / 10
    out = oracle.region_forward(x, num, coords, classes, True).reshape(H * W, num, size)
    for cell in range(H * W):
        for n in range(num):
            src = x.reshape(num, size, H * W)[n, :, cell].astype(np.float64)
            np.testing.assert_allclose(out[cell, n, :4], src[:4], rtol=1e-6)
            np.testing.assert_allclose(out[cell, n, 4], 1 / (1 + np.exp(-src[4])), rtol=1e-6)
            e = np.exp(src[5:] - src[5:].max())
            np.testing.assert_allclose(out[cell, n, 5:], e / e.sum(), rtol=1e-6)


def test_avgpool_is_the_plane_mean_in_index_order(oracle):
    """AvgPoolLayer::forward (include/AvgPoolLayer.h:66-87): running float sum over the plane, one division."""
    x = np.arange(2 * 3 * 2 * 2, dtype=np.float32).reshape(2, 3, 2, 2)
    out = oracle.avgpool(x)
    assert out.shape == (2, 3, 1, 1)
    assert np.array_equal(out.ravel(), np.array([1.5, 5.5, 9.5, 13.5, 17.5, 21.5], np.float32))
    # order matters in float: 1e8 + 1 - 1e8 summed left to right loses the 1
    y = np.array([1e8, 1.0, -1e8, 0.0], np.float32).reshape(1, 1, 2, 2)
    assert oracle.avgpool(y).ravel()[0] == 0.0


def test_yolov1_detection_decode_known_answer(oracle):
    """DetectLayer::addDetects (include/DetectLayer.h:166-209) on a 2x2 grid, one box per cell, two classes:
    cell 3 (row 1, col 1) has scale 0.8 and class scores (0.25, 0.5); squared sizes."""
    side, num, classes = 2, 1, 2
    loc = side * side
    pred = np.zeros(loc * (classes + num * 5), np.float32)
    pred[3 * classes + 0], pred[3 * classes + 1] = 0.25, 0.5
    pred[loc * classes + 3] = 0.8                                  # scale of cell 3
    pred[loc * classes + 1] = -0.5                                 # a negative scale emits nothing
    box = loc * (classes + num) + 3 * 4
    pred[box:box + 4] = [0.5, 0.25, 0.5, 0.4]
    dets, n = oracle.detect_decode(pred[None], side, num, classes, 0.3, squared=True)
    assert n == 1
    d = dets[0]
    assert d["class_id"] == 1 and d["batch_id"] == 0 and d["source"] == 3
    assert abs(d["prob"] - 0.4) < 1e-7
    w, h = 0.25, 0.16000001
    assert abs(d["w"] - w) < 1e-6 and abs(d["h"] - h) < 1e-6
    assert abs(d["x"] - ((0.5 + 1) / 2 - w / 2)) < 1e-6 and abs(d["y"] - ((0.25 + 1) / 2 - h / 2)) < 1e-6
    assert oracle.detect_decode(pred[None], side, num, classes, 0.41, squared=True)[1] == 0
