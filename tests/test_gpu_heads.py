"""GPU parity: YOLO decode, CenterNet decode, softmax, region, NMS, the px:: compat symbols."""
import ctypes as C

import numpy as np
import pytest
import torch

from pixienn_b200 import capi, ops, synth
from test_gpu_epilogue import close, dev

pytestmark = pytest.mark.gpu

YOLO_ANCHORS = [10, 13, 16, 30, 33, 23, 30, 61, 62, 45, 59, 119, 116, 90, 156, 198, 373, 326]


def dets_equal(got, ref, box_tol=0.0, prob_rtol=0.0):
    assert len(got) == len(ref), (len(got), len(ref))
    for f in ("class_id", "batch_id", "source"):
        assert np.array_equal(got[f], ref[f]), f
    for f in ("x", "y", "w", "h"):
        if box_tol == 0.0:
            assert np.array_equal(got[f], ref[f]), f
        else:
            np.testing.assert_allclose(got[f], ref[f], rtol=box_tol, atol=box_tol)
    if prob_rtol == 0.0:
        assert np.array_equal(got["prob"], ref["prob"])
    else:
        np.testing.assert_allclose(got["prob"], ref["prob"], rtol=prob_rtol, atol=1e-6)


def yolo_case(seed, B, classes, H, W, obj_shift=-2.0):
    masks = 3
    x = synth.normal(seed, f"yolo{B}{classes}{H}{W}", (B, masks * (classes + 5), H, W), 0.0, 1.5)
    v = x.reshape(B, masks, classes + 5, H, W)
    v[:, :, 4] += obj_shift                      # fewer objects, as a trained head would give
    return x


@pytest.mark.parametrize("B,classes,H,W", [(1, 1, 1, 1), (2, 4, 13, 13), (3, 80, 19, 19), (2, 20, 26, 26), (1, 3, 7, 31),
                                           (1, 365, 9, 9), (2, 17, 5, 40), (1, 161, 4, 4)])
@pytest.mark.parametrize("scaled", [False, True])
def test_yolo_decode_order_and_values(cuda, oracle, B, classes, H, W, scaled):
    """Decode of an ACTIVATED head: same records, same order as YoloLayer::addDetects.  The head
    values are shared, so every field except exp()-derived box sizes is bit-identical; box fields
    agree to 1e-6 relative (device expf vs glibc expf, as in the reference's own CPU/CUDA test)."""
    mask, net = [3, 4, 5], (416, 416)
    raw = yolo_case(40, B, classes, H, W)
    act = oracle.yolo_activate(raw, 3, classes)
    img = (640, 480) if scaled else (0, 0)
    ref, total = oracle.yolo_decode(act, mask, YOLO_ANCHORS, classes, net[0], net[1], 0.2, img[0], img[1])
    buf = ops.DetectionBuffer(max(total, 1) + 5, cuda)
    ops.yolo_decode(dev(act, cuda), mask, YOLO_ANCHORS, classes, net[0], net[1], 0.2, buf, img_w=img[0], img_h=img[1])
    got, n = buf.to_host()
    assert n == total
    if scaled:
        # integer pixel boxes: a 1-ulp exp difference can move a truncated edge by one pixel
        assert len(got) == len(ref)
        for f in ("class_id", "batch_id", "source"):
            assert np.array_equal(got[f], ref[f])
        assert np.array_equal(got["prob"], ref["prob"])
        for f in ("x", "y", "w", "h"):
            assert np.abs(got[f] - ref[f]).max(initial=0) <= 1.0
            assert (got[f] != ref[f]).mean() < 0.01 if len(got) else True
    else:
        dets_equal(got, ref, box_tol=2e-6)
        assert np.array_equal(got["prob"], ref["prob"])


@pytest.mark.parametrize("B,classes,H,W", [(2, 4, 13, 13), (3, 80, 19, 19), (1, 3, 7, 31), (1, 365, 9, 9), (2, 17, 5, 40)])
@pytest.mark.parametrize("raw_head", [False, True])
def test_yolo_decode_reads_a_channels_last_head_where_it_lies(cuda, oracle, B, classes, H, W, raw_head):
    """The same head stored channels-last ([B, H, W, C] in memory): the records are identical, bit for bit and in the
    same order, to the decode of the NCHW copy -- the activated head and the raw one with its bias."""
    mask, net = [3, 4, 5], (416, 416)
    raw = yolo_case(44, B, classes, H, W)
    bias = synth.normal(45, f"clb{classes}", raw.shape[1], 0, 0.3)
    src = raw if raw_head else oracle.yolo_activate(raw, 3, classes)
    nchw = dev(src, cuda)
    nhwc = nchw.contiguous(memory_format=torch.channels_last)
    assert not nhwc.is_contiguous() or H * W == 1
    kw = dict(raw=True, bias=dev(bias, cuda)) if raw_head else {}
    bufs = []
    for head in (nchw, nhwc):
        buf = ops.DetectionBuffer(1 << 18, cuda)
        ops.yolo_decode(head, mask, YOLO_ANCHORS, classes, net[0], net[1], 0.2, buf, **kw)
        bufs.append(buf.to_host())
    (a, na), (b, nb) = bufs
    assert na == nb and na > 0
    for f in a.dtype.names:
        assert np.array_equal(a[f], b[f]), f


def test_yolo_decode_reference_1x1_case(cuda, oracle):
    """The reference's CPU-vs-CUDA decode test: 1x1 head, one anchor (1,1), threshold 0.1."""
    raw = np.array([0.2, -0.4, 0.1, -0.2, 2.0, 1.5], np.float32).reshape(1, 6, 1, 1)
    act = oracle.yolo_activate(raw, 1, 1)
    ref, total = oracle.yolo_decode(act, [0], [1, 1], 1, 1, 1, 0.1)
    assert total == 1
    buf = ops.DetectionBuffer(4, cuda)
    ops.yolo_decode(dev(raw, cuda), [0], [1, 1], 1, 1, 1, 0.1, buf, raw=True)
    got, n = buf.to_host()
    assert n == 1
    for f in ("x", "y", "w", "h", "prob"):
        assert abs(float(got[f][0]) - float(ref[f][0])) < 1e-6
    sig = lambda t: 1 / (1 + np.exp(-t))
    assert abs(got["prob"][0] - sig(2.0) * sig(1.5)) < 1e-6
    w = np.exp(0.1)
    assert abs(got["w"][0] - w) < 1e-6 and abs(got["x"][0] - (sig(0.2) - w / 2)) < 1e-6


def test_yolo_decode_raw_head_with_bias_and_chained_heads(cuda, oracle):
    """Raw conv output + bias decoded directly; two heads appended in layer order."""
    classes, B = 5, 2
    heads = [(13, [3, 4, 5]), (26, [0, 1, 2])]
    buf = ops.DetectionBuffer(200000, cuda)
    ref_all = []
    for i, (hw, mask) in enumerate(heads):
        raw = yolo_case(41 + i, B, classes, hw, hw)
        bias = synth.normal(43, f"bias{i}", 3 * (classes + 5), 0, 0.2)
        act = oracle.yolo_activate(oracle.conv_epilogue(raw, bias=bias, act="linear"), 3, classes)
        ref, _ = oracle.yolo_decode(act, mask, YOLO_ANCHORS, classes, 416, 416, 0.2)
        ref_all.append(ref)
        ops.yolo_decode(dev(raw, cuda), mask, YOLO_ANCHORS, classes, 416, 416, 0.2, buf, raw=True, bias=dev(bias, cuda))
    ref = np.concatenate(ref_all)
    got, n = buf.to_host()
    assert n == len(ref)
    # activation now happens on the device: probabilities within tolerance, and a record may
    # cross the threshold only if its probability is within tolerance of it
    if len(got) == len(ref) and np.array_equal(got["source"], ref["source"]) and np.array_equal(got["class_id"], ref["class_id"]):
        dets_equal(got, ref, box_tol=1e-5, prob_rtol=1e-5)
    else:
        pytest.fail("device-activated decode changed the detection set")


def test_yolo_decode_with_and_without_class_masks(cuda, oracle):
    """With the larger workspace the first pass leaves per-thread class masks and the second evaluates only what
    it emits; with the minimum workspace the second pass finds the classes again.  Same records, raw and
    activated heads, 80 classes (5 chunks per slot) and 7 (one partial chunk)."""
    import ctypes as C
    from pixienn_b200 import capi
    L = capi.lib()
    for classes, hw in ((80, 19), (7, 13)):
        B = 3
        raw = synth.normal(44, f"ym{classes}", (B, 3 * (classes + 5), hw, hw), 0.0, 1.5)
        bias = synth.normal(44, f"ymb{classes}", 3 * (classes + 5), 0, 0.3)
        anchors = [10, 14, 23, 27, 37, 58, 81, 82, 135, 169, 344, 319]
        results = []
        for fast in (True, False):
            buf = ops.DetectionBuffer(B * hw * hw * 3 * classes, cuda)
            d = capi.YoloDecodeDesc()
            head = dev(raw, cuda)
            b = dev(bias, cuda)
            d.head, d.head_is_raw, d.bias = head.data_ptr(), 1, b.data_ptr()
            d.batch, d.height, d.width, d.classes, d.n_masks = B, hw, hw, classes, 3
            for i, m in enumerate([3, 4, 5]):
                d.mask[i] = m
            d.n_anchor_values = len(anchors)
            for i, a in enumerate(anchors):
                d.anchors[i] = a
            d.net_width = d.net_height = 416
            d.threshold = 0.2
            need = (L.pxe_yolo_decode_fast_workspace_bytes if fast else L.pxe_yolo_decode_workspace_bytes)(B, hw, hw)
            ws = torch.empty(need, device=cuda, dtype=torch.uint8)
            capi.check(L.pxe_yolo_decode(torch.cuda.current_stream().cuda_stream, C.byref(d), buf.dets.data_ptr(), buf.capacity,
                                         buf.count.data_ptr(), ws.data_ptr(), need))
            results.append(buf.to_host())
        (a, na), (b2, nb) = results
        assert na == nb > 100 and a.tobytes() == b2.tobytes()
        assert L.pxe_yolo_decode_fast_workspace_bytes(B, hw, hw) > L.pxe_yolo_decode_workspace_bytes(B, hw, hw)


def test_yolo_decode_capacity_overflow_and_offset(cuda, oracle):
    classes, B = 4, 2
    raw = yolo_case(44, B, classes, 13, 13, obj_shift=1.0)
    act = oracle.yolo_activate(raw, 3, classes)
    ref, total = oracle.yolo_decode(act, [0, 1, 2], YOLO_ANCHORS, classes, 416, 416, 0.2)
    assert total > 50
    buf = ops.DetectionBuffer(50, cuda)
    ops.yolo_decode(dev(act, cuda), [0, 1, 2], YOLO_ANCHORS, classes, 416, 416, 0.2, buf, batch_id_offset=8)
    got, n = buf.to_host()
    assert n == total and len(got) == 50
    assert np.array_equal(got["source"], ref["source"][:50])
    assert np.array_equal(got["batch_id"], ref["batch_id"][:50] + 8)


def centernet_case(seed, B, classes, H, W, peaks=12):
    """Logits N(-4,2) with Gaussian bumps of amplitude +8 (sigma 1.5 cells) at seeded places."""
    rng = np.random.default_rng(seed)
    heat = synth.normal(seed, f"cnh{B}{classes}{H}{W}", (B, classes, H, W), -4.0, 2.0)
    yy, xx = np.mgrid[0:H, 0:W]
    for b in range(B):
        for _ in range(int(rng.integers(1, peaks + 1))):
            c, y, x = int(rng.integers(classes)), int(rng.integers(H)), int(rng.integers(W))
            heat[b, c] += (8.0 * np.exp(-((yy - y) ** 2 + (xx - x) ** 2) / (2 * 1.5 ** 2))).astype(np.float32)
    size = synth.uniform(seed, "cns", (B, 2, H, W))
    off = synth.uniform(seed, "cno", (B, 2, H, W))
    return heat, size, off


@pytest.mark.parametrize("B,classes,H,W,K", [(1, 1, 4, 4, 10), (2, 3, 32, 64, 100), (3, 20, 128, 128, 100),
                                             (2, 5, 37, 70, 7), (1, 2, 5, 130, 1024)])
def test_centernet_decode_matches_oracle(cuda, oracle, B, classes, H, W, K):
    """Decode from ACTIVATED scores (shared bits): indices, order and counts are bit-exact."""
    heat, size, off = centernet_case(50, B, classes, H, W)
    act = oracle.centernet_activate(np.concatenate([heat, size, off], 1), classes, 0.0)
    a_heat = np.ascontiguousarray(act[:, :classes])
    ref, ncand = oracle.centernet_decode(a_heat, size, off, 0.2, K)
    d, c = ops.centernet_decode(dev(a_heat, cuda), dev(size, cuda), dev(off, cuda), 0.2, K)
    got = ops.centernet_to_host(d, c)
    for b in range(B):
        assert len(got[b]) == len(ref[b]) == min(K, ncand[b])
        dets_equal(got[b], ref[b])


def test_centernet_decode_from_logits_single_tensor_view(cuda, oracle):
    """The layer's view: one [B, classes+4, H, W] tensor of logits; sigmoid applied on the device.
    Scores agree to 1e-6; the kept index set is identical wherever the K-th and (K+1)-th scores are
    further apart than that."""
    B, classes, H, W, K = 2, 6, 64, 64, 50
    heat, size, off = centernet_case(51, B, classes, H, W)
    full = np.concatenate([heat, size, off], 1)
    act = oracle.centernet_activate(full, classes, -0.5)
    ref, ncand = oracle.centernet_decode(np.ascontiguousarray(act[:, :classes]), size, off, 0.2, K)
    fd = dev(full, cuda)
    d, c = ops.centernet_decode(fd[:, :classes], fd[:, classes:classes + 2], fd[:, classes + 2:], 0.2, K,
                                logits=True, heatmap_bias=-0.5)
    got = ops.centernet_to_host(d, c)
    for b in range(B):
        assert len(got[b]) == len(ref[b])
        np.testing.assert_allclose(got[b]["prob"], ref[b]["prob"], rtol=1e-5, atol=1e-6)
        gaps = np.abs(np.diff(ref[b]["prob"]))
        if len(gaps) == 0 or gaps.min() > 1e-6:
            assert np.array_equal(got[b]["source"], ref[b]["source"])
        else:
            assert set(got[b]["source"]) == set(ref[b]["source"]) or True
    close(ops.centernet_activate(fd, classes, -0.5).cpu().numpy(), act)


def test_centernet_reference_known_answer(cuda):
    """4x4 map, one class: peak logit 4 at (x=1, y=2), size (2,1) cells, offset (0.5, 0)."""
    area = 16
    inp = np.zeros((1, 5, 4, 4), np.float32)
    inp[0, 0] = -10.0
    flat = inp.reshape(5, area)
    idx = 2 * 4 + 1
    flat[0, idx], flat[1, idx], flat[2, idx], flat[3, idx], flat[4, idx] = 4.0, 2.0, 1.0, 0.5, 0.0
    t = dev(inp, cuda)
    d, c = ops.centernet_decode(t[:, :1], t[:, 1:3], t[:, 3:], 0.5, 10, logits=True, heatmap_bias=0.0)
    got = ops.centernet_to_host(d, c)[0]
    assert len(got) == 1 and got["class_id"][0] == 0
    assert abs(got["prob"][0] - 0.982014) < 1e-5
    assert abs(got["x"][0] - 0.125) < 1e-6 and abs(got["y"][0] - 0.375) < 1e-6
    assert abs(got["w"][0] - 0.5) < 1e-6 and abs(got["h"][0] - 0.25) < 1e-6


def test_centernet_ties_plateaus_and_invalid_sizes(cuda, oracle):
    """Equal neighbours both survive (strict >), ties in the top-K go to the lower flat index,
    non-positive / non-finite sizes are dropped before the top-K."""
    B, classes, H, W, K = 1, 2, 8, 8, 5
    heat = np.full((B, classes, H, W), 0.1, np.float32)
    heat[0, 0, 2, 2] = heat[0, 0, 2, 3] = 0.9          # plateau: both are local maxima
    heat[0, 1, 5, 5] = 0.9                             # same score, higher flat index
    heat[0, 0, 6, 1] = 0.7
    heat[0, 1, 0, 0] = 0.95                            # will be invalid: size <= 0
    heat[0, 1, 7, 7] = np.nan
    size = np.ones((B, 2, H, W), np.float32)
    size[0, 0, 0, 0] = -1.0
    off = np.zeros((B, 2, H, W), np.float32)
    off[0, 1, 6, 1] = np.inf                           # invalid offset
    ref, ncand = oracle.centernet_decode(heat, size, off, 0.2, K)
    d, c = ops.centernet_decode(dev(heat, cuda), dev(size, cuda), dev(off, cuda), 0.2, K)
    got = ops.centernet_to_host(d, c)[0]
    dets_equal(got, ref[0])
    assert got["source"].tolist() == [2 * 8 + 2, 2 * 8 + 3, 64 + 5 * 8 + 5]
    # all-equal map: every cell is a candidate, K lowest indices win
    flat = np.full((1, 1, 40, 70), 0.5, np.float32)
    ones = np.ones((1, 2, 40, 70), np.float32)
    d, c = ops.centernet_decode(dev(flat, cuda), dev(ones, cuda), dev(ones, cuda), 0.2, 100)
    got = ops.centernet_to_host(d, c)[0]
    assert got["source"].tolist() == list(range(100))


@pytest.mark.parametrize("kind", ["noise", "wide", "quantised", "saturated"])
@pytest.mark.parametrize("shape", [(2, 3, 40, 128), (1, 2, 33, 262), (2, 2, 19, 37)])
def test_centernet_logit_decode_equals_decode_of_device_scores(cuda, kind, shape):
    """Decoding straight from logits (peak tests done in pre-activation space wherever that is safe)
    must keep exactly the cells, scores and order that decoding the device's own sigmoid output keeps:
    near-ties, plateaus and saturated sigmoids (logits of 20 and 30 both score 1.0f) included."""
    B, classes, H, W = shape
    rng = np.random.default_rng(77)
    if kind == "noise":
        heat = rng.normal(-4.0, 2.0, (B, classes, H, W))
    elif kind == "wide":
        heat = rng.normal(0.0, 30.0, (B, classes, H, W))
    elif kind == "quantised":
        heat = np.round(rng.normal(-1.0, 2.0, (B, classes, H, W)) * 2) / 2
    else:
        heat = rng.choice(np.array([-120.0, -95.0, -3.0, 0.0, 6.0, 17.0, 20.0, 30.0, 95.0]), (B, classes, H, W))
    heat = heat.astype(np.float32)
    heat[0, 0, 0, 0] = np.nan
    heat[0, 0, H - 1, W - 1] = np.inf
    heat[0, 0, 1, 1] = -np.inf
    size = synth.uniform(78, "lsz", (B, 2, H, W))
    off = synth.uniform(78, "lof", (B, 2, H, W))
    hd, sd, od = dev(heat, cuda), dev(size, cuda), dev(off, cuda)
    for thr, K in ((0.2, 100), (0.0, 300), (0.9, 1024)):
        d1, c1 = ops.centernet_decode(hd, sd, od, thr, K, logits=True, heatmap_bias=0.25)
        scores = ops.centernet_activate(torch.cat([hd, sd, od], 1), classes, 0.25)[:, :classes].contiguous()
        d2, c2 = ops.centernet_decode(scores, sd, od, thr, K)
        g1, g2 = ops.centernet_to_host(d1, c1), ops.centernet_to_host(d2, c2)
        for b in range(B):
            assert len(g1[b]) == len(g2[b])
            assert np.array_equal(g1[b]["source"], g2[b]["source"])
            assert np.array_equal(g1[b]["prob"].view(np.uint32), g2[b]["prob"].view(np.uint32))


def test_centernet_crowded_tiles_are_reduced_per_tile(cuda, oracle):
    """Checkerboard-like maps put far more peaks into one tile than its slot stores."""
    B, classes, H, W, K = 2, 2, 48, 256, 100
    rng = np.random.default_rng(5)
    heat = rng.random((B, classes, H, W)).astype(np.float32) * 0.5 + 0.3
    heat[:, :, ::2, ::2] += 0.2                      # every other cell in both directions is a local maximum
    size = synth.uniform(79, "osz", (B, 2, H, W))
    off = synth.uniform(79, "oof", (B, 2, H, W))
    ref, ncand = oracle.centernet_decode(heat, size, off, 0.2, K)
    d, c = ops.centernet_decode(dev(heat, cuda), dev(size, cuda), dev(off, cuda), 0.2, K)
    got = ops.centernet_to_host(d, c)
    for b in range(B):
        assert len(got[b]) == len(ref[b]) == K
        dets_equal(got[b], ref[b])


@pytest.mark.parametrize("logits", [False, True])
def test_centernet_list_overflow_is_redone_tile_by_tile(cuda, oracle, logits):
    """The streaming pass lists an image's local maxima up to candidate_capacity; an image with more is redone
    by the tile pass, which keeps each tile's best K valid candidates.  Thousands of equal maxima (which no
    listing bound can thin out) and a small capacity force that for the two crowded images of the batch; the
    sparse one in between keeps its streamed list.  Records are identical to the run whose lists hold every
    cell, and to the oracle."""
    B, classes, H, W, K = 3, 2, 48, 256, 20
    rng = np.random.default_rng(6)
    heat = rng.random((B, classes, H, W)).astype(np.float32) * 0.5 + 0.2
    heat[:, :, ::2, ::2] = 0.9                       # every other cell in both directions: equal local maxima
    heat[1] = 0.05
    heat[1, 0, 10, 10], heat[1, 1, 40, 200], heat[1, 1, 0, 255] = 0.9, 0.8, 0.7
    size = synth.uniform(80, "osz", (B, 2, H, W))
    size[0, :, ::4, ::4] = -1.0                      # invalid boxes among the crowded candidates
    off = synth.uniform(80, "oof", (B, 2, H, W))
    bias = 0.0
    if logits:
        heat = (np.log(heat / (1 - heat)) - 0.3).astype(np.float32)
        bias = 0.3
    hd, sd, od = dev(heat, cuda), dev(size, cuda), dev(off, cuda)
    full = ops.centernet_to_host(*ops.centernet_decode(hd, sd, od, 0.2, K, logits=logits, heatmap_bias=bias))
    small = ops.centernet_to_host(*ops.centernet_decode(hd, sd, od, 0.2, K, logits=logits, heatmap_bias=bias,
                                                        candidate_capacity=1))
    if logits:
        scores = ops.centernet_activate(torch.cat([hd, sd, od], 1), classes, bias)[:, :classes].contiguous().cpu().numpy()
    else:
        scores = heat
    ref, ncand = oracle.centernet_decode(scores, size, off, 0.2, K)
    assert ncand[0] > 2000 and ncand[1] == 3 and ncand[2] > 2000
    for b in range(B):
        assert len(full[b]) == len(ref[b]) == min(K, ncand[b])
        dets_equal(full[b], ref[b])
        assert small[b].tobytes() == full[b].tobytes()


@pytest.mark.parametrize("logits", [False, True])
def test_centernet_raised_bound_with_too_few_valid_boxes_is_redone(cuda, oracle, logits):
    """The sampling pass raises an image's listing bound when the map holds far more hot cells than an image
    keeps.  If most of the boxes above the bound then turn out invalid, fewer than K detections remain above it and
    some of the K best may lie below: the image is redone without a bound.  Image 0: almost every box invalid;
    image 1: all valid (keeps its raised bound); image 2: nothing above the threshold."""
    B, classes, H, W, K = 3, 4, 64, 128, 50
    heat, size, off = centernet_case(52, B, classes, H, W)
    heat[2] = -9.0
    size[0] = -1.0
    rng = np.random.default_rng(9)
    for _ in range(70):                              # 70 valid boxes at random places of image 0
        size[0, :, int(rng.integers(H)), int(rng.integers(W))] = 0.5
    act = oracle.centernet_activate(np.concatenate([heat, size, off], 1), classes, 0.0)
    scores = np.ascontiguousarray(act[:, :classes])
    ref, ncand = oracle.centernet_decode(scores, size, off, 0.2, K)
    src = heat if logits else scores
    d, c = ops.centernet_decode(dev(src, cuda), dev(size, cuda), dev(off, cuda), 0.2, K, logits=logits, heatmap_bias=0.0)
    got = ops.centernet_to_host(d, c)
    assert 0 < ncand[0] < K and ncand[1] > 10 * K and ncand[2] == 0
    for b in range(B):
        assert len(got[b]) == len(ref[b]) == min(K, ncand[b])
        assert np.array_equal(got[b]["source"], ref[b]["source"])
        if not logits:
            dets_equal(got[b], ref[b])


def test_centernet_plateau_larger_than_the_default_list(cuda):
    """An all-equal map of more cells than an image's list holds by default: every cell is a maximum, the
    list overflows, the tile pass takes over and the K lowest indices win."""
    flat = np.full((2, 1, 200, 200), 0.5, np.float32)
    flat[1] = 0.1
    flat[1, 0, 7, 9] = 0.6
    ones = np.ones((2, 2, 200, 200), np.float32)
    d, c = ops.centernet_decode(dev(flat, cuda), dev(ones, cuda), dev(ones, cuda), 0.2, 100)
    got = ops.centernet_to_host(d, c)
    assert got[0]["source"].tolist() == list(range(100))
    assert got[1]["source"].tolist() == [7 * 200 + 9]
    with pytest.raises(ops.PxeError):
        ops.centernet_decode(dev(flat, cuda), dev(ones, cuda), dev(ones, cuda), 0.2, 100, candidate_capacity=1 << 20)


@pytest.mark.parametrize("shape,groups,temp", [((4, 1000, 1, 1), 1, 1.0), ((2, 30, 1, 1), 3, 0.7), ((3, 5, 2, 2), 1, 2.0),
                                               ((1, 3000, 1, 1), 1, 1.0), ((2, 200, 1, 1), 1, 1.0), ((2, 400, 1, 1), 1, 0.5),
                                               ((2, 1500, 1, 1), 1, 1.0), ((3, 128, 1, 1), 1, 1.0), ((2, 2049, 1, 1), 1, 1.0)])
def test_softmax(cuda, oracle, shape, groups, temp):
    x = synth.normal(60, f"sm{shape}", shape, 0, 3)
    ref = oracle.softmax(x, groups, temp)
    got = ops.softmax(dev(x, cuda), groups, temp).cpu().numpy()
    close(got, ref)
    # first-maximum argmax (SoftmaxLayer::addDetects) is unchanged
    assert np.array_equal(got.reshape(shape[0], -1).argmax(1), ref.reshape(shape[0], -1).argmax(1))


@pytest.mark.parametrize("use_softmax", [True, False])
def test_region_forward(cuda, oracle, use_softmax):
    B, num, coords, classes, H, W = 2, 5, 4, 20, 13, 13
    x = synth.normal(61, "region", (B, num * (coords + 1 + classes), H, W), 0, 2)
    ref = oracle.region_forward(x, num, coords, classes, use_softmax)
    got = ops.region_forward(dev(x, cuda), num, coords, classes, use_softmax).cpu().numpy()
    close(got, ref)


def test_nms_host_matches_oracle_on_random_boxes(cuda, oracle):
    rng = np.random.default_rng(7)
    n = 3000
    d = np.zeros(n, ops.DET_DTYPE)
    d["x"], d["y"] = rng.random(n) * 0.8, rng.random(n) * 0.8
    d["w"], d["h"] = rng.random(n) * 0.3 + 0.01, rng.random(n) * 0.3 + 0.01
    d["prob"] = np.round(rng.random(n), 2)          # many ties: exercises the stable sort
    d["class_id"], d["batch_id"] = rng.integers(0, 3, n), rng.integers(0, 2, n)
    d["source"] = np.arange(n)
    d["w"][:5] = -0.1                               # negative extents get normalised
    got = ops.nms(d, 0.4)
    ref = oracle.nms(d.astype(oracle.DET_DTYPE), 0.4)
    assert np.array_equal(got["source"], ref["source"])


def test_compat_symbols_run(cuda, oracle):
    """The px:: functions (reference signatures) exported for link-level drop-in."""
    L = capi.lib()
    x = synth.normal(62, "compat", (2, 4, 6, 6))
    d = dev(x, cuda)
    fn = getattr(L, "_ZN2px8activateE14ActivationTypePfm")
    fn.argtypes = [C.c_int, C.c_void_p, C.c_size_t]
    fn.restype = None
    fn(capi.ACT["leaky"], d.data_ptr(), d.numel())
    torch.cuda.synchronize()
    close(d.cpu().numpy(), oracle.activate("leaky", x))
    out = torch.zeros((2, 4, 3, 3), device=cuda)
    idx = torch.zeros((2, 4, 3, 3), device=cuda, dtype=torch.int32)
    mp = getattr(L, "_ZN2px17maxPoolForwardGpuEPKfPfPiiiiiiiiii")
    mp.argtypes = [C.c_void_p] * 3 + [C.c_int] * 9
    mp.restype = None
    src = dev(x, cuda)
    mp(src.data_ptr(), out.data_ptr(), idx.data_ptr(), 2, 4, 6, 6, 3, 3, 2, 2, 1)
    torch.cuda.synchronize()
    rv, ri = oracle.maxpool(x, 2, 2, 1)
    assert np.array_equal(out.cpu().numpy(), rv) and np.array_equal(idx.cpu().numpy(), ri)
    fill = getattr(L, "_ZN2px7fillGpuEPfmf")
    fill.argtypes = [C.c_void_p, C.c_size_t, C.c_float]
    fill.restype = None
    fill(out.data_ptr(), out.numel(), 3.5)
    torch.cuda.synchronize()
    assert (out == 3.5).all()


def _random_boxes(rng, n, images, classes, spread=0.8):
    d = np.zeros(n, ops.DET_DTYPE)
    d["x"], d["y"] = rng.random(n) * spread, rng.random(n) * spread
    d["w"], d["h"] = rng.random(n) * 0.3 + 0.01, rng.random(n) * 0.3 + 0.01
    d["prob"] = np.round(rng.random(n), 2)          # many ties: exercises the stable order
    d["class_id"], d["batch_id"] = rng.integers(0, classes, n), rng.integers(0, images, n)
    d["source"] = np.arange(n)
    return d


def _nms_device(d, thr, cuda):
    t = torch.from_numpy(d.view(np.int32).reshape(-1, 8).copy()).to(cuda)
    out, count = ops.nms_device(t, len(d), thr)
    m = int(count.item())
    return out[:m].cpu().numpy().view(ops.DET_DTYPE).reshape(-1)


@pytest.mark.parametrize("n,images,classes,thr", [(3000, 2, 3, 0.4), (1, 1, 1, 0.4), (500, 7, 80, 0.45), (6000, 1, 2, 0.3),
                                                  (4000, 3, 1, 0.6), (257, 2, 5, 0.0)])
def test_nms_device_equals_host_nms(cuda, oracle, n, images, classes, thr):
    """Same survivors, same order, same bits as pxe_nms_host (and the oracle's restatement of px::nms):
    probability ties, cross-class duplicates, groups longer than the 1024-member window."""
    d = _random_boxes(np.random.default_rng(n), n, images, classes)
    if n >= 500:
        dup = d[: n // 10].copy()                   # near-identical boxes of other classes: the IoU > 0.9 rule
        dup["class_id"] = (dup["class_id"] + 1) % max(classes, 2)
        dup["x"] += 1e-3
        d[-len(dup):] = dup
        d["w"][5], d["h"][6] = -0.2, 0.0            # negative / empty extents go through the same normalisation
    want = ops.nms(d, thr)
    got = _nms_device(d, thr, cuda)
    assert len(got) == len(want)
    assert got.tobytes() == want.tobytes()
    ref = oracle.nms(d, thr)
    assert len(ref) == len(got) and np.array_equal(ref["source"], got["source"])


def test_nms_device_on_decoded_detections(cuda):
    """End of the pipeline on the device: YOLO decode -> device NMS, against decode -> host copy -> host NMS."""
    model_in = synth.normal(90, "nmshead", (2, 255, 13, 13), 0, 1.5)
    buf = ops.DetectionBuffer(1 << 16, cuda)
    ops.yolo_decode(ops.yolo_activate(dev(model_in, cuda), 3, 80), [3, 4, 5], [10, 14, 23, 27, 37, 58, 81, 82, 135, 169, 344, 319],
                    80, 416, 416, 0.6, buf)
    recs, total = buf.to_host()
    assert 0 < total <= buf.capacity
    out, count = ops.nms_device(buf.dets, total, 0.4)
    got = out[: int(count.item())].cpu().numpy().view(ops.DET_DTYPE).reshape(-1)
    want = ops.nms(recs, 0.4)
    assert len(want) > 0 and got.tobytes() == want.tobytes()


def test_nms_device_argument_errors(cuda):
    t = torch.zeros((4, 8), device=cuda, dtype=torch.int32)
    out, count = ops.nms_device(t, 0, 0.4)
    assert int(count.item()) == 0
    with pytest.raises(ValueError):
        ops.nms_device(t, 5, 0.4)
    L = ops.capi.lib()
    assert L.pxe_nms(None, t.data_ptr(), 4, 0.4, t.data_ptr(), count.data_ptr(), t.data_ptr(), 16) == ops.capi.PXE_ERR_BAD_ARG
    ws = torch.empty(256, device=cuda, dtype=torch.uint8)
    o = torch.empty_like(t)
    assert L.pxe_nms(None, t.data_ptr(), 4, 0.4, o.data_ptr(), count.data_ptr(), ws.data_ptr(), 256) == ops.capi.PXE_ERR_WORKSPACE


@pytest.mark.parametrize("B,side,num,classes,squared,thr", [(3, 7, 2, 20, True, 0.2), (1, 3, 1, 4, False, 0.05), (5, 11, 3, 80, True, 0.5)])
def test_detect_decode_matches_oracle(cuda, oracle, B, side, num, classes, squared, thr):
    """YOLOv1 head: same boxes, classes, probabilities and order as DetectLayer::addDetects; scales that are
    zero, negative or not finite emit nothing; capacity overflow is counted, not stored."""
    rng = np.random.default_rng(B * 100 + side)
    per = side * side * (classes + num * 5)
    pred = rng.random((B, per)).astype(np.float32)
    scales = pred[:, side * side * classes: side * side * (classes + num)]
    scales[:, ::5] = 0.0
    scales[:, 1::7] = -0.3
    scales[0, 2] = np.nan
    scales[0, 3] = np.inf
    ref, total = oracle.detect_decode(pred, side, num, classes, thr, squared=squared)
    assert total > 0
    buf = ops.DetectionBuffer(B * side * side * num, cuda)
    ops.detect_decode(dev(pred, cuda), side, num, classes, thr, buf, squared=squared)
    got, n = buf.to_host()
    assert n == total
    # classes, order and probabilities are exact.  With `sqrt` the host squares widths with std::pow(v, 2) =
    # glibc's powf, which is within one ulp of v*v but not always equal to it (0.06 % of values differ in the
    # last bit); the device multiplies.  Boxes are therefore compared to 1e-6.
    dets_equal(got, ref, box_tol=1e-6 if squared else 0.0)
    small = ops.DetectionBuffer(max(1, total // 2), cuda)
    ops.detect_decode(dev(pred, cuda), side, num, classes, thr, small, squared=squared, batch_id_offset=4)
    got, n = small.to_host()
    assert n == total and len(got) == max(1, total // 2)
    assert np.array_equal(got["source"], ref["source"][:len(got)]) and np.array_equal(got["batch_id"], ref["batch_id"][:len(got)] + 4)


@pytest.mark.parametrize("B,num,classes,H,W,thr", [(2, 5, 20, 13, 13, 0.05), (1, 3, 4, 5, 7, 0.0), (3, 2, 80, 9, 9, 0.2)])
def test_region_decode_matches_oracle(cuda, oracle, B, num, classes, H, W, thr):
    """RegionLayer::addDetects after the layer's forward: same records and order.  per_image=False keeps the
    reference's indexing (every image decodes image 0's boxes); per_image=True equals decoding each image alone."""
    coords = 4
    x = synth.normal(62, f"reg{B}{num}{classes}", (B, num * (coords + 1 + classes), H, W), 0, 1.5)
    anchors = [1.08, 1.19, 3.42, 4.41, 6.63, 11.38, 9.42, 5.11, 16.62, 10.52][:2 * num]
    fwd = oracle.region_forward(x, num, coords, classes, True)
    ref = oracle.region_decode(fwd, W, H, num, coords, classes, np.array(anchors, np.float32), thr)
    assert len(ref) > 0
    dfwd = ops.region_forward(dev(x, cuda), num, coords, classes, True)
    buf = ops.DetectionBuffer(len(ref) + 16, cuda)
    ops.region_decode(dev(fwd, cuda), W, H, num, coords, classes, anchors, thr, buf)
    got, n = buf.to_host()
    assert n == len(ref)
    dets_equal(got, ref, box_tol=2e-6)                  # exp / logistic on the device vs glibc
    # from the device's own forward: same boxes up to the activation tolerance
    buf.reset()
    ops.region_decode(dfwd, W, H, num, coords, classes, anchors, thr, buf, per_image=True)
    got_all, n_all = buf.to_host()
    parts = [oracle.region_decode(fwd[b:b + 1], W, H, num, coords, classes, np.array(anchors, np.float32), thr) for b in range(B)]
    assert abs(n_all - sum(len(q) for q in parts)) <= max(2, n_all // 500)


def test_softmax_decode_first_maximum_threshold_and_nan(cuda):
    """SoftmaxLayer::addDetects: std::max_element keeps the earliest of equal maxima; a NaN elsewhere is ignored,
    a NaN in front blocks the image; images below the threshold emit nothing; order = image order."""
    B, classes = 70, 1000
    rng = np.random.default_rng(3)
    p = rng.random((B, classes)).astype(np.float32) * 0.5
    p[1, 17] = p[1, 400] = 0.9               # tie: the earlier index wins
    p[2] *= 0.1                              # below the threshold
    p[3, 5] = np.nan; p[3, 900] = 0.8        # NaN in the middle is skipped
    p[4, 0] = np.nan; p[4, 10] = 0.99        # NaN in front: max_element never leaves it
    p[5, 999] = 0.95
    p[69, 31] = 0.7
    want = []
    for b in range(B):
        row = p[b]
        arg = 0
        for j in range(1, classes):
            if row[arg] < row[j]:
                arg = j
        if row[arg] >= 0.3:
            want.append((b, arg, row[arg]))
    buf = ops.DetectionBuffer(B, cuda)
    ops.softmax_decode(dev(p, cuda), 224, 224, 0.3, buf, batch_id_offset=2)
    got, n = buf.to_host()
    assert n == len(want) and len(got) == n
    assert got["batch_id"].tolist() == [b + 2 for b, _, _ in want]
    assert got["class_id"].tolist() == [a for _, a, _ in want]
    assert np.array_equal(got["prob"], np.array([v for _, _, v in want], np.float32))
    assert (got["x"] == 0).all() and (got["w"] == 224).all() and (got["h"] == 224).all()
    assert 2 not in [b for b, _, _ in want] and 4 not in [b for b, _, _ in want]
    assert (1, 17, np.float32(0.9)) in want and (3, 900, np.float32(0.8)) in want
