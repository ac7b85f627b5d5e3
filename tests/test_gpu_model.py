"""GPU parity on whole graphs: the planned (fused) schedule against the layer-by-layer schedule,
and the YOLOv3-tiny 416 forward against the CPU oracle (the reference's CPU path)."""
import numpy as np
import pytest
import torch

from pixienn_b200 import graph, ops, presets, synth
from pixienn_b200.runner import Runner, synth_weights
from test_gpu_epilogue import close, dev

pytestmark = pytest.mark.gpu


def make_input(seed, batch, model):
    return np.stack([synth.uniform(seed, f"input/{b}", (model.channels, model.height, model.width)) for b in range(batch)])


def run(model, weights, x, cuda, **kw):
    r = Runner(model, weights, x.shape[0], cuda, **kw)
    r.forward(dev(x, cuda))
    torch.cuda.synchronize()
    return r


@pytest.fixture(autouse=True)
def exact_fp32_convolutions():
    """cuDNN may use TF32 tensor cores for fp32 convolutions (the reference leaves cuDNN's default
    math mode on, which allows it).  Parity with a CPU forward needs true fp32 products."""
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cudnn.allow_tf32 = old


@pytest.mark.parametrize("name,hw,batch,head_bias", [("yolov3-tiny", 160, 3, -3.0), ("yolov3", 128, 2, -3.0),
                                                     ("yolov7", 128, 2, 0.0), ("yolov7", 160, 1, 0.0),
                                                     ("centernet-tiny", 128, 2, 0.0)])
def test_fused_plan_equals_layer_by_layer(cuda, name, hw, batch, head_bias):
    """Fusion and route elimination move stores around; they never change a value.  Detections of
    the fused schedule are bit-identical to the one-launch-per-layer schedule."""
    model = graph.parse_model(presets.PRESETS[name](hw, hw))
    weights = synth_weights(model, 7, head_bias=head_bias)
    x = make_input(8, batch, model)
    fused = run(model, weights, x, cuda, fuse=True, raw_heads=True)
    plain = run(model, weights, x, cuda, fuse=False, raw_heads=False)
    a, na = fused.detections()
    b, nb = plain.detections()
    assert na == nb and na > 0
    assert a.tobytes() == b.tobytes()
    assert fused.launches < plain.launches
    assert fused.contiguous_copies == 0


def test_spp_block_takes_the_conv_epilogue(cuda):
    """YOLOv7's SPP block: the conv before it hands its raw output to the block, which applies the epilogue while
    it stages each plane (one launch, "epilogue+spp"); every layer's tensor equals the run that keeps them apart."""
    model = graph.parse_model(presets.PRESETS["yolov7"](128, 128))
    weights = synth_weights(model, 7)
    x = make_input(8, 2, model)
    runs = []
    for fold in (True, False):
        r = Runner(model, weights, 2, cuda)
        r.fold_spp = fold
        r.keep = set(range(len(model.layers)))
        r.timer.enabled = True
        r.forward(torch.from_numpy(x).to(cuda))
        torch.cuda.synchronize()
        runs.append(r)
    a, b = runs
    assert "epilogue+spp" in a.timer.summary() and "epilogue+spp" not in b.timer.summary()
    assert "spp" in b.timer.summary() and a.launches == b.launches - 1
    assert set(a.kept) == set(b.kept)
    for i in sorted(a.kept):
        assert torch.equal(a.kept[i], b.kept[i]), f"layer {i} ({model.layers[i].type})"
    assert a.detections()[0].tobytes() == b.detections()[0].tobytes()


def test_tiny416_matches_cpu_reference_path(cuda, oracle):
    """Config 0: YOLOv3-tiny, batch 1, 416x416, seeded weights, against the CPU forward.
    (i)  every conv epilogue, fed the CPU path's own conv output, within 1e-5 rel / 1e-6 abs;
    (ii) the heads of the full GPU forward close to the CPU heads (the convolutions differ in
         summation order, so this is a looser, end-to-end sanity bound);
    (iii) decode + NMS of the CPU path's activated heads: identical detections after NMS."""
    from oracle.pxmodel import CpuModel
    doc = presets.yolov3_tiny()
    model = graph.parse_model(doc)
    weights = synth_weights(model, 1234, head_bias=-4.0)
    x = make_input(1234, 1, model)
    cpu = CpuModel(doc, weights, eps_mode=1)
    cpu.forward(x)

    # (i)
    for l in model.layers:
        if l.type != "conv":
            continue
        w = weights[l.index]
        raw = dev(cpu.raw_conv[l.index], cuda)
        if l.batch_norm:
            got = ops.conv_epilogue(raw, gamma=dev(w["scales"], cuda), beta=dev(w["biases"], cuda),
                                    mean=dev(w["rolling_mean"], cuda), var=dev(w["rolling_var"], cuda),
                                    act=l.activation, eps_mode=1)
        else:
            got = ops.conv_epilogue(raw, bias=dev(w["biases"], cuda), act=l.activation)
        close(got.cpu().numpy(), cpu.outputs[l.index])

    # (ii)
    gpu = Runner(model, weights, 1, cuda, raw_heads=False, eps_mode=1)
    gpu.keep = {16, 23}
    gpu.forward(dev(x, cuda))
    torch.cuda.synchronize()
    for h in (16, 23):
        g, c = gpu.kept[h].cpu().numpy(), cpu.outputs[h]
        assert np.abs(g - c).max() < 2e-3, f"head {h}: {np.abs(g - c).max()}"

    # (iii)
    ref = cpu.detections(0.2)
    buf = ops.DetectionBuffer(len(ref) + 16, cuda)
    for h in (16, 23):
        ld = doc["model"]["layers"][h]
        ops.yolo_decode(dev(cpu.outputs[h], cuda), ld["mask"], ld["anchors"], 80, 416, 416, 0.2, buf)
    got, total = buf.to_host()
    assert total == len(ref) and total > 10
    assert np.array_equal(got["source"], ref["source"]) and np.array_equal(got["class_id"], ref["class_id"])
    assert np.array_equal(got["prob"], ref["prob"])
    kept_gpu = ops.nms(got, 0.4)
    kept_ref = oracle.nms(ref, 0.4)
    # boxes differ by an ulp of exp(); report how close any IoU came to the thresholds
    assert len(kept_gpu) == len(kept_ref)
    assert np.array_equal(kept_gpu["source"], kept_ref["source"]) and np.array_equal(kept_gpu["class_id"], kept_ref["class_id"])


def test_batch_sharding_gives_identical_detections(cuda):
    """Every op is per-image: running images [0,2) and [2,4) as two shards (batch_id_offset marks the
    global image number) and merging per head reproduces the 4-image run record for record."""
    from pixienn_b200 import sharding
    model = graph.parse_model(presets.yolov3_tiny(160, 160))
    weights = synth_weights(model, 5, head_bias=-3.0)
    x = make_input(6, 4, model)
    whole, n = run(model, weights, x, cuda).detections()
    shards = []
    for s in range(2):
        first, last = sharding.shard_range(4, s, 2)
        r = Runner(model, weights, last - first, cuda, batch_id_offset=first)
        r.forward(dev(x[first:last], cuda))
        shards.append(r.detections_by_head())
    merged = sharding.merge_shards(shards)
    assert n == len(whole) == len(merged) and n > 0
    assert merged.tobytes() == whole.tobytes()


@pytest.mark.parametrize("use_graphs", [False, True])
def test_pipelined_predictor_equals_sequential_predict(cuda, use_graphs):
    """Overlapping the copies of neighbouring batches with compute changes no record; neither does
    replaying the forward pass as a CUDA graph (one graph per buffer slot)."""
    from pixienn_b200.runner import PipelinedPredictor
    model = graph.parse_model(presets.yolov3_tiny(160, 160))
    weights = synth_weights(model, 9, head_bias=-3.0)
    batches = [torch.from_numpy(make_input(20 + i, 2, model)).pin_memory() for i in range(4)]
    seq = Runner(model, weights, 2, cuda)
    want = [seq.predict(b)[0].copy() for b in batches]
    pipe = PipelinedPredictor(Runner(model, weights, 2, cuda), tuple(batches[0].shape), use_graphs=use_graphs)
    got = []
    for b in batches:
        r = pipe.submit(b)
        if r is not None:
            got.append(r[0].copy())
    got.append(pipe.drain()[0].copy())
    assert len(got) == len(want) == 4
    for g, w in zip(got, want):
        assert len(w) > 0 and g.tobytes() == w.tobytes()


def test_pipelined_predictor_with_device_nms_returns_the_survivors(cuda):
    """nms_threshold: px::nms runs on the device beside the next batch's forward pass and only the survivors are
    copied to the host: the same records as predict() with host NMS, batch by batch."""
    from pixienn_b200.runner import PipelinedPredictor
    model = graph.parse_model(presets.yolov3_tiny(160, 160))
    weights = synth_weights(model, 9, head_bias=-3.0)
    batches = [torch.from_numpy(make_input(60 + i, 2, model)).pin_memory() for i in range(4)]
    seq = Runner(model, weights, 2, cuda)
    want = [seq.predict(b, nms_threshold=0.4) for b in batches]
    pipe = PipelinedPredictor(Runner(model, weights, 2, cuda), tuple(batches[0].shape), use_graphs=True, nms_threshold=0.4)
    got = []
    for b in batches:
        r = pipe.submit(b)
        if r is not None:
            got.append((r[0].copy(), r[1]))
    last = pipe.drain()
    got.append((last[0].copy(), last[1]))
    assert len(got) == 4
    for (g, gt), (w, wt) in zip(got, want):
        assert gt == wt and 0 < len(w) < wt and g.tobytes() == w.tobytes()


@pytest.mark.parametrize("name", ["yolov3_tiny", "centernet_tiny"])
def test_cuda_graph_replay_equals_eager_forward(cuda, name):
    """Runner.capture: replays read the captured input tensor's current contents and rewrite the same
    detection buffers; records and per-head marks equal an eager pass on the same input."""
    builder = getattr(presets, name)
    model = graph.parse_model(builder(128, 128))
    weights = synth_weights(model, 11, head_bias=-3.0 if name == "yolov3_tiny" else 0.0)
    eager = Runner(model, weights, 2, cuda)
    captured = Runner(model, weights, 2, cuda)
    x = dev(make_input(30, 2, model), cuda)
    captured.forward(x)
    g = captured.capture(x)
    for seed in (31, 32):
        xin = dev(make_input(seed, 2, model), cuda)
        x.copy_(xin)
        g.replay()
        eager.forward(xin)
        want, wt = eager.detections()
        got, gt = captured.detections()
        assert wt == gt and len(want) > 0 and got.tobytes() == want.tobytes()
        assert [h.tobytes() for h in captured.detections_by_head()] == [h.tobytes() for h in eager.detections_by_head()]


def test_yolov1_style_graph_runs_connected_and_detection_layers(cuda, oracle):
    """conv + pool -> avgpool-free YOLOv1 tail: connected layer (cuBLAS GEMM + the epilogue kernel on
    [B, outputs, 1, 1]) and the detection head decoded on the device.  The decode is checked exactly against
    the oracle on the head values the device produced; the connected layer against a float64 product."""
    side, num, classes = 3, 2, 4
    doc = {"model": {"channels": 3, "height": 24, "width": 24, "layers": [
        {"type": "conv", "filters": 8, "kernel": 3, "stride": 1, "pad": True, "batch_normalize": True, "activation": "leaky"},
        {"type": "maxpool", "kernel": 2, "stride": 2},
        {"type": "conv", "filters": 16, "kernel": 3, "stride": 2, "pad": True, "batch_normalize": True, "activation": "leaky"},
        {"type": "connected", "output": side * side * (classes + num * 5), "activation": "linear"},
        {"type": "detection", "side": side, "num": num, "coords": 4, "sqrt": True, "softmax": False},
    ]}}
    model = graph.parse_model(doc)
    assert model.classes == classes
    weights = synth_weights(model, 13)
    weights[3]["biases"] = weights[3]["biases"] + 0.3
    r = Runner(model, weights, 2, cuda, threshold=0.05)
    r.keep = {2, 3}
    x = dev(make_input(40, 2, model), cuda)
    r.forward(x)
    head = r.kept[3].cpu().numpy().reshape(2, -1)
    feat = r.kept[2].cpu().numpy().reshape(2, -1).astype(np.float64)
    want_head = feat @ weights[3]["weights"].astype(np.float64).T + weights[3]["biases"]
    np.testing.assert_allclose(head, want_head, rtol=2e-3, atol=2e-3)      # cuBLAS may use TF32 products
    ref, total = oracle.detect_decode(head, side, num, classes, 0.05, squared=True)
    got, n = r.detections()
    assert n == total > 0 and len(got) == len(ref)
    for f in ("class_id", "batch_id", "source", "prob"):
        assert np.array_equal(got[f], ref[f]), f
    for f in ("x", "y", "w", "h"):                   # squared widths: the host's powf(v, 2) vs v*v, one ulp apart at most
        np.testing.assert_allclose(got[f], ref[f], rtol=1e-6, atol=1e-6)


def test_predict_with_device_nms_equals_host_nms(cuda):
    """Runner.predict: NMS on the device buffer + a copy of the survivors == a copy of everything + host NMS."""
    model = graph.parse_model(presets.yolov3_tiny(160, 160))
    weights = synth_weights(model, 9, head_bias=-3.0)
    r = Runner(model, weights, 3, cuda)
    xb = torch.from_numpy(make_input(50, 3, model)).pin_memory()
    want, total = r.predict(xb, nms_threshold=0.4)
    got, total2 = r.predict(xb, nms_threshold=0.4, nms_on_device=True)
    assert total == total2 and 0 < len(want) < total
    assert got.tobytes() == want.tobytes()


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_route_of_a_head_type_layer_and_shortcut_across_shapes(cuda, oracle, layout):
    """Two graph shapes outside the presets: a route that concatenates a dropout layer's output (a head-type step,
    whose dense output has to be copied into the route's buffer) and a shortcut whose `from` tensor has another
    shape, which the reference reads with this layer's own dimensions (resnet18.yml does that across its stride-2
    stages).  Every layer equals the CPU walk, which follows the same rule."""
    from oracle.pxmodel import CpuModel
    conv = lambda f, k, s, act="leaky": {"type": "conv", "filters": f, "kernel": k, "stride": s, "pad": True,
                                         "batch_normalize": True, "activation": act}
    doc = {"model": {"channels": 3, "height": 16, "width": 16, "layers": [
        conv(8, 3, 1),                                   # 0: 8 x 16 x 16
        conv(16, 3, 2),                                  # 1: 16 x 8 x 8
        conv(16, 1, 1, "linear"),                        # 2
        {"type": "shortcut", "from": 0, "activation": "leaky"},      # 3: from is 8 x 16 x 16 = the same element count, another shape
        {"type": "dropout"},                             # 4
        {"type": "route", "layers": [4, 1]},             # 5: 32 x 8 x 8
        {"type": "conv", "filters": 18, "kernel": 1, "stride": 1, "pad": True, "activation": "linear"},
        {"type": "yolo", "mask": [0, 1, 2], "anchors": [10, 14, 23, 27, 37, 58]},
    ]}}
    model = graph.parse_model(doc)
    weights = synth_weights(model, 21, head_bias=-1.0)
    x = make_input(22, 2, model)
    cpu = CpuModel(doc, weights, eps_mode=0)
    cpu.forward(x)
    r = Runner(model, weights, 2, cuda, layout=layout, raw_heads=False)
    r.keep = set(range(len(model.layers)))
    r.forward(dev(x, cuda))
    torch.cuda.synchronize()
    for i in (0, 1, 3, 4, 5):
        np.testing.assert_allclose(r.kept[i].contiguous().cpu().numpy(), cpu.outputs[i], rtol=2e-3, atol=2e-3, err_msg=f"layer {i}")
    # the route's buffer holds the dropout output and layer 1, in that order
    assert torch.equal(r.kept[5][:, :16].contiguous(), r.kept[4].contiguous()) and torch.equal(r.kept[5][:, 16:].contiguous(), r.kept[1].contiguous())
