"""GPU parity of the channels-last tier: the NHWC kernels produce, element for element, what the NCHW
kernels produce on the same values; a whole graph run channels-last agrees with the NCHW run up to the
convolutions' own rounding (cuDNN uses different kernels for the two layouts)."""
import numpy as np
import pytest
import torch

from pixienn_b200 import graph, ops, presets, synth
from pixienn_b200.runner import Runner, synth_weights
from test_gpu_epilogue import bn, dev

pytestmark = pytest.mark.gpu


def nhwc(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous(memory_format=torch.channels_last)


def same(a: torch.Tensor, b: torch.Tensor):
    assert a.shape == b.shape
    assert torch.equal(a.contiguous(), b.contiguous())


@pytest.mark.parametrize("shape", [(2, 8, 16, 16), (3, 5, 13, 13), (1, 255, 19, 19), (2, 64, 1, 1), (1, 12, 7, 33)])
@pytest.mark.parametrize("act", ["leaky", "mish", "swish", "logistic", "linear", "relu"])
@pytest.mark.parametrize("use_bn", [True, False])
def test_epilogue_nhwc_equals_nchw(cuda, shape, act, use_bn):
    B, C, H, W = shape
    x = dev(synth.normal(71, f"x{shape}", shape), cuda)
    (g, b, m, v), dp = bn(72, f"bn{shape}", C, cuda)
    bias = dev(synth.normal(73, f"b{shape}", C, 0, 0.1), cuda)
    kw = dict(gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], bias=bias) if use_bn else dict(bias=bias)
    want = ops.conv_epilogue(x.clone(), act=act, **kw)
    fa, fb = ops.fold_bn(C, cuda, **kw)
    got = ops.conv_epilogue_nhwc(nhwc(x.clone()), a=fa, b=fb, act=act)
    same(got, want)


def test_epilogue_nhwc_residual_and_slot_stores(cuda):
    B, C, H, W = 2, 16, 10, 12
    x = dev(synth.normal(74, "xr", (B, C, H, W)), cuda)
    frm = dev(synth.normal(75, "fr", (B, C, H, W)), cuda)
    (g, b, m, v), dp = bn(76, "bnr", C, cuda)
    want = ops.conv_epilogue(x.clone(), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act="leaky", residual=frm,
                             res_alpha=1.0, res_beta=1.0, res_act="linear")
    fa, fb = ops.fold_bn(C, cuda, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3])
    wide = ops.empty_nhwc((B, C + 8, H, W), cuda)
    wide.fill_(5.0)
    wide_res = ops.empty_nhwc((B, C + 4, H, W), cuda)
    wide_res[:, 4:] = frm
    dense = ops.empty_nhwc((B, C, H, W), cuda)
    ops.conv_epilogue_nhwc(nhwc(x), y=dense, y2=wide[:, 8:], a=fa, b=fb, act="leaky", residual=wide_res[:, 4:])
    same(dense, want)
    same(wide[:, 8:], want)
    assert (wide[:, :8] == 5.0).all()
    # the stand-alone shortcut and the plain copy are the same kernel without coefficients
    sc = ops.conv_epilogue_nhwc(nhwc(x), y=ops.empty_nhwc((B, C, H, W), cuda), residual=nhwc(frm), res_alpha=1.0, res_beta=1.0,
                                res_act="leaky")
    same(sc, ops.shortcut(x, frm, 1.0, 1.0, "leaky"))
    cp = ops.conv_epilogue_nhwc(nhwc(x), y=ops.empty_nhwc((B, C, H, W), cuda))
    same(cp, x)
    # odd channel counts take the scalar form
    x3 = dev(synth.normal(77, "x3", (2, 3, 5, 7)), cuda)
    b3 = dev(synth.normal(78, "b3", 3, 0, 0.1), cuda)
    a_, b_ = ops.fold_bn(3, cuda, bias=b3)
    same(ops.conv_epilogue_nhwc(nhwc(x3.clone()), a=a_, b=b_, act="mish"), ops.conv_epilogue(x3.clone(), bias=b3, act="mish"))


@pytest.mark.parametrize("shape", [(2, 8, 16, 16), (2, 16, 13, 13), (1, 5, 26, 26), (1, 12, 7, 12), (2, 32, 52, 52)])
@pytest.mark.parametrize("act", ["leaky", "mish"])
@pytest.mark.parametrize("keep_full", [False, True])
def test_epilogue_nhwc_with_folded_pool(cuda, shape, act, keep_full):
    """Pooled (and full-resolution) outputs equal the NCHW fused kernel's, element for element."""
    B, C, H, W = shape
    x = dev(synth.normal(83, f"xp{shape}", shape), cuda)
    (g, b, m, v), dp = bn(84, f"bnp{shape}", C, cuda)
    kw = dict(gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3])
    wy, wp = ops.conv_epilogue(x.clone(), y=None if keep_full else False, act=act, pool=(2, 2, 1), **kw)
    fa, fb = ops.fold_bn(C, cuda, **kw)
    xin = nhwc(x.clone())
    gy, gp = ops.conv_epilogue_nhwc(xin, y=None if keep_full else False, a=fa, b=fb, act=act, pool=(2, 2, 1))
    same(gp, wp)
    if keep_full:
        same(gy, wy)
    else:
        assert gy is None and torch.equal(xin, nhwc(x))
    wide = ops.empty_nhwc((B, C + 4, wp.shape[2], wp.shape[3]), cuda)
    wide.fill_(1.5)
    ops.conv_epilogue_nhwc(nhwc(x.clone()), y=False, a=fa, b=fb, act=act, pool=(2, 2, 1), y_pool=wide[:, 4:])
    same(wide[:, 4:], wp)
    assert (wide[:, :4] == 1.5).all()


@pytest.mark.parametrize("shape,stride", [((2, 8, 13, 13), 2), ((1, 6, 5, 9), 3), ((2, 256, 19, 19), 2)])
def test_upsample_nhwc(cuda, shape, stride):
    x = dev(synth.normal(79, f"up{shape}", shape), cuda)
    want = ops.upsample(x, stride, 1.0)
    same(ops.upsample_nhwc(nhwc(x), stride, 1.0), want)
    B, C, H, W = shape
    wide = ops.empty_nhwc((B, C + 4, H * stride, W * stride), cuda)
    wide.fill_(2.0)
    ops.upsample_nhwc(nhwc(x), stride, 0.5, out=wide[:, :C])
    same(wide[:, :C], ops.upsample(x, stride, 0.5))
    assert (wide[:, C:] == 2.0).all()


@pytest.mark.parametrize("shape,k,s,pad", [((2, 8, 16, 16), 2, 2, 1), ((1, 16, 13, 13), 2, 1, 1), ((2, 4, 20, 20), 5, 1, 4),
                                           ((1, 3, 13, 13), 13, 1, 12), ((2, 5, 7, 12), 3, 2, 0), ((1, 8, 26, 26), 2, 2, 0)])
def test_maxpool_nhwc(cuda, shape, k, s, pad):
    x = dev(synth.normal(80, f"mp{shape}", shape), cuda)
    same(ops.maxpool_nhwc(nhwc(x), k, s, pad), ops.maxpool(x, k, s, pad))


def test_nhwc_to_nchw(cuda):
    for shape in [(2, 255, 19, 19), (1, 3, 5, 5), (3, 24, 32, 40), (2, 70, 1, 1)]:
        x = dev(synth.normal(81, f"tr{shape}", shape), cuda)
        out = ops.nhwc_to_nchw(nhwc(x))
        assert out.is_contiguous() and torch.equal(out, x)
    wide = nhwc(dev(synth.normal(82, "trw", (2, 40, 6, 6)), cuda))
    assert torch.equal(ops.nhwc_to_nchw(wide[:, 8:32]), wide[:, 8:32].contiguous())


@pytest.fixture()
def exact_fp32_convolutions():
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cudnn.allow_tf32 = old


@pytest.mark.parametrize("name,hw,batch,head_bias", [("yolov3-tiny", 160, 2, -3.0), ("yolov3", 128, 2, -3.0),
                                                     ("yolov7", 128, 1, 0.0), ("centernet-tiny", 128, 2, 0.0)])
def test_channels_last_run_agrees_with_nchw_run(cuda, exact_fp32_convolutions, name, hw, batch, head_bias):
    model = graph.parse_model(presets.PRESETS[name](hw, hw))
    weights = synth_weights(model, 7, head_bias=head_bias)
    x = dev(np.stack([synth.uniform(8, f"input/{b}", (model.channels, hw, hw)) for b in range(batch)]), cuda)
    runs = {}
    for layout in ("nchw", "nhwc"):
        r = Runner(model, weights, batch, cuda, layout=layout)
        r.keep = set(range(len(model.layers)))
        r.forward(x)
        torch.cuda.synchronize()
        assert r.contiguous_copies == 0
        runs[layout] = r
    a, b = runs["nchw"], runs["nhwc"]
    assert set(a.kept) == set(b.kept)
    for i in sorted(a.kept):
        ta, tb = a.kept[i], b.kept[i]
        assert ta.shape == tb.shape, i
        scale = float(ta.abs().max()) + 1e-6
        assert float((ta - tb).abs().max()) <= 2e-4 * scale, f"layer {i} ({model.layers[i].type})"
    da, na = a.detections()
    db, nb = b.detections()
    # scores near the threshold flip with the convolutions' rounding: the counts agree closely, and where the
    # heads are biased away from the threshold (few, confident detections) so do the sets
    assert na > 0 and abs(na - nb) <= max(2, na // 50)
    if head_bias != 0.0:
        key = lambda d: set(zip(d["batch_id"].tolist(), d["class_id"].tolist(), d["source"].tolist()))
        assert len(key(da) & key(db)) >= 0.9 * max(len(da), len(db))


@pytest.mark.parametrize("shape,cout", [((2, 3, 40, 150), 32), ((1, 3, 9, 7), 16), ((2, 1, 33, 129), 8), ((1, 4, 16, 260), 64)])
@pytest.mark.parametrize("act", ["leaky", "mish", "linear"])
@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_fused_stem_convolution(cuda, exact_fp32_convolutions, shape, cout, act, layout):
    """First-layer convolution + epilogue in one launch == cuDNN convolution (true fp32) + the epilogue kernel,
    to fp32 rounding of a 27-term sum; both output layouts, ragged tile edges, stores into a wider buffer."""
    import torch.nn.functional as F
    B, Cin, H, W = shape
    x = dev(synth.uniform(85, f"stem{shape}", shape), cuda)
    w = dev(synth.normal(86, f"stemw{shape}{cout}", (cout, Cin, 3, 3), 0.0, 0.3), cuda)
    (g, b, m, v), dp = bn(87, f"stembn{cout}", cout, cuda)
    fa, fb = ops.fold_bn(cout, cuda, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3])
    want = ops.conv_epilogue(F.conv2d(x, w, None, 1, 1), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act)
    got = ops.conv_stem(x, w, a=fa, b=fb, act=act, nhwc=layout == "nhwc")
    assert got.is_contiguous(memory_format=torch.channels_last if layout == "nhwc" and cout > 1 and H * W > 1 else torch.contiguous_format)
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) <= 2e-6 * scale + 1e-6
    wide = ops.empty_nhwc((B, cout + 8, H, W), cuda) if layout == "nhwc" else torch.empty((B, cout + 8, H, W), device=cuda)
    wide.fill_(3.0)
    ops.conv_stem(x, w, a=fa, b=fb, act=act, out=wide[:, 8:], nhwc=layout == "nhwc")
    assert torch.equal(wide[:, 8:].contiguous(), got.contiguous()) and bool((wide[:, :8] == 3.0).all())
    bare = ops.conv_stem(x, w, act="linear", nhwc=layout == "nhwc")
    ref = F.conv2d(x, w, None, 1, 1)
    assert float((bare - ref).abs().max()) <= 2e-6 * float(ref.abs().max()) + 1e-6


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_runner_with_fused_stem_agrees_with_the_cudnn_stem(cuda, exact_fp32_convolutions, layout):
    model = graph.parse_model(presets.PRESETS["yolov3"](128, 128))
    weights = synth_weights(model, 7, head_bias=-3.0)
    x = dev(np.stack([synth.uniform(8, f"input/{b}", (3, 128, 128)) for b in range(2)]), cuda)
    runs = []
    for fused in (False, True):
        r = Runner(model, weights, 2, cuda, layout=layout, fused_stem=fused)
        assert (r.stem is not None) == fused
        r.keep = set(range(len(model.layers)))
        r.forward(x)
        torch.cuda.synchronize()
        runs.append(r)
    a, b = runs
    assert b.launches == a.launches                       # one library launch either way: the cuDNN call is what goes
    for i in sorted(a.kept):
        ta, tb = a.kept[i], b.kept[i]
        assert float((ta - tb).abs().max()) <= 2e-4 * (float(ta.abs().max()) + 1e-6), f"layer {i}"
    na, nb = a.detections()[1], b.detections()[1]
    assert na > 0 and abs(na - nb) <= max(2, na // 50)


@pytest.mark.parametrize("name,hw,batch", [("yolov3", 128, 2), ("yolov7", 128, 1)])
def test_runner_with_cudnn_conv_fusion_agrees_with_the_split_form(cuda, name, hw, batch):
    """conv + epilogue (+ shortcut) as one cuDNN runtime-fusion launch per layer == cuDNN convolution + the
    library's epilogue, to the convolutions' own rounding (both use TF32 tensor cores with different summation
    orders, and the difference grows through a hundred layers: 2e-3 of a tensor's range by the last ones); first
    pass (plans are timed) and second pass (cached plans) alike."""
    pytest.importorskip("cudnn")
    model = graph.parse_model(presets.PRESETS[name](hw, hw))
    weights = synth_weights(model, 7, head_bias=-3.0)
    x = dev(np.stack([synth.uniform(8, f"input/{b}", (model.channels, hw, hw)) for b in range(batch)]), cuda)
    ref = Runner(model, weights, batch, cuda, layout="nhwc")
    ref.keep = set(range(len(model.layers)))
    ref.forward(x)
    r = Runner(model, weights, batch, cuda, layout="nhwc", conv_fusion=True)
    r.fused_conv.prefer_fused = True          # small shapes: take a fused plan wherever cuDNN has one
    r.keep = set(range(len(model.layers)))
    with pytest.raises(ValueError):
        Runner(model, weights, batch, cuda, layout="nchw", conv_fusion=True)
    for attempt in range(2):
        r.forward(x)
        torch.cuda.synchronize()
        assert set(r.kept) == set(ref.kept)
        for i in sorted(ref.kept):
            ta, tb = ref.kept[i], r.kept[i]
            assert ta.shape == tb.shape, i
            assert float((ta - tb).abs().max()) <= 1e-2 * (float(ta.abs().max()) + 1e-6), f"pass {attempt} layer {i}"
    assert r.fused_conv_launches > 0, r.fused_conv.log
    s = r.fused_conv.summary()
    assert s["fused"] > 0 and s["shapes"] >= s["fused"]
    # replayed as a CUDA graph the fused launches are part of the graph
    g = r.capture(x)
    g.replay()
    torch.cuda.synchronize()
    for i in sorted(ref.kept):
        assert float((ref.kept[i] - r.kept[i]).abs().max()) <= 1e-2 * (float(ref.kept[i].abs().max()) + 1e-6)
