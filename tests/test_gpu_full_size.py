"""Parity at BASELINE.json's full sizes, where the CPU oracle would take minutes: properties that do not depend
on size (round trips, identities, idempotence, order) and plain PyTorch fp32 forms of the same operations, which
share no code with the kernels under test."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from pixienn_b200 import ops, synth

pytestmark = pytest.mark.gpu

SWEEP = [(64, 32, 208, 208), (64, 64, 104, 104), (64, 128, 52, 52), (64, 256, 26, 26), (64, 512, 13, 13)]


def randn(shape, cuda, seed=0):
    return torch.randn(shape, device=cuda, generator=torch.Generator(cuda).manual_seed(seed))


def params(C, cuda):
    g, b, m, v = (torch.from_numpy(t).to(cuda) for t in synth.bn_params(3, f"full{C}", C))
    bias = torch.from_numpy(synth.normal(3, f"fullb{C}", C, 0, 0.1)).to(cuda)
    return g, b, m, v, bias


def torch_epilogue(x, g, b, m, v, bias, act):
    y = (x - m[None, :, None, None]) / torch.sqrt(v + 1e-5)[None, :, None, None] * g[None, :, None, None] \
        + (b + bias)[None, :, None, None]
    if act == "leaky":
        return torch.where(y > 0, y, 0.1 * y)
    if act == "mish":
        return y * torch.tanh(F.softplus(y, threshold=20.0))
    if act == "swish":
        return y * torch.sigmoid(y)
    return torch.sigmoid(y)


def assert_close(got, ref, rtol=1e-5, atol=1e-6):
    bad = (got - ref).abs() > atol + rtol * ref.abs()
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} outside tolerance, worst {float((got - ref).abs().max())}"


@pytest.mark.parametrize("shape", SWEEP)
@pytest.mark.parametrize("act", ["leaky", "mish", "swish", "logistic"])
def test_sweep_cells_against_torch_and_their_own_identities(cuda, shape, act):
    """One sweep cell at full size: the fused kernel against the PyTorch form; the pooled output is exactly the
    max pool of the full-resolution output; in place == out of place == stored into a concat slot == NHWC."""
    B, C, H, W = shape
    x = randn(shape, cuda)
    g, b, m, v, bias = params(C, cuda)
    kw = dict(gamma=g, beta=b, mean=m, var=v, bias=bias, act=act)
    y = ops.conv_epilogue(x, in_place=False, **kw)
    # folding BN into one multiply-add reorders the arithmetic: 2e-5 of the value plus 2e-6 covers it at any size
    assert_close(y, torch_epilogue(x, g, b, m, v, bias, act), rtol=2e-5, atol=2e-6)
    full, pooled = ops.conv_epilogue(x.clone(), pool=(2, 2, 1), **kw)
    assert torch.equal(full, y)
    assert torch.equal(pooled, ops.maxpool(y, 2, 2, 1))
    assert torch.equal(pooled, F.max_pool2d(F.pad(y, (0, W % 2, 0, H % 2), value=float("-inf")), 2, 2))
    _, pooled_only = ops.conv_epilogue(x.clone(), y=False, pool=(2, 2, 1), **kw)
    assert torch.equal(pooled_only, pooled)
    wide = torch.empty((B, C + 4, H, W), device=cuda)
    ops.conv_epilogue(x, y=wide[:, 4:], **kw)
    assert torch.equal(wide[:, 4:], y)
    xin = x.clone()
    assert torch.equal(ops.conv_epilogue(xin, **kw), y) and xin.data_ptr() != x.data_ptr()
    fa, fb = ops.fold_bn(C, cuda, gamma=g, beta=b, mean=m, var=v, bias=bias)
    yn = ops.conv_epilogue_nhwc(x.contiguous(memory_format=torch.channels_last), a=fa, b=fb, act=act)
    assert torch.equal(yn.contiguous(), y)


def test_identities_at_full_size(cuda):
    """No parameters and a linear activation is the identity; relu is idempotent; the fused shortcut with a
    linear epilogue is a plain sum; upsample x2 followed by the 2x2/2 max pool returns the input."""
    x = randn((64, 32, 208, 208), cuda, 1)
    assert torch.equal(ops.conv_epilogue(x, act="linear", in_place=False), x)
    r = ops.conv_epilogue(x, act="relu", in_place=False)
    assert torch.equal(ops.conv_epilogue(r, act="relu", in_place=False), r) and torch.equal(r, torch.relu(x))
    frm = randn((64, 32, 208, 208), cuda, 2)
    assert torch.equal(ops.conv_epilogue(x, act="linear", residual=frm, in_place=False), x + frm)
    assert torch.equal(ops.shortcut(x, frm, 1.0, 1.0, "linear"), x + frm)
    del r, frm
    small = randn((64, 256, 38, 38), cuda, 3)
    up = ops.upsample(small, 2, 1.0)
    assert up.shape == (64, 256, 76, 76) and torch.equal(ops.maxpool(up, 2, 2, 1), small)
    assert torch.equal(up, small.repeat_interleave(2, 2).repeat_interleave(2, 3))


def test_yolov3_608_heads_decode_counts_and_order(cuda):
    """The three heads of YOLOv3-608 at 64 images: the number of records equals the number of (cell, slot,
    class) triples PyTorch finds above the threshold, and records come out image-major, then cell, slot, class."""
    anchors = [10, 13, 16, 30, 33, 23, 30, 61, 62, 45, 59, 119, 116, 90, 156, 198, 373, 326]
    thr, classes = 0.6, 80
    buf = ops.DetectionBuffer(1 << 23, cuda)
    start = 0
    for hw, mask in ((19, [6, 7, 8]), (38, [3, 4, 5]), (76, [0, 1, 2])):
        head = randn((64, 255, hw, hw), cuda, hw) * 1.5 - 1.0
        act = ops.yolo_activate(head, 3, classes)
        ops.yolo_decode(act, mask, anchors, classes, 608, 608, thr, buf)
        a = act.view(64, 3, 85, hw * hw)
        obj = a[:, :, 4]
        prob = obj[:, :, None] * a[:, :, 5:]
        want = int(((obj >= thr)[:, :, None] & (prob >= thr)).sum().item())
        total = int(buf.count.item())
        assert total - start == want and total <= buf.capacity
        recs = buf.dets[start:total].cpu().numpy().view(ops.DET_DTYPE).reshape(-1)
        key = (recs["batch_id"].astype(np.int64) * (hw * hw * 3) + recs["source"]) * classes + recs["class_id"]
        assert np.all(np.diff(key) > 0), "records are not in (image, cell, slot, class) order"
        assert recs["prob"].min() >= thr
        start = total


def test_centernet_decode_at_batch_256_against_torch(cuda):
    """BASELINE.json's CenterNet case: [256, 20, 128, 128] logits.  Per image: at most K records, scores
    descending with ties by flat index, every record a thresholded 3x3 local maximum, and the kept scores are
    exactly the K largest candidate scores PyTorch finds."""
    B, classes, H, W, K, thr = 256, 20, 128, 128, 100, 0.2
    heat = randn((B, classes, H, W), cuda, 5) * 2.0 - 4.0
    size = torch.rand((B, 2, H, W), device=cuda, generator=torch.Generator(cuda).manual_seed(6)) + 0.01
    off = torch.rand((B, 2, H, W), device=cuda, generator=torch.Generator(cuda).manual_seed(7))
    d, c = ops.centernet_decode(heat, size, off, thr, K, logits=True, heatmap_bias=0.0)
    counts = c.cpu().numpy()
    recs = ops.centernet_to_host(d, c)
    scores = ops.centernet_activate(torch.cat([heat, size, off], 1), classes, 0.0)[:, :classes]
    peak = (F.max_pool2d(scores, 3, 1, 1) == scores) & (scores >= thr)
    for b in (0, 1, 100, 255):
        r = recs[b]
        assert len(r) == counts[b] == K
        p = r["prob"]
        assert np.all(p[:-1] >= p[1:])
        tie = p[:-1] == p[1:]
        assert np.all(r["source"][:-1][tie] < r["source"][1:][tie])
        flat = torch.from_numpy(r["source"].astype(np.int64)).to(cuda)
        assert bool(peak[b].reshape(-1)[flat].all())
        cand = scores[b][peak[b]]
        top = torch.sort(cand, descending=True).values[:K].cpu().numpy()
        assert np.array_equal(p, top)
