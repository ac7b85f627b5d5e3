"""Host logic of the optional cuDNN conv + epilogue fusion: which layers are eligible and how a destination
that is a channel slot of a concat buffer is described to cuDNN (no GPU, no cuDNN call)."""
import pytest
import torch

from pixienn_b200.cudnn_fused import FusedConvPlanner, _pixel_stride


def nhwc(shape):
    return torch.empty(shape).contiguous(memory_format=torch.channels_last)


def test_pixel_stride_of_dense_tensors_and_channel_slots():
    t = nhwc((2, 16, 8, 8))
    assert _pixel_stride(t) == 16
    wide = nhwc((2, 48, 8, 8))
    assert _pixel_stride(wide[:, 16:32]) == 48          # a route's slot: same pixels, the buffer's channel count
    assert _pixel_stride(torch.empty(2, 16, 8, 8)) is None      # NCHW
    assert _pixel_stride(nhwc((2, 16, 1, 1))) is None            # no pixel grid to take a stride from
    assert _pixel_stride(nhwc((1, 16, 8, 1))) == 16


def test_key_accepts_what_the_graph_can_express_and_nothing_else():
    x, w, out = nhwc((2, 8, 16, 16)), nhwc((16, 8, 3, 3)), nhwc((2, 16, 16, 16))
    k = FusedConvPlanner.key(x, w, 1, 1, "leaky", out, None, "linear")
    assert k == ((2, 8, 16, 16), (16, 8, 3, 3), 1, 1, "leaky", (2, 16, 16, 16), 16, 0, "linear")
    res = nhwc((2, 40, 16, 16))[:, 8:24]
    k2 = FusedConvPlanner.key(x, w, 1, 1, "swish", out, res, "leaky")
    assert k2[6:] == (16, 40, "leaky") and k2 != k
    assert FusedConvPlanner.key(x, w, 1, 1, "mish", out, None, "linear") is None          # no cuDNN pointwise op
    assert FusedConvPlanner.key(x, w, 1, 1, "leaky", out, res, "mish") is None
    assert FusedConvPlanner.key(torch.empty(2, 8, 16, 16), w, 1, 1, "leaky", out, None, "linear") is None   # NCHW input
    assert FusedConvPlanner.key(x, w, 1, 1, "leaky", torch.empty(2, 16, 16, 16), None, "linear") is None     # NCHW output
    assert FusedConvPlanner.key(x, nhwc((1, 8, 3, 3)), 1, 1, "leaky", nhwc((2, 1, 16, 16)), None, "linear") is None
    # keys work on meta tensors: the runner asks before it allocates the destination
    probe = torch.empty_strided((2, 16, 16, 16), (16 * 16 * 24, 1, 16 * 24, 24), device="meta")
    assert FusedConvPlanner.key(x, w, 1, 1, "leaky", probe, None, "linear")[6] == 24


def test_tensor_of_another_device_is_refused(monkeypatch):
    """The library launches on the current device: a tensor that lives elsewhere is refused before any launch."""
    import torch
    from pixienn_b200 import ops
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    ops._check_device(0, "x")
    with pytest.raises(ValueError, match="cuda:1 but the current device is cuda:0"):
        ops._check_device(1, "x")
