"""The reference checks its layers against tensors generated with PyTorch from a layer spec (its
tests/src/model.cpp:179-266 reads them from an HDF5 file written by python/compile_model_spec.py:216-310:
seed 42, uniform weights, conv -> batch_norm(eps 1e-5) -> activation, MaxPool2d, Linear).  The file needs h5py
and an image that are not available here, so the same generation runs in place, layer by layer in isolation as
in that test, on a seeded synthetic image, and this library's calls are compared with PyTorch's results."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from pixienn_b200 import ops

pytestmark = pytest.mark.gpu

# python/specs/model_test.yaml: the YOLOv1-tiny trunk on a 1 x 448 x 448 image
SPEC = [("conv", 16), ("maxpool",), ("conv", 32), ("maxpool",), ("conv", 64), ("maxpool",), ("conv", 128), ("maxpool",),
        ("conv", 256), ("maxpool",), ("conv", 512), ("maxpool",), ("conv", 1024), ("conv", 256), ("connected", 1470)]


def close(got, ref, what):
    scale = float(ref.abs().max()) + 1e-12
    err = float((got - ref).abs().max())
    assert err <= 2e-5 * scale, f"{what}: max abs err {err} against a range of {scale}"


def test_layers_match_the_pytorch_generated_spec(cuda):
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        torch.manual_seed(42)
        x = torch.rand((1, 1, 448, 448), device=cuda)
        with torch.no_grad():
            for i, layer in enumerate(SPEC):
                nxt = SPEC[i + 1] if i + 1 < len(SPEC) else None
                if layer[0] == "conv":
                    filters = layer[1]
                    w = torch.empty(filters, x.shape[1], 3, 3, device=cuda).uniform_(0.0, 1.0)
                    bias = torch.empty(filters, device=cuda).uniform_(0.0, 1.0)
                    out = F.conv2d(x, w, bias, stride=1, padding=1)
                    mean = torch.empty(filters, device=cuda).uniform_(0.0, 1.0)
                    var = torch.empty(filters, device=cuda).uniform_(0.5, 1.5)
                    scale = torch.empty(filters, device=cuda).uniform_(0.5, 1.5)
                    ref = F.leaky_relu(F.batch_norm(out, mean, var, scale, bias, False, 0.0, 1e-5), 0.1)
                    # the generator adds the bias before normalising AND uses it as beta: the first is a shift of the mean
                    raw = F.conv2d(x, w, None, stride=1, padding=1)
                    kw = dict(gamma=scale, beta=bias, mean=mean - bias, var=var, act="leaky")
                    if nxt is not None and nxt[0] == "maxpool":
                        y, yp = ops.conv_epilogue(raw.clone(), pool=(2, 2, 0), **kw)
                        close(yp, F.max_pool2d(ref, 2, 2, 0), f"layer {i} pooled")
                        assert torch.equal(yp, F.max_pool2d(y, 2, 2, 0))
                    else:
                        y = ops.conv_epilogue(raw.clone(), **kw)
                    close(y, ref, f"layer {i} conv")
                    x = ref
                elif layer[0] == "maxpool":
                    ref = F.max_pool2d(x, 2, 2, 0)
                    assert torch.equal(ops.maxpool(x, 2, 2, 0), ref), f"layer {i} maxpool"
                    x = ref
                else:
                    flat = x.reshape(x.shape[0], -1)
                    w = torch.empty(layer[1], flat.shape[1], device=cuda).uniform_(0.0, 1.0)
                    bias = torch.empty(layer[1], device=cuda).uniform_(0.0, 1.0)
                    ref = F.linear(flat, w, bias)
                    raw = F.linear(flat, w).reshape(x.shape[0], layer[1], 1, 1)
                    y = ops.conv_epilogue(raw, bias=bias, act="linear")
                    close(y.reshape(ref.shape), ref, f"layer {i} connected")
                    x = ref
    finally:
        torch.backends.cudnn.allow_tf32 = old
