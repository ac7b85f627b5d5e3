"""GPU parity: batch normalisation in training mode, forward and backward, against the oracle (both arithmetic
modes: the reference's CPU code, to which the oracle is pinned, and cuDNN's documented forms, which the reference's
CUDA layers call) and against PyTorch's own batch norm and autograd.  Floating point with sums over batch * H * W
terms taken in different orders: tolerances are relative to the tensors' scale and written at each comparison."""
import ctypes as C

import numpy as np
import pytest
import torch

from pixienn_b200 import capi, ops, synth
from test_gpu_epilogue import dev

pytestmark = pytest.mark.gpu

SHAPES = [(4, 8, 16, 16), (3, 5, 13, 13), (2, 32, 52, 52), (64, 6, 1, 1), (2, 2, 200, 200), (1, 3, 7, 5), (5, 4, 19, 19),
          (4, 8, 13, 13), (16, 12, 13, 13), (2, 1030, 3, 3)]


def params(C_, seed):
    g, b, rm, rv = synth.bn_params(seed, f"bnt{C_}", C_)
    return g, b, rm, rv


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("eps_mode", [capi.EPS_CUDNN, capi.EPS_CPU])
def test_forward_training_equals_the_oracle(cuda, oracle, shape, eps_mode):
    B, Cc, H, W = shape
    x = synth.normal(130, f"x{shape}", shape, 0.7, 2.0)
    g, b, rm, rv = params(Cc, 131)
    y_ref, rm_ref, rv_ref, sm_ref, ss_ref = oracle.batchnorm_forward_training(x, g, b, rm, rv, 0.01, 1e-5, eps_mode)
    drm, drv = dev(rm, cuda), dev(rv, cuda)
    y, y_act, sm, ss = ops.batchnorm_forward_training(dev(x, cuda), dev(g, cuda), dev(b, cuda), running_mean=drm,
                                                      running_var=drv, eps_mode=eps_mode, act="leaky")
    np.testing.assert_allclose(sm.cpu().numpy(), sm_ref, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ss.cpu().numpy(), ss_ref, rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(drm.cpu().numpy(), rm_ref, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(drv.cpu().numpy(), rv_ref, rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=1e-4, atol=2e-5)
    # the activated output is the activation of exactly the y that was stored
    assert np.array_equal(y_act.cpu().numpy(), oracle.activate("leaky", y.cpu().numpy()))


@pytest.mark.parametrize("shape", SHAPES)
def test_forward_and_backward_equal_pytorch(cuda, shape):
    """cuDNN mode against torch.nn.functional.batch_norm(training=True) and its autograd: y, both running statistics
    (momentum = the reference's 0.01, unbiased variance), dx, dgamma, dbeta."""
    B, Cc, H, W = shape
    x = dev(synth.normal(132, f"tx{shape}", shape, -0.3, 1.7), cuda)
    g, b, rm, rv = (dev(t, cuda) for t in params(Cc, 133))
    xt = x.clone().requires_grad_(True)
    gt, bt = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    trm, trv = rm.clone(), rv.clone()
    with torch.backends.cudnn.flags(enabled=True):
        yt = torch.nn.functional.batch_norm(xt, trm, trv, gt, bt, training=True, momentum=0.01, eps=1e-5)
    dy = dev(synth.normal(134, f"tdy{shape}", shape, 0, 1.3), cuda)
    yt.backward(dy)
    y, _, sm, ss = ops.batchnorm_forward_training(x, g, b, running_mean=rm, running_var=rv)
    scale = float(yt.detach().abs().max())
    assert float((y - yt).abs().max()) <= 2e-5 * max(1.0, scale)
    torch.testing.assert_close(rm, trm, rtol=1e-5, atol=1e-6)
    if B * H * W > 1:
        torch.testing.assert_close(rv, trv, rtol=1e-4, atol=1e-6)
    dg0, db0 = torch.full((Cc,), 0.5, device=cuda), torch.full((Cc,), -0.25, device=cuda)
    dg, db = dg0.clone(), db0.clone()
    dx = ops.batchnorm_backward(x, dy, g, sm, ss, dgamma=dg, dbeta=db)
    n = B * H * W
    torch.testing.assert_close(db - db0, bt.grad, rtol=1e-4, atol=1e-5 * n ** 0.5)
    torch.testing.assert_close(dg - dg0, gt.grad, rtol=1e-4, atol=2e-5 * n ** 0.5)
    assert float((dx - xt.grad).abs().max()) <= 1e-4 * max(1.0, float(xt.grad.abs().max()))


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("eps_mode", [capi.EPS_CUDNN, capi.EPS_CPU])
def test_backward_equals_the_oracle(cuda, oracle, shape, eps_mode):
    B, Cc, H, W = shape
    x = synth.normal(135, f"bx{shape}", shape, 0.4, 1.5)
    dy = synth.normal(136, f"bdy{shape}", shape, 0, 2.0)
    g, b, rm, rv = params(Cc, 137)
    _, _, _, sm, ss = oracle.batchnorm_forward_training(x, g, b, rm, rv, 0.01, 1e-5, eps_mode)
    dg0, db0 = synth.normal(138, "dg", Cc), synth.normal(138, "db", Cc)
    dx_ref, dg_ref, db_ref = oracle.batchnorm_backward(x, dy, g, sm, ss, dg0, db0, 1e-5, eps_mode)
    dg, db = dev(dg0, cuda), dev(db0, cuda)
    ddy = dev(dy, cuda)
    dx = ops.batchnorm_backward(dev(x, cuda), ddy, dev(g, cuda), dev(sm, cuda), dev(ss, cuda), dgamma=dg, dbeta=db,
                                eps_mode=eps_mode)
    n = B * H * W
    np.testing.assert_allclose(db.cpu().numpy(), db_ref, rtol=1e-4, atol=1e-5 * n ** 0.5)
    np.testing.assert_allclose(dg.cpu().numpy(), dg_ref, rtol=1e-4, atol=2e-5 * n ** 0.5)
    np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=1e-4, atol=1e-4 * max(1.0, float(np.abs(dx_ref).max())))
    # in place on dy, without parameter gradients: the same dx
    dx2 = ops.batchnorm_backward(dev(x, cuda), ddy, dev(g, cuda), dev(sm, cuda), dev(ss, cuda), eps_mode=eps_mode, dx=ddy)
    assert dx2 is ddy and torch.equal(dx2, dx)


def test_in_place_fixed_order_and_refusals(cuda):
    shape = (8, 16, 26, 26)
    x = dev(synth.normal(139, "ip", shape, 3.0, 0.5), cuda)        # |mean| >> sigma: the shifted sums keep the variance
    g, b = torch.ones(16, device=cuda), torch.zeros(16, device=cuda)
    y1, _, m1, s1 = ops.batchnorm_forward_training(x, g, b)
    y2, _, m2, s2 = ops.batchnorm_forward_training(x, g, b)
    assert torch.equal(y1, y2) and torch.equal(m1, m2) and torch.equal(s1, s2)          # same bits every time
    assert float(y1.mean(dim=(0, 2, 3)).abs().max()) < 1e-5 and float((y1.var(dim=(0, 2, 3), unbiased=False) - 1).abs().max()) < 1e-3
    xin = x.clone()
    y3, _, _, _ = ops.batchnorm_forward_training(xin, g, b, y=xin)
    assert y3 is xin and torch.equal(y3, y1)
    # refusals: a short workspace, an activated output that aliases x
    d = capi.BnTrainDesc()
    sm = torch.empty(16, device=cuda)
    ws = torch.empty(64, device=cuda, dtype=torch.uint8)
    d.x, d.y, d.batch, d.channels, d.height, d.width = x.data_ptr(), y1.data_ptr(), *shape
    d.gamma, d.beta, d.save_mean, d.save_scale = g.data_ptr(), b.data_ptr(), sm.data_ptr(), sm.data_ptr()
    d.workspace, d.workspace_bytes, d.eps = ws.data_ptr(), 64, 1e-5
    assert capi.lib().pxe_batchnorm_forward_training(None, C.byref(d)) == capi.PXE_ERR_BAD_ARG
    need = capi.lib().pxe_batchnorm_workspace_bytes(*shape)
    ws = torch.empty(need, device=cuda, dtype=torch.uint8)
    d.workspace, d.workspace_bytes, d.y_act = ws.data_ptr(), need, x.data_ptr()
    assert capi.lib().pxe_batchnorm_forward_training(None, C.byref(d)) == capi.PXE_ERR_BAD_ARG
    torch.cuda.synchronize()
