"""Out-of-bounds stores, looked for without a memory checker: every output of every kernel family is carved out
of a larger buffer whose surroundings hold a bit pattern no kernel produces; after the call the surroundings must
be untouched, bit for bit.  Shapes are the odd ones (prime widths, planes smaller than a vector, batch strides
that leave vectors unaligned, the last image ending exactly at the guard) on which an index error would land a
store outside its tensor.  Results are checked elsewhere; here only the guards are."""
import numpy as np
import pytest
import torch

from pixienn_b200 import capi, ops, synth
from test_gpu_epilogue import bn, dev

pytestmark = pytest.mark.gpu

GUARD = 2048                     # elements on each side
PATTERN = 0x7FC5A5A5             # a NaN payload: compares unequal to everything, bit pattern checked as int32


class Guarded:
    """A tensor of `shape` (float32 or int32) in the middle of a buffer filled with PATTERN; `lead` shifts its
    start off 16-byte alignment."""

    def __init__(self, shape, device, dtype=torch.float32, lead=0, fill=None):
        n = int(np.prod(shape))
        self.buf = torch.full((GUARD + lead + n + GUARD,), PATTERN, dtype=torch.int32, device=device)
        self.lo, self.hi = GUARD + lead, GUARD + lead + n
        self.t = self.buf[self.lo:self.hi].view(dtype).view(*shape)
        if fill is not None:
            self.t.copy_(fill)

    def intact(self):
        return bool((self.buf[:self.lo] == PATTERN).all()) and bool((self.buf[self.hi:] == PATTERN).all())


SHAPES = [(2, 3, 13, 13), (1, 5, 19, 19), (3, 2, 7, 5), (1, 1, 1, 1), (2, 7, 1, 3), (1, 2, 37, 31), (2, 4, 26, 26),
          (1, 3, 52, 52), (2, 9, 3, 129), (2, 4, 13, 13), (3, 8, 11, 13), (1, 4, 7, 5)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("lead", [0, 1, 3])
def test_conv_epilogue_stays_inside_its_outputs(cuda, shape, lead):
    B, C, H, W = shape
    x = synth.normal(120, f"gz{shape}", shape)
    _, dp = bn(121, f"gzbn{shape}", C, cuda)
    res = dev(synth.normal(122, f"gzr{shape}", shape), cuda)
    for act in ("leaky", "mish"):
        # plain, into a guarded tensor; with a residual and a second store; in place inside a guarded buffer
        y, y2 = Guarded(shape, cuda, lead=lead), Guarded(shape, cuda, lead=lead)
        ops.conv_epilogue(dev(x, cuda), y=y.t, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act)
        ops.conv_epilogue(dev(x, cuda), y=y.t, y2=y2.t, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act,
                          residual=res, res_act="linear")
        xin = Guarded(shape, cuda, lead=lead, fill=dev(x, cuda))
        ops.conv_epilogue(xin.t, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act)
        # folded pool, both paddings, pooled only and with the full-resolution output
        for pad in (0, 1):
            oh, ow = ops.maxpool_out_dim(H, 2, 2, pad), ops.maxpool_out_dim(W, 2, 2, pad)
            if oh <= 0 or ow <= 0:
                continue
            for variant in (capi.POOL_AUTO, capi.POOL_GENERAL):
                yp = Guarded((B, C, oh, ow), cuda, lead=lead)
                ops.conv_epilogue(dev(x, cuda), y=False, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act,
                                  pool=(2, 2, pad), y_pool=yp.t, pool_variant=variant)
                assert yp.intact(), (act, pad, variant)
                if 2 * oh >= H and 2 * ow >= W:
                    yf, yp2 = Guarded(shape, cuda, lead=lead), Guarded((B, C, oh, ow), cuda, lead=lead)
                    ops.conv_epilogue(dev(x, cuda), y=yf.t, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act,
                                      pool=(2, 2, pad), y_pool=yp2.t, pool_variant=variant)
                    assert yf.intact() and yp2.intact(), (act, pad, variant)
        torch.cuda.synchronize()
        assert y.intact() and y2.intact() and xin.intact(), act


@pytest.mark.parametrize("shape", SHAPES)
def test_channel_slots_of_a_guarded_concat_buffer(cuda, shape):
    """Stores into a channel slot must stay inside the slot: the neighbouring slots and the buffer's surroundings
    keep their pattern."""
    B, C, H, W = shape
    x = dev(synth.normal(123, f"gs{shape}", shape), cuda)
    wide = Guarded((B, C + 5, H, W), cuda, lead=1)
    ops.conv_epilogue(x.clone(), y=wide.t[:, 2:2 + C], act="leaky")
    ops.shortcut(x, x, 1.0, 1.0, "linear", out=wide.t[:, 2:2 + C])
    up = Guarded((B, C + 5, 2 * H, 2 * W), cuda, lead=3)
    ops.upsample(x, 2, 1.0, out=up.t[:, 3:3 + C])
    torch.cuda.synchronize()
    raw = wide.buf[wide.lo:wide.hi].view(B, C + 5, H, W)
    assert wide.intact() and bool((raw[:, :2] == PATTERN).all()) and bool((raw[:, 2 + C:] == PATTERN).all())
    raw = up.buf[up.lo:up.hi].view(B, C + 5, 2 * H, 2 * W)
    assert up.intact() and bool((raw[:, :3] == PATTERN).all()) and bool((raw[:, 3 + C:] == PATTERN).all())


@pytest.mark.parametrize("shape,k,stride", [((2, 3, 13, 13), 2, 1), ((1, 5, 20, 20), 5, 1), ((2, 2, 7, 9), 3, 2),
                                            ((1, 4, 13, 13), 13, 1), ((3, 1, 5, 5), 2, 2)])
def test_pool_kernels_stay_inside_their_outputs(cuda, shape, k, stride):
    B, C, H, W = shape
    x = dev(synth.normal(124, f"gp{shape}", shape), cuda)
    oh, ow = ops.maxpool_out_dim(H, k, stride, k - 1), ops.maxpool_out_dim(W, k, stride, k - 1)
    y = Guarded((B, C, oh, ow), cuda, lead=1)
    ops.maxpool(x, k, stride, out=y.t)
    if stride == 1:
        outs = [Guarded(shape, cuda, lead=i) for i in range(3)]
        ops.spp(x, [5, 9, 13], [o.t for o in outs])
        ident = Guarded(shape, cuda, lead=2)
        a, b = torch.ones(C, device=cuda), torch.zeros(C, device=cuda)
        ops.spp(x, [5, 9, 13], [o.t for o in outs], a=a, b=b, act="swish", y_identity=ident.t)
        torch.cuda.synchronize()
        assert all(o.intact() for o in outs) and ident.intact()
    avg = Guarded((B, C, 1, 1), cuda, lead=1)
    ops.avgpool(x, out=avg.t)
    grad, delta = Guarded(shape, cuda, lead=1, fill=torch.zeros(shape, device=cuda)), dev(synth.normal(125, "gd", (B, C, oh, ow)), cuda)
    _, idx = ops.maxpool(x, k, stride, with_indexes=True)
    ops.maxpool_backward(delta, idx, grad.t)
    torch.cuda.synchronize()
    assert y.intact() and avg.intact() and grad.intact()


def test_channels_last_kernels_stay_inside_their_outputs(cuda):
    for shape in [(2, 4, 13, 13), (1, 12, 7, 5), (2, 36, 3, 3), (1, 8, 26, 26)]:
        B, C, H, W = shape
        x = dev(synth.normal(126, f"gn{shape}", shape), cuda).contiguous(memory_format=torch.channels_last)
        a, b = torch.ones(C, device=cuda), torch.zeros(C, device=cuda)
        y = Guarded((B, H, W, C), cuda)
        yv = y.t.permute(0, 3, 1, 2)                                   # logical [B, C, H, W], channels-last storage
        ops.conv_epilogue_nhwc(x.clone(), y=yv, a=a, b=b, act="leaky")
        oh, ow = ops.maxpool_out_dim(H, 2, 2, 1), ops.maxpool_out_dim(W, 2, 2, 1)
        yp = Guarded((B, oh, ow, C), cuda)
        ops.conv_epilogue_nhwc(x.clone(), y=False, a=a, b=b, act="leaky", pool=(2, 2, 1), y_pool=yp.t.permute(0, 3, 1, 2))
        up = Guarded((B, 2 * H, 2 * W, C), cuda)
        ops.upsample_nhwc(x, 2, 1.0, out=up.t.permute(0, 3, 1, 2))
        torch.cuda.synchronize()
        assert y.intact() and yp.intact() and up.intact(), shape


def test_decodes_stay_inside_their_record_buffers(cuda):
    """A detection buffer with room for fewer records than the head emits: the count keeps running, the stores
    stop at the capacity."""
    B, classes, hw = 2, 5, 13
    raw = synth.normal(127, "gy", (B, 3 * (classes + 5), hw, hw), 0.0, 2.0)
    buf = ops.DetectionBuffer(64, cuda)
    g = Guarded((64, 8), cuda, dtype=torch.int32)
    buf.dets = g.t
    ops.yolo_decode(ops.yolo_activate(dev(raw, cuda), 3, classes), [0, 1, 2], [10, 14, 23, 27, 37, 58], classes, 416, 416, 0.2, buf)
    torch.cuda.synchronize()
    assert int(buf.count.item()) > 64 and g.intact()
    from test_gpu_heads import centernet_case
    heat, size, off = centernet_case(128, 3, 4, 37, 70)
    d, c = ops.centernet_decode(dev(heat, cuda), dev(size, cuda), dev(off, cuda), 0.2, 7, logits=True)
    assert int(c.max().item()) <= 7


@pytest.mark.parametrize("shape", [(3, 5, 13, 13), (4, 8, 13, 13), (2, 6, 16, 16), (64, 3, 1, 1), (1, 2, 95, 97)])
def test_training_side_calls_stay_inside_their_outputs(cuda, shape):
    """Batch norm with batch statistics (all outputs, both directions), the Adam step and the softmax loss."""
    import ctypes as C
    B, Cc, H, W = shape
    x = dev(synth.normal(128, f"gt{shape}", shape, 0.5, 2.0), cuda)
    g, b = torch.rand(Cc, device=cuda) + 0.5, torch.randn(Cc, device=cuda)
    y, ya, dx = Guarded(shape, cuda, lead=1), Guarded(shape, cuda, lead=2), Guarded(shape, cuda, lead=3)
    sm, ss, rm, rv, dg, db = (Guarded((Cc,), cuda, lead=1, fill=torch.ones(Cc, device=cuda)) for _ in range(6))
    nbytes = capi.lib().pxe_batchnorm_workspace_bytes(B, Cc, H, W)
    ws = torch.empty(nbytes + 4096, device=cuda, dtype=torch.uint8)
    ws[nbytes:] = 0xA5
    d = capi.BnTrainDesc()
    d.x, d.y, d.y_act, d.act = x.data_ptr(), y.t.data_ptr(), ya.t.data_ptr(), capi.ACT["mish"]
    d.batch, d.channels, d.height, d.width = shape
    d.gamma, d.beta, d.running_mean, d.running_var = g.data_ptr(), b.data_ptr(), rm.t.data_ptr(), rv.t.data_ptr()
    d.exp_avg_factor, d.eps, d.save_mean, d.save_scale = 0.01, 1e-5, sm.t.data_ptr(), ss.t.data_ptr()
    d.workspace, d.workspace_bytes = ws.data_ptr(), nbytes
    capi.check(capi.lib().pxe_batchnorm_forward_training(None, C.byref(d)))
    e = capi.BnBackwardDesc()
    dy = dev(synth.normal(129, f"gdy{shape}", shape), cuda)
    e.x, e.dy, e.dx = x.data_ptr(), dy.data_ptr(), dx.t.data_ptr()
    e.batch, e.channels, e.height, e.width = shape
    e.gamma, e.dgamma, e.dbeta = g.data_ptr(), dg.t.data_ptr(), db.t.data_ptr()
    e.save_mean, e.save_scale, e.eps = sm.t.data_ptr(), ss.t.data_ptr(), 1e-5
    e.workspace, e.workspace_bytes = ws.data_ptr(), nbytes
    capi.check(capi.lib().pxe_batchnorm_backward(None, C.byref(e)))
    n = x.numel()
    px, pm, pv = Guarded((n,), cuda, lead=1, fill=x.flatten()), torch.randn(n, device=cuda), torch.rand(n, device=cuda)
    ops.adam_update(px.t, pm, pv, 0.9, 0.999, -1e-3, 1e-8, 3)
    delta, err = Guarded((n,), cuda, lead=3), Guarded((n,), cuda, lead=1)
    pred, truth = torch.rand(n, device=cuda), (torch.rand(n, device=cuda) > 0.9).float()
    capi.check(capi.lib().pxe_softmax_cross_entropy(None, n, pred.data_ptr(), truth.data_ptr(), delta.t.data_ptr(), err.t.data_ptr()))
    torch.cuda.synchronize()
    assert all(t.intact() for t in (y, ya, dx, sm, ss, rm, rv, dg, db, px, delta, err))
    assert bool((ws[nbytes:] == 0xA5).all())


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("lead", [0, 1, 2])
def test_reads_outside_the_inputs_never_reach_the_outputs(cuda, shape, lead):
    """The reading side of the same question: every input is carved out of a buffer whose surroundings hold NaNs (the
    pattern above is one), at an offset that breaks 16-byte alignment, and the results must equal, bit for bit, those
    computed from ordinary tensors.  A tap, a vector or a plane index that strays outside an input would drag a NaN
    (or a neighbour's value) into some output."""
    B, C, H, W = shape
    xh = synth.normal(140, f"rx{shape}", shape)
    rh = synth.normal(141, f"rr{shape}", shape)
    _, dp = bn(142, f"rbn{shape}", C, cuda)
    plain_x, plain_r = dev(xh, cuda), dev(rh, cuda)
    gx, gr = Guarded(shape, cuda, lead=lead, fill=plain_x), Guarded(shape, cuda, lead=lead, fill=plain_r)

    def both(fn):
        a, b = fn(plain_x, plain_r), fn(gx.t, gr.t)
        a, b = (a if isinstance(a, (list, tuple)) else [a]), (b if isinstance(b, (list, tuple)) else [b])
        for u, v in zip(a, b):
            if u is not None:
                assert torch.equal(u.contiguous().view(torch.int32), v.contiguous().view(torch.int32))

    kw = dict(gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3])
    for act in ("leaky", "swish"):
        both(lambda x, r: ops.conv_epilogue(x, y=torch.empty(shape, device=cuda), act=act, **kw))
        both(lambda x, r: ops.conv_epilogue(x, y=torch.empty(shape, device=cuda), act=act, residual=r, res_act="leaky", **kw))
        for pad in (0, 1):
            oh, ow = ops.maxpool_out_dim(H, 2, 2, pad), ops.maxpool_out_dim(W, 2, 2, pad)
            if oh > 0 and ow > 0:
                for variant in (capi.POOL_AUTO, capi.POOL_GENERAL):
                    both(lambda x, r: ops.conv_epilogue(x, y=False, act=act, pool=(2, 2, pad), pool_variant=variant, **kw)[1])
    both(lambda x, r: ops.shortcut(x, r, 0.5, 2.0, "leaky", out=torch.empty(shape, device=cuda)))
    both(lambda x, r: ops.upsample(x, 2, 0.5))
    both(lambda x, r: ops.concat([x, r]))
    both(lambda x, r: ops.avgpool(x))
    for k, s_ in ((2, 1), (3, 2), (5, 1), (13, 1)):
        if ops.maxpool_out_dim(H, k, s_, k - 1) > 0 and ops.maxpool_out_dim(W, k, s_, k - 1) > 0:
            both(lambda x, r: list(ops.maxpool(x, k, s_, with_indexes=True)))
            both(lambda x, r: ops.maxpool(x, k, s_))
    both(lambda x, r: list(ops.spp(x, [5, 9, 13], [torch.empty(shape, device=cuda) for _ in range(3)])))
    # batch-norm statistics are sums whose grouping depends on whether the input allows 128-bit loads: equal to rounding
    # of the sums, and free of NaNs
    a = ops.batchnorm_forward_training(plain_x, dp[0], dp[1], act="leaky")
    b = ops.batchnorm_forward_training(gx.t.contiguous() if not gx.t.is_contiguous() else gx.t, dp[0], dp[1], act="leaky")
    for u, v in zip(a, b):
        torch.testing.assert_close(u, v, rtol=1e-5, atol=1e-6)
    torch.cuda.synchronize()
