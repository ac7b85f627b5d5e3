"""GPU parity: max pooling (fused and stand-alone), SPP, upsample, route concat -- all bit-exact
against the CPU oracle (np.array_equal, i.e. -0.0 == +0.0; NaN positions compared separately)."""
import numpy as np
import pytest
import torch

from pixienn_b200 import capi, ops, synth
from test_gpu_epilogue import bn, close, dev

pytestmark = pytest.mark.gpu


def same(got, ref):
    got, ref = np.asarray(got), np.asarray(ref)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    nan_g, nan_r = np.isnan(got), np.isnan(ref)
    assert np.array_equal(nan_g, nan_r)
    assert np.array_equal(got[~nan_g], ref[~nan_r]), f"{(got != ref).sum()} values differ"


POOL_CASES = [
    # (shape, kernel, stride, padding)      padding None = layer default kernel-1
    ((2, 3, 16, 16), 2, 2, None), ((2, 3, 13, 13), 2, 2, None), ((1, 4, 26, 26), 2, 2, None),
    ((2, 2, 52, 52), 2, 2, None), ((1, 2, 8, 24), 2, 2, None), ((2, 3, 13, 13), 2, 1, None),
    ((1, 2, 3, 3), 2, 1, 1), ((2, 3, 20, 20), 5, 1, None), ((1, 2, 20, 20), 9, 1, None),
    ((1, 2, 20, 20), 13, 1, None), ((2, 3, 9, 11), 3, 2, 1), ((1, 2, 7, 7), 3, 2, 0),
    ((1, 2, 8, 8), 2, 2, 0), ((1, 2, 9, 9), 2, 2, 0), ((1, 1, 5, 5), 3, 3, 4),
]


@pytest.mark.parametrize("shape,k,s,pad", POOL_CASES)
def test_maxpool_values_and_indexes(cuda, oracle, shape, k, s, pad):
    x = synth.normal(30, f"p{shape}{k}{s}{pad}", shape)
    ref_v, ref_i = oracle.maxpool(x, k, s, pad)
    out, idx = ops.maxpool(dev(x, cuda), k, s, pad, with_indexes=True)
    same(out.cpu().numpy(), ref_v)
    assert np.array_equal(idx.cpu().numpy(), ref_i)
    same(ops.maxpool(dev(x, cuda), k, s, pad).cpu().numpy(), ref_v)     # vectorised 2x2 path has no indexes


def test_maxpool_reference_known_answer(cuda):
    """3x3 input, kernel 2, stride 1, padding 1: window origin -1/2 == 0, so only the bottom/right
    edges see out-of-range taps (the reference's CUDA maxpool test)."""
    x = np.arange(1, 10, dtype=np.float32).reshape(1, 1, 3, 3)
    out, idx = ops.maxpool(dev(x, cuda), 2, 1, 1, with_indexes=True)
    assert out.cpu().numpy().ravel().tolist() == [5, 6, 6, 8, 9, 9, 8, 9, 9]
    assert idx.cpu().numpy().ravel().tolist() == [4, 5, 5, 7, 8, 8, 7, 8, 8]


def test_maxpool_ties_nan_and_signed_zero(cuda, oracle):
    x = np.zeros((1, 1, 4, 4), np.float32)
    x[0, 0] = [[1, 1, -0.0, 0.0], [1, 1, 0.0, -0.0], [np.nan, 5, 3, np.nan], [2, 7, np.nan, 4]]
    for k, s, pad in [(2, 2, 1), (2, 1, 1), (3, 1, 2)]:
        ref_v, ref_i = oracle.maxpool(x, k, s, pad)
        out, idx = ops.maxpool(dev(x, cuda), k, s, pad, with_indexes=True)
        g = out.cpu().numpy()
        same(g, ref_v)
        assert np.array_equal(np.signbit(g[~np.isnan(g)]), np.signbit(ref_v[~np.isnan(ref_v)]))
        assert np.array_equal(idx.cpu().numpy(), ref_i)
        g2 = ops.maxpool(dev(x, cuda), k, s, pad).cpu().numpy()
        same(g2, ref_v)
        assert np.array_equal(np.signbit(g2[~np.isnan(g2)]), np.signbit(ref_v[~np.isnan(ref_v)]))


@pytest.mark.parametrize("shape", [(2, 4, 16, 16), (2, 3, 13, 13), (1, 5, 26, 26), (2, 2, 52, 52), (1, 3, 8, 24),
                                   (1, 2, 7, 12), (2, 37, 13, 13), (1, 10, 26, 26), (1, 2, 104, 104),
                                   (2, 8, 13, 13), (3, 4, 13, 13), (2, 36, 13, 13), (1, 12, 11, 11), (2, 4, 9, 13), (1, 8, 7, 7)])
@pytest.mark.parametrize("act", ["leaky", "mish", "swish", "logistic"])
@pytest.mark.parametrize("keep_full", [False, True])
@pytest.mark.parametrize("variant", [capi.POOL_AUTO, capi.POOL_GENERAL])
def test_epilogue_with_folded_pool(cuda, oracle, shape, act, keep_full, variant):
    """BN + bias + activation + 2x2/2 maxpool in one pass == the oracle's separate layers.
    Pooling picks among the SAME activated values, so pooled == maxpool(full) exactly.
    pool_variant = PXE_POOL_GENERAL runs the general pooled kernel where the even-height fast form would run."""
    B, C, H, W = shape
    x = synth.normal(31, f"x{shape}", shape)
    (g, b, m, v), dp = bn(32, f"bn{shape}", C, cuda)
    bias = synth.normal(33, f"b{shape}", C, 0, 0.1)
    ref_full = oracle.conv_epilogue(x, g, b, m, v, bias, act)
    xd = dev(x, cuda)
    y, yp = ops.conv_epilogue(xd, y=None if keep_full else False, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3],
                              bias=dev(bias, cuda), act=act, pool=(2, 2, 1), pool_variant=variant)
    if keep_full:
        close(y.cpu().numpy(), ref_full)
        full = y.cpu().numpy()
    else:
        assert y is None
        assert np.array_equal(xd.cpu().numpy(), x)
        full = ops.conv_epilogue(dev(x, cuda), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], bias=dev(bias, cuda),
                                 act=act).cpu().numpy()
    close(yp.cpu().numpy(), oracle.maxpool(ref_full, 2, 2, 1)[0])
    same(yp.cpu().numpy(), oracle.maxpool(full, 2, 2, 1)[0])


@pytest.mark.parametrize("shape", [(3, 5, 7, 7), (2, 37, 13, 13), (2, 9, 19, 19), (1, 11, 27, 27), (1, 3, 33, 33),
                                   (1, 70, 5, 9), (2, 130, 13, 13), (1, 4, 3, 31), (2, 8, 13, 13), (1, 132, 13, 13),
                                   (3, 4, 11, 13), (2, 12, 7, 7), (1, 8, 9, 5), (2, 5, 26, 26), (1, 3, 22, 22), (2, 2, 6, 10), (1, 7, 3, 12), (1, 4, 18, 14)])
@pytest.mark.parametrize("act", ["leaky", "mish"])
@pytest.mark.parametrize("padding", [0, 1])
def test_folded_pool_small_odd_planes(cuda, oracle, shape, act, padding):
    """Odd widths with 33 to 128 pooled outputs per plane (13x13, 19x19 here) run the warp-per-plane form (two or
    four output slots per lane), planes of 33 to 192 elements in aligned tensors with channels in fours the flat
    vector form, the other shapes the general one; the former two must equal the general scalar
    form bit for bit (pool_variant = PXE_POOL_GENERAL runs that one) and the oracle's separate layers, pooled-only and with the full-resolution output, dense and into channel
    slots of wider buffers, NaNs included."""
    B, C, H, W = shape
    x = synth.normal(36, f"sp{shape}", shape)
    x[0, 0, 0, 0] = np.nan
    x[-1, -1, -1, -1] = np.nan
    (g, b, m, v), dp = bn(37, f"spbn{shape}", C, cuda)
    oh, ow = (H + padding - 2) // 2 + 1, (W + padding - 2) // 2 + 1
    covered = 2 * oh >= H and 2 * ow >= W
    got = {}
    for env, variant in (("1", capi.POOL_AUTO), ("0", capi.POOL_GENERAL)):
        wide = torch.full((B, C + 3, oh, ow), 9.0, device=cuda)
        wide_full = torch.full((B, C + 4, H, W), 7.0, device=cuda)       # slot at four planes: 16-byte aligned
        _, yp = ops.conv_epilogue(dev(x, cuda), y=False, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act,
                                  pool=(2, 2, padding), pool_variant=variant)
        # the full-resolution output is offered only where the windows cover every input element
        ops.conv_epilogue(dev(x, cuda), y=wide_full[:, 4:] if covered else False, gamma=dp[0], beta=dp[1], mean=dp[2],
                          var=dp[3], act=act, pool=(2, 2, padding), y_pool=wide[:, 3:], pool_variant=variant)
        assert bool((wide[:, :3] == 9.0).all()) and bool((wide_full[:, :4] == 7.0).all())
        got[env] = (yp.cpu().numpy(), wide[:, 3:].cpu().numpy(), wide_full[:, 4:].cpu().numpy())
    for a, c in zip(got["1"], got["0"]):
        same(a, c)
    yp, yp_slot, full = got["1"]
    same(yp, yp_slot)
    ref_full = oracle.conv_epilogue(x, g, b, m, v, None, act)
    if covered:
        close(full, ref_full)
        same(yp, oracle.maxpool(full, 2, 2, padding)[0])
    close(yp, oracle.maxpool(ref_full, 2, 2, padding)[0])


@pytest.mark.parametrize("shape", [(2, 6, 16, 16), (3, 5, 12, 20), (2, 3, 10, 6)])
def test_folded_pool_into_concat_slot(cuda, oracle, shape):
    """Pooled output AND the full-resolution output stored into channel slots of wider buffers."""
    B, C, H, W = shape
    x = synth.normal(34, f"xs{shape}", (B, C, H, W))
    wide = torch.full((B, C + 5, H // 2, W // 2), 9.0, device=cuda)
    wide_full = torch.full((B, C + 4, H, W), 7.0, device=cuda)
    _, yp = ops.conv_epilogue(dev(x, cuda), y=wide_full[:, 4:], act="leaky", pool=(2, 2, 1), y_pool=wide[:, 5:])
    full = oracle.activate("leaky", x)
    same(wide[:, 5:].cpu().numpy(), oracle.maxpool(full, 2, 2, 1)[0])
    same(wide_full[:, 4:].cpu().numpy(), full)
    assert (wide[:, :5] == 9.0).all() and (wide_full[:, :4] == 7.0).all()


@pytest.mark.parametrize("shape", [(2, 8, 20, 20), (1, 3, 13, 13), (2, 2, 19, 19), (1, 2, 5, 40)])
def test_spp_block(cuda, oracle, shape):
    B, C, H, W = shape
    x = synth.normal(35, f"spp{shape}", shape)
    # the SPP concat of yolov7: [pool13, pool9, pool5, x] as slots of one buffer
    cat = torch.zeros((B, 4 * C, H, W), device=cuda)
    xd = dev(x, cuda)
    ops.spp(xd, [13, 9, 5], [cat[:, 0:C], cat[:, C:2 * C], cat[:, 2 * C:3 * C]])
    cat[:, 3 * C:] = xd
    ref = oracle.route([oracle.maxpool(x, 13, 1)[0], oracle.maxpool(x, 9, 1)[0], oracle.maxpool(x, 5, 1)[0], x])
    same(cat.cpu().numpy(), ref)


def test_spp_block_nan_infinities_and_signed_zeros(cuda, oracle):
    """The row / column form of the SPP kernel keeps the reference scan's corner cases: a NaN as the first tap of
    a window is the result, NaNs elsewhere are ignored, -inf planes stay -inf, the first of +0 / -0 wins."""
    B, C, H, W = 1, 6, 12, 12
    x = synth.normal(36, "sppnan", (B, C, H, W))
    x[0, 0, 0, 0] = np.nan                     # first tap of the windows in the top-left corner
    x[0, 0, 5, 5] = np.nan
    x[0, 1, 3, :] = np.nan                     # a whole row of NaNs
    x[0, 2] = -np.inf
    x[0, 3] = 0.0
    x[0, 3, ::2, ::2] = -0.0
    x[0, 4, 6, 6] = np.inf
    x[0, 5, :, 0] = np.nan                     # first column: first tap of every window that touches it
    outs = [torch.empty((B, C, H, W), device=cuda) for _ in range(3)]
    ops.spp(dev(x, cuda), [13, 9, 5], outs)
    for k, o in zip((13, 9, 5), outs):
        ref = oracle.maxpool(x, k, 1)[0]
        got = o.cpu().numpy()
        assert np.array_equal(np.isnan(got), np.isnan(ref))
        m = ~np.isnan(ref)
        assert np.array_equal(got[m], ref[m]) and np.array_equal(np.signbit(got[m]), np.signbit(ref[m]))


@pytest.mark.parametrize("shape", [(3, 5, 20, 20), (2, 7, 19, 19), (1, 9, 13, 13), (1, 3, 24, 24), (2, 3, 7, 9), (1, 2, 33, 31),
                                   (1, 2, 40, 40), (2, 3, 1, 1), (1, 4, 3, 50), (1, 130, 20, 20)])
@pytest.mark.parametrize("kernels", [(5, 9, 13), (13, 9, 5), (5,), (9,), (13, 5), (9, 13), (3, 7), (5, 9, 13, 17)])
def test_spp_any_subset_and_order_against_the_scan(cuda, oracle, shape, kernels):
    """Planes that fit three copies per warp in shared memory run the chain of 5-wide row windows for any subset and order of
    5 / 9 / 13 (dense aligned tensors with 128-bit moves, anything else element by element), other kernel sizes
    and larger planes the row / column form: every output equals the reference scan bit for bit, into dense
    tensors and into slots of a wider buffer whose other channels stay untouched."""
    B, C, H, W = shape
    x = synth.normal(40, f"sppany{shape}", shape)
    x[np.abs(x) < 0.3] = 0.0                      # many ties
    x[(x == 0) & (synth.normal(41, f"sppsign{shape}", shape) < 0)] = -0.0
    xd = dev(x, cuda)
    n = len(kernels)
    outs = [torch.empty((B, C, H, W), device=cuda) for _ in range(n)]
    ops.spp(xd, list(kernels), outs)
    wide = torch.full((B, n * C + 1, H, W), 5.0, device=cuda)          # slots start one plane in: unaligned for odd planes
    ops.spp(xd, list(kernels), [wide[:, 1 + i * C:1 + (i + 1) * C] for i in range(n)])
    assert bool((wide[:, 0] == 5.0).all())
    for i, k in enumerate(kernels):
        ref = oracle.maxpool(x, k, 1)[0]
        for got in (outs[i].cpu().numpy(), wide[:, 1 + i * C:1 + (i + 1) * C].cpu().numpy()):
            assert np.array_equal(got, ref) and np.array_equal(np.signbit(got), np.signbit(ref)), (k,)


@pytest.mark.parametrize("shape", [(1, 8, 13, 13), (2, 4, 20, 20), (1, 6, 19, 19)])
def test_spp_planes_with_nans_follow_the_scan(cuda, oracle, shape):
    """A plane that holds a NaN leaves the chain of windows and is scanned window by window, as the reference does;
    its neighbours in the same launch are not affected."""
    B, C, H, W = shape
    x = synth.normal(42, f"sppn{shape}", shape)
    x[0, 0, 0, 0] = np.nan
    x[0, 1, H // 2, W // 2] = np.nan
    x[0, 2, :, 0] = np.nan
    x[0, 3, H - 1, :] = np.nan
    x[-1, -1, 2, 3] = -np.inf
    outs = [torch.empty((B, C, H, W), device=cuda) for _ in range(3)]
    ops.spp(dev(x, cuda), [5, 9, 13], outs)
    for k, o in zip((5, 9, 13), outs):
        same(o.cpu().numpy(), oracle.maxpool(x, k, 1)[0])


@pytest.mark.parametrize("shape", [(2, 4, 16, 16), (2, 3, 13, 13), (1, 5, 38, 38), (2, 2, 19, 19), (1, 3, 5, 7)])
@pytest.mark.parametrize("stride,scale", [(2, 1.0), (2, 0.5), (3, 1.0)])
def test_upsample(cuda, oracle, shape, stride, scale):
    x = synth.normal(36, f"u{shape}", shape)
    same(ops.upsample(dev(x, cuda), stride, scale).cpu().numpy(), oracle.upsample(x, stride, scale))


def test_upsample_into_concat_slot(cuda, oracle):
    """yolov3-tiny: upsample(128x13x13) lands in the first 128 channels of the 384-channel route."""
    B, C, H, W = 2, 8, 13, 13
    x = synth.normal(37, "us", (B, C, H, W))
    other = synth.normal(38, "uo", (B, 5, 2 * H, 2 * W))
    cat = torch.zeros((B, C + 5, 2 * H, 2 * W), device=cuda)
    ops.upsample(dev(x, cuda), 2, 1.0, out=cat[:, :C])
    cat[:, C:] = dev(other, cuda)
    same(cat.cpu().numpy(), oracle.route([oracle.upsample(x, 2, 1.0), other]))


@pytest.mark.parametrize("hw", [(13, 13), (16, 16), (19, 19), (1, 1)])
def test_concat(cuda, oracle, hw):
    H, W = hw
    B = 3
    srcs = [synth.normal(39, f"c{i}{hw}", (B, c, H, W)) for i, c in enumerate([4, 1, 7, 3])]
    same(ops.concat([dev(s, cuda) for s in srcs]).cpu().numpy(), oracle.route(srcs))
    # a source that is itself a slot of a wider tensor
    wide = torch.zeros((B, 10, H, W), device=cuda)
    wide[:, 2:6] = dev(srcs[0], cuda)
    same(ops.concat([wide[:, 2:6], dev(srcs[1], cuda)]).cpu().numpy(), oracle.route(srcs[:2]))


def test_pool_and_move_argument_errors(cuda):
    x = torch.zeros((1, 1, 4, 4), device=cuda)
    with pytest.raises(capi.PxeError):
        ops.maxpool(x, 0, 1, 0)
    with pytest.raises(capi.PxeError):
        ops.maxpool(x, 9, 1, 0)           # empty output
    with pytest.raises(capi.PxeError):
        ops.upsample(x, 0)
    assert capi.lib().pxe_concat(None, 0, None, None, None, None, 0, 1, 1, 1) == capi.PXE_ERR_BAD_ARG
    torch.cuda.synchronize()


@pytest.mark.parametrize("shape", [(2, 512, 7, 7), (3, 5, 1, 1), (1, 3, 13, 40), (2, 1000, 2, 2)])
def test_avgpool(cuda, oracle, shape):
    x = synth.normal(41, f"avg{shape}", shape, 0.5, 2.0)
    ref = oracle.avgpool(x)
    close(ops.avgpool(dev(x, cuda)).cpu().numpy(), ref)
    wide = torch.zeros((shape[0], shape[1] + 3, shape[2], shape[3]), device=cuda)
    wide[:, 3:] = dev(x, cuda)
    close(ops.avgpool(wide[:, 3:]).cpu().numpy(), ref)          # a channel slot of a wider buffer


@pytest.mark.parametrize("shape", [(2, 8, 20, 20), (1, 3, 13, 13), (2, 5, 19, 19), (1, 2, 5, 40)])
@pytest.mark.parametrize("act", ["leaky", "mish", "swish", "linear"])
@pytest.mark.parametrize("use_bn", [True, False])
def test_spp_block_with_folded_epilogue(cuda, oracle, shape, act, use_bn):
    """pxe_spp_epilogue on a raw conv output == pxe_conv_epilogue followed by pxe_spp, bit for bit: the pass-through
    slot and the three pools, all as channel slots of the SPP concat buffer; and the oracle's separate layers."""
    B, C, H, W = shape
    x = synth.normal(38, f"sppe{shape}", shape)
    x[0, 0, 0, 0] = np.nan
    (g, b, m, v), dp = bn(39, f"sppebn{shape}", C, cuda)
    xd = dev(x, cuda)
    if use_bn:
        fa, fb = ops.fold_bn(C, cuda, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3])
        full = ops.conv_epilogue(dev(x, cuda), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act)
        ref_full = oracle.conv_epilogue(x, g, b, m, v, None, act)
    else:
        fa = fb = None
        full = ops.conv_epilogue(dev(x, cuda), act=act)
        ref_full = oracle.activate(act, x)
    want = torch.zeros((B, 4 * C, H, W), device=cuda)
    ops.spp(full, [13, 9, 5], [want[:, 0:C], want[:, C:2 * C], want[:, 2 * C:3 * C]])
    want[:, 3 * C:] = full
    got = torch.full((B, 4 * C + 2, H, W), 5.0, device=cuda)
    ops.spp(xd, [13, 9, 5], [got[:, 0:C], got[:, C:2 * C], got[:, 2 * C:3 * C]], a=fa, b=fb, act=act,
            y_identity=got[:, 3 * C:4 * C])
    same(got[:, :4 * C].cpu().numpy(), want.cpu().numpy())
    assert bool((got[:, 4 * C:] == 5.0).all())
    assert np.array_equal(xd.cpu().numpy()[~np.isnan(x)], x[~np.isnan(x)])          # the raw input is not modified
    close(got[:, 3 * C:4 * C].cpu().numpy(), ref_full)
    # without an identity destination only the pools are written
    got2 = torch.zeros((B, 3 * C, H, W), device=cuda)
    ops.spp(xd, [13, 9, 5], [got2[:, 0:C], got2[:, C:2 * C], got2[:, 2 * C:]], a=fa, b=fb, act=act)
    same(got2.cpu().numpy(), want[:, :3 * C].cpu().numpy())
    # a plane that does not fit shared memory is refused, not silently run another way
    big = torch.zeros((1, 1, 96, 96), device=cuda)
    with pytest.raises(Exception):
        ops.spp(big, [5], [torch.zeros_like(big)], act="leaky")
