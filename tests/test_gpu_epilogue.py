"""GPU parity: fused conv epilogue, activation, bias, shortcut vs the CPU oracle.

Tolerance for fp32 elementwise results: |gpu - ref| <= 1e-6 + 1e-5 * |ref|.
"""
import numpy as np
import pytest
import torch

from pixienn_b200 import capi, ops, synth

pytestmark = pytest.mark.gpu

ACTS = ["leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"]


def close(got, ref, rtol=1e-5, atol=1e-6):
    got = np.asarray(got, np.float32)
    ref = np.asarray(ref, np.float32)
    assert got.shape == ref.shape
    both_nan = np.isnan(got) & np.isnan(ref)
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    bad = ~((err <= atol + rtol * np.abs(ref.astype(np.float64))) | both_nan | (got == ref))
    assert not bad.any(), (f"{bad.sum()} of {bad.size} outside tolerance; worst abs err "
                           f"{np.nanmax(np.where(bad, err, 0))} at {np.argwhere(bad)[:3].tolist()}")


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def bn(seed, tag, c, cuda):
    g, b, m, v = synth.bn_params(seed, tag, c)
    return (g, b, m, v), tuple(dev(t, cuda) for t in (g, b, m, v))


# shapes exercise: plane-aligned vectors (HW%4==0), dense straddling vectors (13x13, 19x19),
# scalar path (odd base offset via channel slot), tiny planes, many planes per block
SHAPES = [(2, 8, 16, 16), (3, 5, 13, 13), (2, 7, 19, 19), (1, 3, 1, 1), (4, 33, 2, 2), (2, 6, 26, 26),
          (1, 1, 1, 7), (2, 300, 1, 1), (1, 2, 52, 52)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("act", ACTS)
def test_bn_act_matches_oracle(cuda, oracle, shape, act):
    B, C, H, W = shape
    x = synth.normal(1, f"x{shape}", shape, 0.0, 2.0)
    (g, b, m, v), dp = bn(2, f"bn{shape}", C, cuda)
    for eps_mode in (capi.EPS_CUDNN, capi.EPS_CPU):
        ref = oracle.conv_epilogue(x, g, b, m, v, None, act, 1e-5, eps_mode)
        got = ops.conv_epilogue(dev(x, cuda), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act=act,
                                eps_mode=eps_mode)
        close(got.cpu().numpy(), ref)


@pytest.mark.parametrize("shape", SHAPES[:5])
@pytest.mark.parametrize("act", ["leaky", "mish", "swish", "logistic"])
def test_bn_plus_bias_sweep_op(cuda, oracle, shape, act):
    """The sweep's op: BN inference, then a per-channel bias, then the activation."""
    B, C, H, W = shape
    x = synth.normal(3, f"x{shape}", shape)
    (g, b, m, v), dp = bn(4, f"bn{shape}", C, cuda)
    bias = synth.normal(5, f"bias{shape}", C, 0.0, 0.1)
    ref = oracle.conv_epilogue(x, g, b, m, v, bias, act)
    xd = dev(x, cuda)
    out = ops.conv_epilogue(xd, gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], bias=dev(bias, cuda), act=act,
                            in_place=False)
    close(out.cpu().numpy(), ref)
    assert np.array_equal(xd.cpu().numpy(), x), "out-of-place call must leave x untouched"


def test_bias_only_and_add_bias(cuda, oracle):
    shape = (2, 255, 19, 19)
    x = synth.normal(6, "head", shape)
    bias = synth.normal(7, "hb", 255, 0.0, 0.5)
    ref = oracle.conv_epilogue(x, bias=bias, act="linear")
    close(ops.conv_epilogue(dev(x, cuda), bias=dev(bias, cuda), act="linear").cpu().numpy(), ref)
    close(ops.add_bias(dev(x, cuda), dev(bias, cuda)).cpu().numpy(), ref)


@pytest.mark.parametrize("act", ACTS)
def test_activate_edge_values(cuda, oracle, act):
    """Whole input range incl. the +-20 softplus branches, huge, tiny, denormal, inf, nan."""
    edge = np.array([0.0, -0.0, 1.0, -2.0, 3.0, -4.0, 19.999, 20.0, 20.001, -19.999, -20.0, -20.001, 50.0, -50.0,
                     88.0, -88.0, 89.0, -104.0, 1e-30, -1e-30, 1e-42, -1e-42, 1e30, -1e30, np.inf, -np.inf, np.nan,
                     0.5, -0.5, 7.0, -7.0], np.float32)
    sweep = np.linspace(-30, 30, 4001, dtype=np.float32)
    x = np.concatenate([edge, sweep, synth.normal(8, "act", 5000, 0, 6)])
    with np.errstate(all="ignore"):
        ref = oracle.activate(act, x)
    got = ops.activate(act, dev(x, cuda)).cpu().numpy()
    close(got, ref)


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 1023, 1 << 20, (1 << 20) + 3])
def test_activate_sizes(cuda, oracle, n):
    x = synth.normal(9, f"n{n}", n)
    close(ops.activate("leaky", dev(x, cuda)).cpu().numpy(), oracle.activate("leaky", x))


def test_activate_unaligned_view(cuda, oracle):
    x = synth.normal(10, "unal", 4099)
    d = dev(x, cuda)
    ops.activate("swish", d[3:])              # 12-byte offset: scalar path
    ref = x.copy()
    ref[3:] = oracle.activate("swish", x[3:])
    close(d.cpu().numpy(), ref)


@pytest.mark.parametrize("shape", [(2, 8, 16, 16), (3, 5, 13, 13), (2, 4, 19, 19), (1, 3, 7, 5)])
@pytest.mark.parametrize("res_act", ["linear", "leaky"])
def test_conv_epilogue_with_shortcut(cuda, oracle, shape, res_act):
    """conv(BN+leaky) followed by a shortcut layer, as one pass."""
    B, C, H, W = shape
    x = synth.normal(11, f"x{shape}", shape)
    frm = synth.normal(12, f"f{shape}", shape)
    (g, b, m, v), dp = bn(13, f"bn{shape}", C, cuda)
    conv_out = oracle.conv_epilogue(x, g, b, m, v, None, "leaky")
    ref = oracle.shortcut(conv_out, frm, 1.0, 1.0, res_act)
    got = ops.conv_epilogue(dev(x, cuda), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act="leaky",
                            residual=dev(frm, cuda), res_act=res_act)
    close(got.cpu().numpy(), ref)


@pytest.mark.parametrize("shape", [(2, 8, 16, 16), (3, 5, 13, 13), (1, 3, 7, 5)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 1.0), (0.5, 2.0)])
def test_shortcut_layer(cuda, oracle, shape, alpha, beta):
    x = synth.normal(14, f"x{shape}", shape)
    frm = synth.normal(15, f"f{shape}", shape)
    ref = oracle.shortcut(x, frm, alpha, beta, "leaky")
    got = ops.shortcut(dev(x, cuda), dev(frm, cuda), alpha, beta, "leaky")
    # alpha*x + beta*from is one fused multiply-add on the GPU (as in the reference's CUDA kernel)
    # and two roundings on the CPU; identical for alpha = beta = 1
    close(got.cpu().numpy(), ref, rtol=1e-5, atol=1e-6)
    if alpha == 1.0 and beta == 1.0:
        lin = ops.shortcut(dev(x, cuda), dev(frm, cuda), 1.0, 1.0, "linear").cpu().numpy()
        assert np.array_equal(lin, oracle.shortcut(x, frm, 1.0, 1.0, "linear"))


def test_shortcut_general_mismatched_shapes(cuda, oracle):
    B, w1, h1, c1, w2, h2, c2 = 2, 8, 8, 6, 4, 4, 4       # stride 2 read of `add`
    add = synth.normal(16, "add", (B, c1, h1, w1))
    out = synth.normal(17, "out", (B, c2, h2, w2))
    ref = oracle.shortcut_raw(B, w1, h1, c1, add, w2, h2, c2, 1.0, 1.0, out)
    got = ops.shortcut_general(B, w1, h1, c1, dev(add, cuda), w2, h2, c2, 1.0, 1.0, dev(out, cuda))
    assert np.array_equal(got.cpu().numpy(), ref.reshape(out.shape))
    w1, h1, c1, w2, h2, c2 = 4, 4, 3, 8, 8, 5            # sample 2 write into `out`
    add = synth.normal(18, "add", (B, c1, h1, w1))
    out = synth.normal(19, "out", (B, c2, h2, w2))
    ref = oracle.shortcut_raw(B, w1, h1, c1, add, w2, h2, c2, 1.0, 1.0, out)
    got = ops.shortcut_general(B, w1, h1, c1, dev(add, cuda), w2, h2, c2, 1.0, 1.0, dev(out, cuda))
    assert np.array_equal(got.cpu().numpy(), ref.reshape(out.shape))


@pytest.mark.parametrize("shape,slot", [((2, 8, 16, 16), 4), ((2, 5, 13, 13), 3), ((3, 4, 26, 26), 0)])
def test_store_into_concat_slot_and_dual_store(cuda, oracle, shape, slot):
    """y2 lands in a channel slot of a wider buffer; the rest of the buffer is untouched."""
    B, C, H, W = shape
    x = synth.normal(20, f"x{shape}", shape)
    (g, b, m, v), dp = bn(21, f"bn{shape}", C, cuda)
    ref = oracle.conv_epilogue(x, g, b, m, v, None, "swish")
    wide = torch.full((B, C + 7, H, W), -7.0, device=cuda)
    y = ops.conv_epilogue(dev(x, cuda), y2=wide[:, slot:slot + C], gamma=dp[0], beta=dp[1], mean=dp[2],
                          var=dp[3], act="swish")
    close(y.cpu().numpy(), ref)
    w = wide.cpu().numpy()
    assert np.array_equal(w[:, slot:slot + C], y.cpu().numpy())
    assert (w[:, :slot] == -7.0).all() and (w[:, slot + C:] == -7.0).all()
    # reading x from a slot as well
    src = torch.zeros((B, C + 3, H, W), device=cuda)
    src[:, 2:2 + C] = dev(x, cuda)
    out = ops.conv_epilogue(src[:, 2:2 + C], gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act="swish",
                            in_place=False)
    close(out.cpu().numpy(), ref)


def test_yolo_head_activation_fused_with_bias(cuda, oracle):
    B, masks, classes, H, W = 2, 3, 4, 13, 13
    x = synth.normal(22, "yh", (B, masks * (classes + 5), H, W), 0, 2)
    bias = synth.normal(23, "yb", masks * (classes + 5), 0, 0.3)
    ref = oracle.yolo_activate(oracle.conv_epilogue(x, bias=bias, act="linear"), masks, classes)
    got = ops.conv_epilogue(dev(x, cuda), bias=dev(bias, cuda), act="yolo_head", yolo_classes=classes)
    close(got.cpu().numpy(), ref)
    close(ops.yolo_activate(dev(x, cuda), masks, classes).cpu().numpy(), oracle.yolo_activate(x, masks, classes))


def test_yolo_activate_known_answer(cuda):
    """Logistic on entries 0,1,4.., identity on 2,3 (the reference's kernel-level YOLO test values)."""
    raw = np.array([0, 0, 0, 0, 0, -1, 1], np.float32).reshape(1, 7, 1, 1)
    out = ops.yolo_activate(dev(raw, cuda), 1, 2).cpu().numpy().ravel()
    assert out[0] == 0.5 and out[1] == 0.5 and out[2] == 0.0 and out[3] == 0.0 and out[4] == 0.5
    assert abs(out[5] - 1 / (1 + np.exp(1.0))) < 1e-6 and abs(out[6] - 1 / (1 + np.exp(-1.0))) < 1e-6


def test_bad_arguments_are_rejected_before_launch(cuda):
    x = torch.zeros((1, 2, 4, 4), device=cuda)
    with pytest.raises(capi.PxeError) as e:
        ops.conv_epilogue(x, act=42)
    assert e.value.status == capi.PXE_ERR_BAD_ARG
    with pytest.raises(capi.PxeError):
        ops.conv_epilogue(x, act="yolo_head", yolo_classes=1)       # 2 channels % 6 != 0
    with pytest.raises(capi.PxeError) as e:
        ops.conv_epilogue(x, act="linear", pool=(3, 1, 2))
    assert e.value.status == capi.PXE_ERR_UNSUPPORTED
    d = capi.EpilogueDesc()
    assert capi.lib().pxe_conv_epilogue(None, None) == capi.PXE_ERR_BAD_ARG
    assert capi.lib().pxe_conv_epilogue(None, d) == capi.PXE_ERR_BAD_ARG
    assert b"null" in capi.lib().pxe_last_error_string()
    torch.cuda.synchronize()      # the context is still healthy


@pytest.mark.parametrize("shape", [(2, 8, 16, 16), (3, 5, 13, 13), (2, 4, 26, 26), (1, 7, 5, 9), (2, 3, 52, 52), (2, 36, 13, 13),
                                   (1, 2, 1, 1)])
@pytest.mark.parametrize("act", ["leaky", "mish", "linear"])
def test_folded_coefficients_give_the_same_bits(cuda, shape, act):
    """a, b folded once by pxe_fold_bn instead of gamma / beta / mean / var / bias on every launch: every form of the
    epilogue (plain, in place, with residual and a second store, both pooled variants with and without the
    full-resolution output, into channel slots) returns the same bits."""
    B, C, H, W = shape
    x = dev(synth.normal(150, f"fx{shape}", shape), cuda)
    res = dev(synth.normal(151, f"fr{shape}", shape), cuda)
    _, dp = bn(152, f"fbn{shape}", C, cuda)
    bias = dev(synth.normal(153, f"fb{shape}", C, 0, 0.1), cuda)
    raw = dict(gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], bias=bias)
    fa, fb = ops.fold_bn(C, cuda, **raw)
    fold = dict(a=fa, b=fb)

    def same(call):
        u, v = call(raw), call(fold)
        u, v = (u if isinstance(u, tuple) else (u,)), (v if isinstance(v, tuple) else (v,))
        for s, t in zip(u, v):
            if s is not None:
                assert torch.equal(s.contiguous().view(torch.int32), t.contiguous().view(torch.int32))

    same(lambda kw: ops.conv_epilogue(x.clone(), act=act, **kw))
    same(lambda kw: ops.conv_epilogue(x, y=torch.empty_like(x), y2=torch.empty_like(x), act=act, residual=res, res_act="leaky", **kw))
    wide = lambda: torch.zeros((B, C + 3, H, W), device=cuda)
    same(lambda kw: ops.conv_epilogue(x, y=wide()[:, 2:2 + C], act=act, **kw))
    for pad in (0, 1):
        if ops.maxpool_out_dim(H, 2, 2, pad) > 0 and ops.maxpool_out_dim(W, 2, 2, pad) > 0:
            for variant in (capi.POOL_AUTO, capi.POOL_GENERAL):
                same(lambda kw: ops.conv_epilogue(x, y=False, act=act, pool=(2, 2, pad), pool_variant=variant, **kw))
                if 2 * ops.maxpool_out_dim(H, 2, 2, pad) >= H and 2 * ops.maxpool_out_dim(W, 2, 2, pad) >= W:
                    same(lambda kw: ops.conv_epilogue(x, y=torch.empty_like(x), act=act, pool=(2, 2, pad), pool_variant=variant, **kw))
    # folded coefficients alone (no raw parameters in the call) and a head: the YOLO rule keeps its identity channels
    if C % 7 == 0:
        same(lambda kw: ops.conv_epilogue(x.clone(), act="yolo_head", yolo_classes=2, **kw))
