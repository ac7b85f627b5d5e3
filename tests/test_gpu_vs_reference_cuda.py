"""Three-way agreement on the GPU: new kernels vs the reference's own CUDA kernels (its src/*.cu
compiled unchanged for sm_100a into oracle/_ref/libpxref_cuda.so) vs the CPU oracle.
Skipped where that library was not built (it needs a checkout of the reference at build time).

Every test also runs a second time with the same glue -- the reference's call sequences, compiled against the
reference's own headers -- linked against libpxe.so INSTEAD of the reference's .cu files
(oracle/_ref/libpxref_cuda_on_pxe.so, linked with -z defs): the link-compatible tier carrying the reference's
calls.  In that run "theirs" is this library reached through the px:: signatures."""
import numpy as np
import pytest
import torch

from pixienn_b200 import capi, ops, synth
from test_gpu_epilogue import bn, close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["reference-kernels", "glue-linked-against-libpxe"])
def refcu(oracle, request):
    r = oracle.ref_cuda() if request.param == "reference-kernels" else oracle.ref_cuda_on_pxe()
    if r is None:
        pytest.skip("oracle/_ref/libpxref_cuda*.so not built")
    r.kind = request.param
    return r


@pytest.mark.parametrize("act", ["leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"])
def test_activation_vs_reference_kernel(cuda, oracle, refcu, act):
    x = np.concatenate([synth.normal(80, "a", 200000, 0, 6), np.linspace(-25, 25, 20001, dtype=np.float32)])
    mine = ops.activate(act, dev(x, cuda))
    theirs = dev(x, cuda)
    refcu.call("activate", oracle.ACT[act], theirs.data_ptr(), theirs.numel())
    torch.cuda.synchronize()
    m, t = mine.cpu().numpy(), theirs.cpu().numpy()
    close(m, t)
    if act not in ("mish", "logistic", "swish"):        # same expressions, same math library: bit-identical
        assert np.array_equal(m, t)
    # the reference's own CUDA and CPU paths agree to the same tolerance (mish: its exp(x)+1 rounding step makes
    # the two differ by up to |x| * 2^-23 when exp() differs by an ulp, hence the wider absolute bound)
    close(t, oracle.activate(act, x), atol=2e-6 if act == "mish" else 1e-6)


@pytest.mark.parametrize("shape", [(4, 16, 26, 26), (2, 255, 19, 19), (3, 32, 13, 13)])
def test_bn_inference_vs_cudnn_call(cuda, oracle, refcu, shape):
    """cudnnBatchNormalizationForwardInference exactly as the reference's conv layer calls it."""
    B, C, H, W = shape
    x = synth.normal(81, f"x{shape}", shape, 0, 2)
    (g, b, m, v), dp = bn(82, f"bn{shape}", C, cuda)
    theirs = dev(x, cuda)
    refcu.call("batchnorm_inference", theirs.data_ptr(), *(t.data_ptr() for t in dp), B, C, H, W)
    torch.cuda.synchronize()
    mine = ops.conv_epilogue(dev(x, cuda), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act="linear")
    close(mine.cpu().numpy(), theirs.cpu().numpy())
    close(theirs.cpu().numpy(), oracle.conv_epilogue(x, g, b, m, v, None, "linear", 1e-5, 0))


def test_conv_epilogue_replay_vs_fused(cuda, oracle, refcu):
    """The reference's whole epilogue sequence (fills, cuDNN BN, preActivation copy, thrust activation)
    against the one fused pass."""
    shape = (4, 32, 52, 52)
    B, C, H, W = shape
    x = synth.normal(83, "x", shape)
    (g, b, m, v), dp = bn(84, "bn", C, cuda)
    out = dev(x, cuda)
    delta, pre, scratch = (torch.empty_like(out) for _ in range(3))
    refcu.call("conv_epilogue_replay", out.data_ptr(), delta.data_ptr(), pre.data_ptr(), scratch.data_ptr(), B, C, H, W,
               *(t.data_ptr() for t in dp), None, oracle.ACT["leaky"])
    torch.cuda.synchronize()
    mine = ops.conv_epilogue(dev(x, cuda), gamma=dp[0], beta=dp[1], mean=dp[2], var=dp[3], act="leaky")
    close(mine.cpu().numpy(), out.cpu().numpy())
    # bias branch
    bias = synth.normal(85, "b", C, 0, 0.3)
    out = dev(x, cuda)
    refcu.call("conv_epilogue_replay", out.data_ptr(), delta.data_ptr(), pre.data_ptr(), scratch.data_ptr(), B, C, H, W,
               None, None, None, None, dev(bias, cuda).data_ptr(), oracle.ACT["linear"])
    torch.cuda.synchronize()
    mine = ops.conv_epilogue(dev(x, cuda), bias=dev(bias, cuda), act="linear")
    assert np.array_equal(mine.cpu().numpy(), out.cpu().numpy())


@pytest.mark.parametrize("shape,k,s,pad", [((2, 8, 26, 26), 2, 2, 1), ((2, 8, 13, 13), 2, 1, 1), ((1, 4, 20, 20), 5, 1, 4),
                                           ((1, 4, 20, 20), 13, 1, 12), ((2, 3, 9, 11), 3, 2, 1)])
def test_maxpool_vs_reference_kernel(cuda, oracle, refcu, shape, k, s, pad):
    B, C, H, W = shape
    x = synth.normal(86, f"p{shape}{k}", shape)
    mine, idx = ops.maxpool(dev(x, cuda), k, s, pad, with_indexes=True)
    out, ridx = torch.empty_like(mine), torch.empty_like(idx)
    refcu.call("maxpool", dev(x, cuda).data_ptr(), out.data_ptr(), ridx.data_ptr(), B, C, H, W, mine.shape[2], mine.shape[3],
               k, s, pad)
    torch.cuda.synchronize()
    assert np.array_equal(mine.cpu().numpy(), out.cpu().numpy())
    assert np.array_equal(idx.cpu().numpy(), ridx.cpu().numpy())


@pytest.mark.parametrize("shape", [(16, 512, 20, 20), (8, 256, 19, 19), (8, 512, 13, 13)])
def test_spp_block_at_model_size_equals_the_reference_kernel(cuda, refcu, shape):
    """The SPP block of YOLOv7-640 at its configured 16 images per GPU (and the 19x19 / 13x13 planes of the 608 / 416
    presets): every value of the three pools equals what the reference's own maxPoolForwardGpu writes, bit for bit,
    with ties (a quarter of the values are zeros of both signs) and the -infinity planes included."""
    B, C, H, W = shape
    x = synth.normal(88, f"sppfull{shape}", shape)
    x[np.abs(x) < 0.3] = 0.0
    x[(x == 0) & (synth.normal(89, f"sppfs{shape}", shape) < 0)] = -0.0
    x[0, 1] = -np.inf
    xd = dev(x, cuda)
    cat = torch.empty((B, 3 * C, H, W), device=cuda)
    ops.spp(xd, [5, 9, 13], [cat[:, 0:C], cat[:, C:2 * C], cat[:, 2 * C:]])
    ridx = torch.empty((B, C, H, W), device=cuda, dtype=torch.int32)
    ref = torch.empty((B, C, H, W), device=cuda)
    for i, k in enumerate((5, 9, 13)):
        refcu.call("maxpool", xd.data_ptr(), ref.data_ptr(), ridx.data_ptr(), B, C, H, W, H, W, k, 1, k - 1)
        torch.cuda.synchronize()
        got = cat[:, i * C:(i + 1) * C]
        assert torch.equal(got.contiguous().view(torch.int32), ref.view(torch.int32)), k      # bit patterns: -0 and +0 differ
    # one pool alone goes through the same kernel
    alone = ops.maxpool(xd, 13, 1)
    assert torch.equal(alone.view(torch.int32), ref.view(torch.int32))


def test_kernel2_stride1_pool_at_model_size_equals_the_reference_kernel(cuda, refcu):
    """YOLOv3-tiny-416, layer 11 at 64 images: values and argmax planes, bit for bit."""
    B, C, H, W = 64, 512, 13, 13
    x = synth.normal(90, "k2s1full", (B, C, H, W))
    x[np.abs(x) < 0.3] = 0.0
    xd = dev(x, cuda)
    mine, idx = ops.maxpool(xd, 2, 1, 1, with_indexes=True)
    out, ridx = torch.empty_like(mine), torch.empty_like(idx)
    refcu.call("maxpool", xd.data_ptr(), out.data_ptr(), ridx.data_ptr(), B, C, H, W, H, W, 2, 1, 1)
    torch.cuda.synchronize()
    assert torch.equal(mine.view(torch.int32), out.view(torch.int32)) and torch.equal(idx, ridx)
    assert torch.equal(ops.maxpool(xd, 2, 1, 1).view(torch.int32), out.view(torch.int32))


def test_upsample_shortcut_heads_vs_reference_kernels(cuda, oracle, refcu):
    B, C, H, W = 2, 6, 13, 13
    x = synth.normal(87, "u", (B, C, H, W))
    out = torch.zeros((B, C, 2 * H, 2 * W), device=cuda)
    refcu.call("upsample", dev(x, cuda).data_ptr(), W, H, C, B, 2, 0.5, out.data_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(ops.upsample(dev(x, cuda), 2, 0.5).cpu().numpy(), out.cpu().numpy())

    frm = synth.normal(88, "f", (B, C, H, W))
    theirs = dev(x, cuda)
    refcu.call("shortcut", B, W, H, C, dev(frm, cuda).data_ptr(), W, H, C, 0.5, 2.0, theirs.data_ptr())
    torch.cuda.synchronize()
    mine = ops.shortcut(dev(x, cuda), dev(frm, cuda), 0.5, 2.0, "linear")
    close(mine.cpu().numpy(), theirs.cpu().numpy())       # both contract s1*out + s2*add to one fused multiply-add

    classes = 7
    head = synth.normal(89, "h", (B, 3 * (classes + 5), H, W), 0, 3)
    theirs = torch.empty((B, 3 * (classes + 5), H, W), device=cuda)
    refcu.call("yolo_activate", dev(head, cuda).data_ptr(), theirs.data_ptr(), B, 3, classes, H * W)
    torch.cuda.synchronize()
    assert np.array_equal(ops.yolo_activate(dev(head, cuda), 3, classes).cpu().numpy(), theirs.cpu().numpy())

    cn = synth.normal(90, "c", (B, classes + 4, H, W), -2, 2)
    theirs = torch.empty((B, classes + 4, H, W), device=cuda)
    refcu.call("centernet_activate", dev(cn, cuda).data_ptr(), theirs.data_ptr(), B, classes, H * W, -2.19)
    torch.cuda.synchronize()
    assert np.array_equal(ops.centernet_activate(dev(cn, cuda), classes, -2.19).cpu().numpy(), theirs.cpu().numpy())


def test_centernet_topk_indices_bit_exact_vs_reference_cuda_scores(cuda, oracle, refcu):
    """Scores from the reference's CUDA activation kernel, decode of them by the host reference logic
    (the oracle) vs the device decode from logits: same sigmoid expression, so the kept indices and
    their order are bit-exact."""
    from test_gpu_heads import centernet_case
    B, classes, H, W, K = 3, 8, 64, 96, 40
    heat, size, off = centernet_case(91, B, classes, H, W)
    full = np.concatenate([heat, size, off], 1)
    act = torch.empty((B, classes + 4, H, W), device=cuda)
    refcu.call("centernet_activate", dev(full, cuda).data_ptr(), act.data_ptr(), B, classes, H * W, -1.0)
    torch.cuda.synchronize()
    a = act.cpu().numpy()
    ref, _ = oracle.centernet_decode(np.ascontiguousarray(a[:, :classes]), size, off, 0.2, K)
    fd = dev(full, cuda)
    d, c = ops.centernet_decode(fd[:, :classes], fd[:, classes:classes + 2], fd[:, classes + 2:], 0.2, K, logits=True,
                                heatmap_bias=-1.0)
    got = ops.centernet_to_host(d, c)
    for b in range(B):
        assert np.array_equal(got[b]["source"], ref[b]["source"])
        assert np.array_equal(got[b]["prob"], ref[b]["prob"])


# ------------------------------------------------------------------ the backward-side functions
@pytest.mark.parametrize("act", ["leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"])
def test_activation_gradient_three_way(cuda, oracle, refcu, act):
    x = np.concatenate([synth.normal(92, "gx", 100003, 0, 6), np.linspace(-25, 25, 20001, dtype=np.float32)])
    delta = synth.normal(92, "gd", len(x), 0, 2)
    mine = ops.activation_gradient(act, dev(x, cuda), dev(delta, cuda))
    theirs = dev(delta, cuda)
    refcu.call("gradient", oracle.ACT[act], dev(x, cuda).data_ptr(), len(x), theirs.data_ptr())
    torch.cuda.synchronize()
    m, t = mine.cpu().numpy(), theirs.cpu().numpy()
    close(m, t, atol=2e-6)
    if act in ("leaky", "linear", "relu", "loggy"):      # no transcendental: bit-identical
        assert np.array_equal(m, t)
    close(t, oracle.gradient(act, x, delta), atol=4e-6)
    # odd sizes and unaligned starts take the scalar path
    xs, ds = dev(x, cuda)[1:1001], dev(delta, cuda)[1:1001].clone()
    close(ops.activation_gradient(act, xs.contiguous(), ds).cpu().numpy(), oracle.gradient(act, x[1:1001], delta[1:1001]), atol=4e-6)


@pytest.mark.parametrize("shape", [(4, 16, 26, 26), (2, 255, 19, 19), (3, 7, 1, 1), (5, 300, 1, 1), (2, 3, 50, 70),
                                   (8, 16, 104, 104), (8, 16, 51, 53), (2048, 100, 1, 1)])   # the last three: clusters of 8, 2, 8 blocks
def test_backward_bias_three_way(cuda, oracle, refcu, shape):
    """Sums of up to tens of thousands of terms: the reference's kernel, this library's and the CPU loop add in
    different orders; they agree to the rounding of such a sum."""
    delta = synth.normal(93, f"bb{shape}", shape, 0, 1)
    start = synth.normal(93, f"bs{shape}", shape[1])
    mine = ops.backward_bias(dev(start, cuda), dev(delta, cuda))
    again = ops.backward_bias(dev(start, cuda), dev(delta, cuda))
    theirs = dev(start, cuda)
    refcu.call("backward_bias", theirs.data_ptr(), dev(delta, cuda).data_ptr(), shape[0], shape[1], shape[2] * shape[3])
    torch.cuda.synchronize()
    assert torch.equal(mine, again)                        # fixed summation order: the same bits every time
    terms = shape[0] * shape[2] * shape[3]
    tol = 1e-6 * np.sqrt(terms) * 4 + 1e-6
    want = oracle.backward_bias(start, delta)
    assert np.abs(mine.cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())
    assert np.abs(theirs.cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("k,stride", [(2, 2), (2, 1), (5, 1), (3, 2)])
def test_maxpool_backward_three_way(cuda, oracle, refcu, k, stride):
    B, C, H, W = 2, 5, 13, 17
    x = synth.normal(94, "mpx", (B, C, H, W))
    out, idx = ops.maxpool(dev(x, cuda), k, stride, with_indexes=True)
    delta = synth.normal(94, "mpd", tuple(out.shape))
    grad0 = synth.normal(94, "mpg", (B, C, H, W))
    mine = ops.maxpool_backward(dev(delta, cuda), idx, dev(grad0, cuda))
    theirs = dev(grad0, cuda)
    refcu.call("maxpool_backward", dev(delta, cuda).data_ptr(), idx.data_ptr(), theirs.data_ptr(), delta.size)
    torch.cuda.synchronize()
    want = oracle.maxpool_backward(delta, idx.cpu().numpy(), grad0)
    if stride >= k:                                        # no input is named twice: exact
        assert np.array_equal(mine.cpu().numpy(), want) and np.array_equal(theirs.cpu().numpy(), want)
    else:                                                  # several adds per input, in any order
        close(mine.cpu().numpy(), want, atol=2e-6)
        close(theirs.cpu().numpy(), want, atol=2e-6)


@pytest.mark.parametrize("stride,scale", [(2, 1.0), (3, 0.5), (1, 2.0)])
def test_upsample_backward_three_way(cuda, oracle, refcu, stride, scale):
    B, C, H, W = 2, 3, 7, 9
    out = synth.normal(95, "ubo", (B, C, H * stride, W * stride))
    acc0 = synth.normal(95, "uba", (B, C, H, W))
    mine = ops.upsample_backward(dev(acc0, cuda), dev(out, cuda), stride, scale)
    theirs = dev(acc0, cuda)
    refcu.call("upsample_backward", W, H, C, B, stride, scale, theirs.data_ptr(), dev(out, cuda).data_ptr())
    torch.cuda.synchronize()
    want = oracle.upsample_backward(acc0, out, stride, scale)
    close(mine.cpu().numpy(), want, atol=2e-6)
    close(theirs.cpu().numpy(), want, atol=2e-6)


def test_constrain_mul_three_way(cuda, oracle, refcu):
    x = synth.normal(96, "cx", 100001, 0, 4)
    y = synth.normal(96, "cy", 100001, 0, 4)
    mine = ops.constrain(dev(x, cuda), 1.5)
    theirs = dev(x, cuda)
    refcu.call("constrain", len(x), 1.5, theirs.data_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(mine.cpu().numpy(), theirs.cpu().numpy())
    assert np.array_equal(mine.cpu().numpy(), oracle.constrain(x, 1.5))
    my = ops.mul(dev(x, cuda), dev(y, cuda))
    ty = dev(y, cuda)
    refcu.call("mul", len(x), dev(x, cuda).data_ptr(), ty.data_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(my.cpu().numpy(), ty.cpu().numpy()) and np.array_equal(my.cpu().numpy(), x * y)
    # tensors that start 4 bytes past a 16-byte boundary take the element-wise form of the kernels
    ux, uy = dev(x, cuda)[1:], dev(y, cuda)[1:]
    assert ux.data_ptr() % 16 == 4
    assert np.array_equal(ops.constrain(ux, 1.5).cpu().numpy(), oracle.constrain(x[1:], 1.5))
    ux = dev(x, cuda)[1:]
    assert np.array_equal(ops.mul(ux, uy).cpu().numpy(), x[1:] * y[1:])


@pytest.mark.parametrize("t", [1, 2, 10, 1000])
def test_adam_step_three_way(cuda, oracle, refcu, t):
    """px::adamGpu: bit-identical to the reference's kernel (same expressions, same device math library); the oracle's
    host powf / sqrtf may differ in the last place."""
    n = 100003
    x, m = synth.normal(97, "ax", n, 0, 1), synth.normal(97, "am", n, 0, 0.1)
    v = np.abs(synth.normal(97, "av", n, 0, 0.01)).astype(np.float32)
    args = (0.9, 0.999, -1e-3, 1e-8, t)
    mine = ops.adam_update(dev(x, cuda), dev(m, cuda), dev(v, cuda), *args)
    theirs, dm, dv = dev(x, cuda), dev(m, cuda), dev(v, cuda)          # named: the pointers must outlive the call
    refcu.call("adam", n, theirs.data_ptr(), dm.data_ptr(), dv.data_ptr(), *args)
    torch.cuda.synchronize()
    assert np.array_equal(mine.cpu().numpy(), theirs.cpu().numpy())
    np.testing.assert_allclose(mine.cpu().numpy(), oracle.adam(x, m, v, *args), rtol=2e-6, atol=1e-7)
    # off a 16-byte boundary (the element-wise form): the same values
    again = ops.adam_update(dev(x, cuda)[1:], dev(m, cuda)[1:], dev(v, cuda)[1:], *args)
    assert np.array_equal(again.cpu().numpy(), mine.cpu().numpy()[1:])


def test_softmax_cross_entropy_equals_the_restatement(cuda, oracle):
    """px::softmaxCrossEntropy.  The reference's src/SoftmaxKernel.cu cannot be compiled here (its header pulls in
    OpenCV through GroundTruth.h), so this one is two-way: the kernel against the restatement of its two lines."""
    n = 64 * 1000
    logits = synth.normal(98, "sl", (64, 1000), 0, 3)
    pred = np.exp(logits - logits.max(1, keepdims=True))
    pred = (pred / pred.sum(1, keepdims=True)).astype(np.float32).ravel()
    pred[:3] = [0.0, 1.0, 1e-12]
    truth = np.zeros(n, np.float32)
    truth[np.arange(64) * 1000 + (np.arange(64) * 37) % 1000] = 1.0
    truth[:3] = 1.0
    delta, error = ops.softmax_cross_entropy(dev(pred, cuda), dev(truth, cuda))
    d_ref, e_ref = oracle.softmax_cross_entropy(pred, truth)
    assert np.array_equal(delta.cpu().numpy(), d_ref)
    np.testing.assert_allclose(error.cpu().numpy(), e_ref, rtol=1e-6, atol=1e-7)
    assert float(error[0]) == pytest.approx(-np.log(np.float32(1e-9)), rel=1e-6) and float(error[1]) == 0.0


def test_random_fills_follow_the_reference_engine(cuda, refcu):
    """Element i comes from the minimal-standard generator advanced i steps: uniform values equal the reference's
    (thrust) to the last bit or the one before; normal values have the requested moments and, value by value, sit
    where the reference's inversion of the same engine position puts them, to the accuracy of the two erf^-1."""
    n = 200000
    mine = ops.random_uniform(torch.empty(n, device=cuda), -0.25, 0.75).cpu().numpy()
    theirs = torch.empty(n, device=cuda)
    refcu.call("random", theirs.data_ptr(), n, -0.25, 0.75)
    torch.cuda.synchronize()
    t = theirs.cpu().numpy()
    assert mine.min() >= -0.25 and mine.max() < 0.75
    assert np.abs(mine - t).max() <= 1.2e-7
    print(f"\nuniform fill: {np.mean(mine == t) * 100:.2f} % of {n} values bit-identical to the reference ({refcu.kind})")
    mn = ops.random_normal(torch.empty(n, device=cuda), 1.0, 2.0).cpu().numpy()
    tn = torch.empty(n, device=cuda)
    refcu.call("random_normal", tn.data_ptr(), n, 1.0, 2.0)
    torch.cuda.synchronize()
    tn = tn.cpu().numpy()
    assert abs(mn.mean() - 1.0) < 0.02 and abs(mn.std() - 2.0) < 0.02
    assert abs(tn.mean() - 1.0) < 0.02 and abs(tn.std() - 2.0) < 0.02
    print(f"normal fill: max |mine - reference| = {np.abs(mn - tn).max():.3e}, correlation {np.corrcoef(mn, tn)[0, 1]:.6f}")


# ------------------------------------------------------------------ detector losses
def yolo_loss_case(seed, B=3, masks=(3, 4, 5), classes=5, H=13, W=13, max_truth=8):
    rng = np.random.default_rng(seed)
    mc = len(masks)
    raw = synth.normal(seed, "yl", (B, mc * (classes + 5), H, W), 0, 1.0)
    out = raw.reshape(B, mc, classes + 5, H, W).copy()
    sig = lambda v: (1.0 / (1.0 + np.exp(-v.astype(np.float64)))).astype(np.float32)
    out[:, :, :2] = sig(out[:, :, :2]); out[:, :, 4:] = sig(out[:, :, 4:]); out[:, :, 2:4] *= 0.3
    out = np.ascontiguousarray(out.reshape(B, -1, H, W))
    truths = np.zeros((B, max_truth, 5), np.float32)
    counts = np.array([3, 0, 7][:B], np.int32)
    for b in range(B):
        for t in range(counts[b]):
            truths[b, t] = [rng.uniform(0.1, 0.9), rng.uniform(0.1, 0.9), rng.uniform(0.05, 0.5), rng.uniform(0.05, 0.5),
                            rng.integers(classes)]
    slots = B * mc * H * W
    a_cls = np.full(slots, -1, np.int32)
    a_anc = np.zeros(slots, np.int32)
    a_box = np.zeros((slots, 4), np.float32)
    for s_ in rng.choice(slots, 25, replace=False):
        a_cls[s_] = rng.integers(classes)
        a_anc[s_] = rng.integers(6)
        a_box[s_] = [rng.uniform(0.1, 0.9), rng.uniform(0.1, 0.9), rng.uniform(0.05, 0.5), rng.uniform(0.05, 0.5)]
    anchors = np.array([10, 14, 23, 27, 37, 58, 81, 82, 135, 169, 344, 319], np.float32)
    return out, truths, counts, a_cls, a_anc, a_box, np.array(masks, np.int32), anchors


@pytest.mark.parametrize("prior", ["cleared", "kept"])
def test_yolo_loss_three_way(cuda, oracle, refcu, prior):
    """One launch here against the reference's four (region, object, squared norm, components): every delta value
    identical, the twelve statistics and the cost equal to the rounding of their float sums.  `kept`: delta holds
    values the loss does not decide, which must survive and count in the cost."""
    out, truths, counts, a_cls, a_anc, a_box, masks, anchors = yolo_loss_case(97)
    delta0 = np.zeros_like(out) if prior == "cleared" else synth.normal(97, "ylp", out.shape, 0, 0.05)
    kw = dict(ignore_thr=0.5, truth_thr=0.3, coord_scale=1.5, object_scale=5.0, no_object_scale=0.7, class_scale=1.2)
    want_delta, want_stats, want_cost = oracle.yolo_loss(out, delta0, truths, counts, a_cls, a_anc, a_box, masks, anchors,
                                                         416, 416, **kw)
    ti = lambda a: torch.from_numpy(a).to(cuda)
    args = [ti(out), None, ti(truths), ti(counts), ti(a_cls), ti(a_anc), ti(a_box), ti(masks), ti(anchors)]
    mine_d, mine_s, mine_c = ti(delta0), torch.zeros(12, device=cuda), torch.zeros(1, device=cuda)
    ops.yolo_loss(args[0], mine_d, *args[2:], mine_s, mine_c, 416, 416, **kw)
    ref_d, ref_s, ref_c = ti(delta0), torch.zeros(12, device=cuda), torch.zeros(1, device=cuda)
    B, ch, H, W = out.shape
    refcu.call("yolo_loss", args[0].data_ptr(), ref_d.data_ptr(), args[2].data_ptr(), args[3].data_ptr(), args[4].data_ptr(),
               args[5].data_ptr(), args[6].data_ptr(), args[7].data_ptr(), args[8].data_ptr(), ref_s.data_ptr(),
               ref_c.data_ptr(), None, truths.shape[1], B, len(masks), 6, ch // len(masks) - 5, W, H, 416, 416,
               kw["ignore_thr"], kw["truth_thr"], kw["coord_scale"], kw["object_scale"], kw["no_object_scale"], kw["class_scale"])
    torch.cuda.synchronize()
    if capi.lib().pxe_debug_bounds_checked():              # the bounds-checked build: the compiler contracts some
        close(mine_d.cpu().numpy(), ref_d.cpu().numpy(), atol=2e-6)      # multiply-adds differently (last-bit differences)
    else:
        assert torch.equal(mine_d, ref_d)                  # the same expressions: identical deltas
    close(mine_d.cpu().numpy(), want_delta, atol=2e-6)
    assert np.count_nonzero(want_delta != delta0) > 500
    for got in (mine_s.cpu().numpy(), ref_s.cpu().numpy()):
        np.testing.assert_allclose(got, want_stats, rtol=2e-5, atol=1e-5)
    assert want_stats[6] == 25 and want_stats[0] > 0
    for got in (float(mine_c.item()), float(ref_c.item())):
        assert abs(got - want_cost) <= 2e-5 * want_cost


def test_centernet_loss_three_way(cuda, oracle, refcu):
    B, classes, H, W = 3, 4, 16, 24
    rng = np.random.default_rng(98)
    out = synth.uniform(98, "clo", (B, classes + 4, H, W))
    out[:, :classes] = np.clip(out[:, :classes], 1e-5, 1 - 1e-5)
    heat = (synth.uniform(98, "clh", (B, classes, H, W)) ** 4).astype(np.float32)
    mask = np.zeros((B, H, W), np.float32)
    for _ in range(20):
        b, c, y, x = rng.integers(B), rng.integers(classes), rng.integers(H), rng.integers(W)
        heat[b, c, y, x] = 1.0
        mask[b, y, x] = 1.0
    tsize = synth.uniform(98, "cls", (B, 2, H, W)) * 5
    toff = synth.uniform(98, "clf", (B, 2, H, W))
    delta0 = np.zeros_like(out)
    want_delta, want_costs = oracle.centernet_loss(out, delta0, heat, tsize, toff, mask, 1.0 / 20, 2.0, 4.0, 0.1)
    ti = lambda a: torch.from_numpy(a).to(cuda)
    t = [ti(a) for a in (out, heat, tsize, toff, mask)]
    mine_d, mine_c = ti(delta0), torch.zeros(3, device=cuda)
    ops.centernet_loss(t[0], mine_d, t[1], t[2], t[3], t[4], mine_c, 1.0 / 20, 2.0, 4.0, 0.1)
    ref_d, ref_c = ti(delta0), torch.zeros(3, device=cuda)
    refcu.call("centernet_loss", t[0].data_ptr(), ref_d.data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(),
               t[4].data_ptr(), ref_c.data_ptr(), B, classes, H * W, 1.0 / 20, 2.0, 4.0, 0.1)
    torch.cuda.synchronize()
    assert torch.equal(mine_d, ref_d)
    close(mine_d.cpu().numpy(), want_delta, rtol=2e-5, atol=2e-6)     # powf / logf: CUDA's and glibc's differ by ulps
    for got in (mine_c.cpu().numpy(), ref_c.cpu().numpy()):
        np.testing.assert_allclose(got, want_costs, rtol=2e-5)
    assert want_costs.min() > 0
