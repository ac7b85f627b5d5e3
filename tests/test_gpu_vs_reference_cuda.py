"""Three-way agreement on the GPU: new kernels vs the reference's own CUDA kernels (its src/*.cu
compiled unchanged for sm_100a into oracle/_ref/libpxref_cuda.so) vs the CPU oracle.
Skipped where that library was not built (it needs a checkout of the reference at build time)."""
import numpy as np
import pytest
import torch

from pixienn_b200 import ops, synth
from test_gpu_epilogue import bn, close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refcu(oracle):
    r = oracle.ref_cuda()
    if r is None:
        pytest.skip("oracle/_ref/libpxref_cuda.so not built")
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
