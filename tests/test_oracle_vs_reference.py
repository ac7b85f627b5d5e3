"""Checks the C restatement against the reference's own CPU code, compiled in place into
oracle/_ref/libpxref_cpu.so.  Skipped where that library was not built (no reference checkout)."""
import numpy as np
import pytest

from pixienn_b200 import synth


@pytest.fixture(scope="module")
def ref(oracle):
    r = oracle.ref_cpu()
    if r is None:
        pytest.skip("oracle/_ref/libpxref_cpu.so not built")
    return r


@pytest.mark.parametrize("kind", ["leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"])
def test_activations_bit_identical(oracle, ref, kind):
    x = np.concatenate([synth.normal(70, "a", 20000, 0, 8), np.linspace(-25, 25, 5001, dtype=np.float32),
                        np.array([0, -0.0, 20, -20, 1e-40, 90, -90], np.float32)])
    assert np.array_equal(ref.activate(kind, x), oracle.activate(kind, x))


def test_batchnorm_inference_bit_identical(oracle, ref):
    x = synth.normal(71, "x", (3, 7, 5, 9), 0, 2)
    g, b, m, v = synth.bn_params(72, "bn", 7)
    want = ref.batchnorm_inference(x, g, b, m, v)
    assert np.array_equal(ref.batchnorm_inference(x, g, b, m, v, via_vector=True), want)
    assert np.array_equal(oracle.conv_epilogue(x, g, b, m, v, None, "linear", 1e-5, 1), want)


def test_bias_scale_softmax_flatten_bit_identical(oracle, ref):
    x = synth.normal(73, "x", (2, 5, 3, 4))
    bias = synth.normal(74, "b", 5)
    assert np.array_equal(ref.add_bias(x, bias), oracle.conv_epilogue(x, bias=bias, act="linear"))
    y = x.copy()
    oracle.lib().pxo_scale_bias(y.ctypes.data_as(oracle._f), bias.ctypes.data_as(oracle._f), 2, 5, 12)
    assert np.array_equal(ref.scale_bias(x, bias), y)
    v = synth.normal(75, "s", 80, 0, 4)
    for t in (1.0, 0.5):
        assert np.array_equal(ref.softmax_one(v, t), oracle.softmax_one(v, t))
    f = x.reshape(-1)
    z = f.copy()
    oracle.lib().pxo_flatten(z.ctypes.data_as(oracle._f), 12, 5, 2, 1)
    assert np.array_equal(ref.flatten(f, 12, 5, 2, True), z)


def test_conv_forward_im2col_matches(oracle, ref):
    x = synth.uniform(76, "img", (2, 3, 9, 11))
    for (f, k, s, pad) in [(4, 3, 1, 1), (5, 3, 2, 1), (6, 1, 1, 0)]:
        w = synth.normal(77, f"w{f}{k}", (f, 3, k, k), 0, 0.3)
        got = ref.conv_forward(x, w, f, k, s, pad)
        col_ref = np.empty(3 * k * k * got.shape[2] * got.shape[3], np.float32)
        col_mine = np.empty_like(col_ref)
        ref.L.pxref_im2col(x[0].ctypes.data_as(oracle._f), 3, 9, 11, k, k, pad, pad, s, s, 1, 1, col_ref.ctypes.data_as(oracle._f))
        oracle.lib().pxo_im2col(x[0].ctypes.data_as(oracle._f), 3, 9, 11, k, k, pad, pad, s, s, 1, 1, col_mine.ctypes.data_as(oracle._f))
        assert np.array_equal(col_ref, col_mine)
        import torch
        want = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(w), stride=s, padding=pad).numpy()
        np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("kind", ["leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"])
def test_activation_gradients_bit_identical(oracle, ref, kind):
    """Activation<U, CPU>::gradient of the reference's own header against the restatement."""
    x = np.concatenate([synth.normal(73, "gx", 20000, 0, 8), np.linspace(-25, 25, 5001, dtype=np.float32),
                        np.array([0, -0.0, 20, -20, 1e-40, 90, -90], np.float32)])
    delta = synth.normal(73, "gd", len(x), 0, 3)
    assert np.array_equal(ref.gradient(kind, x, delta), oracle.gradient(kind, x, delta))


def test_backward_bias_and_constrain_bit_identical(oracle, ref):
    delta = synth.normal(74, "bd", (3, 5, 7, 9), 0, 2)
    start = synth.normal(74, "bs", 5)
    assert np.array_equal(ref.backward_bias(start, delta), oracle.backward_bias(start, delta))
    conn = synth.normal(74, "bc", (4, 11))
    assert np.array_equal(ref.backward_bias(np.zeros(11, np.float32), conn), oracle.backward_bias(np.zeros(11, np.float32), conn))
    x = synth.normal(75, "cx", 1000, 0, 5)
    assert np.array_equal(ref.constrain(x, 2.5), oracle.constrain(x, 2.5))


@pytest.mark.parametrize("shape", [(3, 5, 7, 9), (1, 4, 13, 13), (6, 2, 1, 1), (2, 3, 16, 16)])
def test_batchnorm_training_forward_and_backward_follow_the_reference(oracle, ref, shape):
    """batchNormForward(training = true) and batchNormBackward of the reference's own compiled code against the
    restatement in its CPU mode.  The reference adds in float, in index order (and through cblas_sdot); the
    restatement adds in double: agreement is to float rounding of sums over batch * spatial terms, not bit for bit."""
    B, C, H, W = shape
    x = synth.normal(76, f"bnx{shape}", shape, 0.7, 2.0)
    g, b, rm, rv = synth.bn_params(77, f"bnp{shape}", C)
    y_ref, m_ref, v_ref, rm_ref, rv_ref, xn_ref = ref.batchnorm_forward_training(x, g, b, rm, rv)
    y, rm2, rv2, sm, ss = oracle.batchnorm_forward_training(x, g, b, rm, rv, 0.01, 1e-5, 1)
    np.testing.assert_allclose(sm, m_ref, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ss, v_ref, rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(rm2, rm_ref, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(rv2, rv_ref, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(y, y_ref, rtol=1e-4, atol=1e-5)
    dy = synth.normal(78, f"bnd{shape}", shape, 0, 1.5)
    su0, bu0 = synth.normal(79, "su", C), synth.normal(79, "bu", C)
    dx_ref, su_ref, bu_ref = ref.batchnorm_backward(dy, x, xn_ref, m_ref, v_ref, g, su0, bu0)
    dx, dg, db = oracle.batchnorm_backward(x, dy, g, m_ref, v_ref, su0, bu0, 1e-5, 1)
    np.testing.assert_allclose(db, bu_ref, rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(dg, su_ref, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(dx, dx_ref, rtol=1e-4, atol=2e-5)


def test_launch_grid_of_the_compat_tier_equals_the_reference(oracle):
    """px::cudaGridsize of libpxe.so against the reference's (src/CudaUtils.cu:28-43), through the same glue built
    twice: over the reference's own sources and over libpxe.so.  Host code: no GPU is touched."""
    import ctypes as C
    theirs, ours = oracle.ref_cuda(), oracle.ref_cuda_on_pxe()
    if theirs is None or ours is None:
        pytest.skip("oracle/_ref/libpxref_cuda*.so not built")
    a, b = (C.c_uint * 3)(), (C.c_uint * 3)()
    for n in [1, 2, 511, 512, 513, 65535 * 512, 65535 * 512 + 1, 10 ** 8, 757 * 10 ** 6, 2 ** 31, 2 ** 32 - 1]:
        theirs.L.pxrefcu_gridsize(n, a)
        ours.L.pxrefcu_gridsize(n, b)
        assert list(a) == list(b), n
        assert a[0] * a[1] * 512 >= n
