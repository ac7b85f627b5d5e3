/*
 * ref_cpu_glue.cpp -- extern "C" doorway into the reference's own CPU code.
 *
 * TEST INFRASTRUCTURE ONLY.  Compiled together with the reference's unmodified
 * src/CpuUtil.cpp, src/BatchNorm.cpp, src/Math.cpp, src/Error.cpp and
 * include/Activation.h (read in place from the reference tree, never copied)
 * into oracle/_ref/libpxref_cpu.so.  Used to validate the C restatement in
 * px_oracle.c and as the timed CPU baseline.  Nothing here computes anything:
 * each function only forwards to the reference function named in its comment.
 */
#include <cstddef>
#include <algorithm>

#include <cblas.h>

#include "Activation.h"
#include "BatchNorm.h"
#include "CpuUtil.h"
#include "Math.h"

#define API extern "C" __attribute__((visibility("default")))

using namespace px;

/* Activation<U, CPU>::apply(T*, T*), include/Activation.h:292-298 */
API int pxref_activate(int type, float* x, std::size_t n)
{
    switch (type) {
    case LEAKY:    { Activation<Leaky> a;    a.apply(x, x + n); return 0; }
    case LINEAR:   { Activation<Linear> a;   a.apply(x, x + n); return 0; }
    case LOGGY:    { Activation<Loggy> a;    a.apply(x, x + n); return 0; }
    case LOGISTIC: { Activation<Logistic> a; a.apply(x, x + n); return 0; }
    case MISH:     { Activation<Mish> a;     a.apply(x, x + n); return 0; }
    case RELU:     { Activation<ReLU> a;     a.apply(x, x + n); return 0; }
    case SOFTPLUS: { Activation<Softplus> a; a.apply(x, x + n); return 0; }
    case SWISH:    { Activation<Swish> a;    a.apply(x, x + n); return 0; }
    case TANH:     { Activation<Tanh> a;     a.apply(x, x + n); return 0; }
    default: return 1;
    }
}

/* addBias, src/CpuUtil.cpp:178 */
/* Activation<U, CPU>::gradient(T* dbegin, T* dend, const T* x), include/Activation.h:306-316 */
API int pxref_gradient(int type, const float* x, std::size_t n, float* delta)
{
    switch (static_cast<ActivationType>(type)) {
    case LEAKY:    { Activation<Leaky> a;    a.gradient(delta, delta + n, x); return 0; }
    case LINEAR:   { Activation<Linear> a;   a.gradient(delta, delta + n, x); return 0; }
    case LOGGY:    { Activation<Loggy> a;    a.gradient(delta, delta + n, x); return 0; }
    case LOGISTIC: { Activation<Logistic> a; a.gradient(delta, delta + n, x); return 0; }
    case MISH:     { Activation<Mish> a;     a.gradient(delta, delta + n, x); return 0; }
    case RELU:     { Activation<ReLU> a;     a.gradient(delta, delta + n, x); return 0; }
    case SOFTPLUS: { Activation<Softplus> a; a.gradient(delta, delta + n, x); return 0; }
    case SWISH:    { Activation<Swish> a;    a.gradient(delta, delta + n, x); return 0; }
    case TANH:     { Activation<Tanh> a;     a.gradient(delta, delta + n, x); return 0; }
    }
    return 1;
}

/* backwardBias, src/CpuUtil.cpp:189-196; constrain, :357-362 */
API void pxref_backward_bias(float* biasUpdates, const float* delta, int batch, int n, int size)
{
    backwardBias(biasUpdates, delta, batch, n, size);
}

API void pxref_constrain(int n, float alpha, float* x)
{
    constrain(n, alpha, x, 1);
}

API void pxref_add_bias(float* out, const float* bias, int batch, int n, int size)
{
    addBias(out, bias, batch, n, size);
}

/* scaleBias, src/CpuUtil.cpp:293 */
API void pxref_scale_bias(float* out, const float* scales, int batch, int n, int size)
{
    scaleBias(out, scales, batch, n, size);
}

/* normalizeCpu, src/CpuUtil.cpp:282 */
API void pxref_normalize(float* x, const float* mean, const float* var, int batch, int filters, int spatial)
{
    normalizeCpu(x, mean, var, batch, filters, spatial);
}

/* Inference branch of batchNormForward, src/BatchNorm.cpp:61-66, on raw pointers. */
API void pxref_batchnorm_inference(float* x, const float* gamma, const float* beta, const float* mean,
                                   const float* var, int batch, int channels, int spatial)
{
    normalizeCpu(x, mean, var, batch, channels, spatial);
    scaleBias(x, gamma, batch, channels, spatial);
    addBias(x, beta, batch, channels, spatial);
}

/* batchNormForward itself (inference), through the PxCpuVector interface. */
API void pxref_batchnorm_forward_vec(float* x, const float* gamma, const float* beta, const float* mean,
                                     const float* var, int batch, int channels, int height, int width)
{
    const std::size_t n = static_cast<std::size_t>(batch) * channels * height * width;
    PxCpuVector io(n), m(channels), v(channels), rm(channels), rv(channels), s(channels), b(channels), xs, xn;
    std::copy(x, x + n, io.begin());
    std::copy(mean, mean + channels, rm.begin());
    std::copy(var, var + channels, rv.begin());
    std::copy(gamma, gamma + channels, s.begin());
    std::copy(beta, beta + channels, b.begin());
    batchNormForward(false, batch, channels, height, width, io, io, m, v, rm, rv, s, b, xs, xn);
    std::copy(io.begin(), io.end(), x);
}

/* batchNormForward(training = true), src/BatchNorm.cpp:24-67, through the PxCpuVector interface.  io: x in, y out;
 * mean / var receive the batch statistics, rolling_mean / rolling_var are updated, xnorm receives the normalised
 * tensor the backward pass wants. */
API void pxref_batchnorm_forward_training(float* io, const float* gamma, const float* beta, float* mean, float* var,
                                          float* rolling_mean, float* rolling_var, float* xnorm, int batch,
                                          int channels, int height, int width)
{
    const std::size_t n = static_cast<std::size_t>(batch) * channels * height * width;
    PxCpuVector v(n), m(channels), va(channels), rm(channels), rv(channels), s(channels), b(channels), xs(n), xn(n);
    std::copy(io, io + n, v.begin());
    std::copy(rolling_mean, rolling_mean + channels, rm.begin());
    std::copy(rolling_var, rolling_var + channels, rv.begin());
    std::copy(gamma, gamma + channels, s.begin());
    std::copy(beta, beta + channels, b.begin());
    batchNormForward(true, batch, channels, height, width, v, v, m, va, rm, rv, s, b, xs, xn);
    std::copy(v.begin(), v.end(), io);
    std::copy(m.begin(), m.end(), mean);
    std::copy(va.begin(), va.end(), var);
    std::copy(rm.begin(), rm.end(), rolling_mean);
    std::copy(rv.begin(), rv.end(), rolling_var);
    std::copy(xn.begin(), xn.end(), xnorm);
}

/* batchNormBackward, src/BatchNorm.cpp:68-98.  delta: dy in, dx out; scale_updates / bias_updates are added to. */
API void pxref_batchnorm_backward(float* delta, const float* x, const float* xnorm, const float* mean, const float* var,
                                  const float* gamma, float* scale_updates, float* bias_updates, int batch,
                                  int channels, int height, int width)
{
    const std::size_t n = static_cast<std::size_t>(batch) * channels * height * width;
    PxCpuVector d(n), m(channels), va(channels), md(channels), vd(channels), s(channels), su(channels), bu(channels),
        xs(n), xn(n);
    std::copy(delta, delta + n, d.begin());
    std::copy(x, x + n, xs.begin());
    std::copy(xnorm, xnorm + n, xn.begin());
    std::copy(mean, mean + channels, m.begin());
    std::copy(var, var + channels, va.begin());
    std::copy(gamma, gamma + channels, s.begin());
    std::copy(scale_updates, scale_updates + channels, su.begin());
    std::copy(bias_updates, bias_updates + channels, bu.begin());
    batchNormBackward(batch, channels, height, width, d, m, va, md, vd, s, su, bu, xs, xn);
    std::copy(d.begin(), d.end(), delta);
    std::copy(su.begin(), su.end(), scale_updates);
    std::copy(bu.begin(), bu.end(), bias_updates);
}

/* softmax(const float*, int, float, float*, int), src/Math.cpp:77 */
API void pxref_softmax_one(const float* in, int n, float temp, float* out, int stride)
{
    softmax(in, n, temp, out, stride);
}

/* softmax batched/grouped, src/Math.cpp:99 */
API void pxref_softmax(const float* in, int n, int batch, int batchOffset, int groups, int groupOffset,
                       int stride, float temp, float* out)
{
    softmax(in, n, batch, batchOffset, groups, groupOffset, stride, temp, out);
}

/* sigmoid(float), src/Math.cpp:121 */
API float pxref_sigmoid(float x) { return sigmoid(x); }

/* flatten, src/CpuUtil.cpp:364 */
API void pxref_flatten(float* x, int size, int layers, int batch, int forward)
{
    flatten(x, size, layers, batch, forward != 0);
}

/* im2ColCpuExt, src/CpuUtil.cpp:74 */
API void pxref_im2col(const float* im, int channels, int height, int width, int kh, int kw, int ph, int pw,
                      int sh, int sw, int dh, int dw, float* col)
{
    im2ColCpuExt(im, channels, height, width, kh, kw, ph, pw, sh, sw, dh, dw, col);
}

/*
 * The conv GEMM loop of ConvLayer<CPU>::forward (include/ConvLayer.h:203-225)
 * for groups == 1: the reference's im2ColCpuExt and the same cblas_sgemm call.
 * The loop itself lives in a header that needs yaml-cpp/OpenCV/Boost to
 * compile, so it is restated here around the reference's two calls.
 */
API void pxref_conv_forward(const float* in, const float* weights, float* out, float* column, int batch,
                            int channels, int height, int width, int filters, int kernel, int stride,
                            int pad, int dilation)
{
    const int eff = dilation * (kernel - 1) + 1;
    const int oh = (height + 2 * pad - eff) / stride + 1;
    const int ow = (width + 2 * pad - eff) / stride + 1;
    const int m = filters, n = oh * ow, k = kernel * kernel * channels;
    for (int i = 0; i < batch; ++i) {
        const float* im = in + static_cast<std::size_t>(i) * channels * height * width;
        im2ColCpuExt(im, channels, height, width, kernel, kernel, pad, pad, stride, stride, dilation, dilation,
                     column);
        cblas_sgemm(CblasRowMajor, CblasNoTrans, CblasNoTrans, m, n, k, 1.0f, weights, k, column, n, 0.0f,
                    out + static_cast<std::size_t>(i) * m * n, n);
    }
}
