/*
 * px_oracle.c -- CPU restatement of PixieNN's per-layer epilogue path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against; it is never linked into, imported by or called from the
 * shipped library.  Every function restates the behaviour of the reference's
 * CPU code and cites the file:line (relative to the trieck/pixienn tree) it
 * follows.  Plain C, single threaded, no dependencies beyond libm.
 *
 * Parity pin: the known-answer cases of the reference's own unit tests
 * (activations, maxpool, addBias/scaleBias, softmax/sigmoid, YOLO activate,
 * CenterNet decode, NMS) are re-derived in tests/test_oracle_golden.py, and
 * where the reference's CPU sources compile stand-alone (CpuUtil.cpp,
 * BatchNorm.cpp, Math.cpp, Activation.h) this file is cross-checked against
 * that compiled code in tests/test_oracle_vs_reference.py.
 */
#include <float.h>
#include <limits.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PXO_API __attribute__((visibility("default")))

/* ActivationType values: include/ActivationTypes.h:19-30 */
enum {
    PXO_LEAKY = 0, PXO_LINEAR, PXO_LOGGY, PXO_LOGISTIC, PXO_MISH,
    PXO_RELU, PXO_SOFTPLUS, PXO_SWISH, PXO_TANH
};

typedef struct {
    float x, y, w, h;      /* cv::Rect2f: left, top, width, height */
    float prob;
    int32_t class_id;
    int32_t batch_id;
    int32_t source;        /* flat slot index that emitted the record */
} pxo_detection;

/* ------------------------------------------------------------------ */
/* Activations: include/Activation.h:40-228                            */
/* ------------------------------------------------------------------ */

/* Softplus with the +-20 thresholds, include/Activation.h:111-119 */
static float softplus_ref(float x)
{
    const float threshold = 20.0f;
    if (x > threshold) return x;
    if (x < -threshold) return expf(x);
    return logf(expf(x) + 1.0f);
}

PXO_API float pxo_activate_one(int type, float x)
{
    switch (type) {
    case PXO_LEAKY:    return x > 0.0f ? x : 0.1f * x;             /* :50-53  */
    case PXO_LINEAR:   return x;                                   /* :68-71  */
    case PXO_LOGGY:    return 2.0f / (1.0f + expf(-x)) - 1.0f;     /* :85-88  */
    case PXO_LOGISTIC: return 1.0f / (1.0f + expf(-x));            /* :102-105 */
    case PXO_SOFTPLUS: return softplus_ref(x);
    case PXO_MISH:     return x * tanhf(softplus_ref(x));          /* :151-157 */
    case PXO_RELU:     return x > 0.0f ? x : 0.0f;                 /* :178-181 */
    case PXO_SWISH:    return x / (1.0f + expf(-1.0f * x));        /* :198-201 */
    case PXO_TANH:     return tanhf(x);                            /* :219-222 */
    default:           return NAN;
    }
}

/* Activation<U,CPU>::apply, include/Activation.h:292-304 (std::for_each). */
PXO_API void pxo_activate(int type, float* x, size_t n)
{
    for (size_t i = 0; i < n; ++i) x[i] = pxo_activate_one(type, x[i]);
}

/* The gradient() members of the same functors, include/Activation.h:54-228. */
static float softplus_gradient_ref(float x)
{
    if (x > 20.0f) return 1.0f;                     /* :120-129 */
    if (x < -20.0f) return expf(x);
    return 1.0f / (1.0f + expf(-x));
}

PXO_API float pxo_gradient_one(int type, float x)
{
    switch (type) {
    case PXO_LEAKY:    return x > 0.0f ? 1.0f : 0.1f;
    case PXO_LINEAR:   return 1.0f;
    case PXO_LOGGY:    { float y = (x + 1.0f) / 2.0f; return 2.0f * (1 - y) * y; }
    case PXO_LOGISTIC: { float y = 1.0f / (1.0f + expf(-x)); return y * (1.0f - y); }
    case PXO_SOFTPLUS: return softplus_gradient_ref(x);
    case PXO_MISH: {
        float sp = softplus_ref(x), grad_sp = softplus_gradient_ref(x);
        float tsp = tanhf(sp);
        float grad_tsp = (1 - tsp * tsp) * grad_sp;
        return x * grad_tsp + tsp;
    }
    case PXO_RELU:     return x > 0.0f ? 1.0f : 0.0f;
    case PXO_SWISH:    { float val = 1 / (1 + expf(-1.0f * x)); return x * val + 1.0f * val * (1 - x * val); }
    case PXO_TANH:     { float y = tanhf(x); return 1.0f - y * y; }
    default:           return NAN;
    }
}

/* Activation<U,CPU>::gradient(dbegin, dend, x), include/Activation.h:306-316: delta *= gradient(x). */
PXO_API void pxo_gradient(int type, const float* x, size_t n, float* delta)
{
    for (size_t i = 0; i < n; ++i) delta[i] *= pxo_gradient_one(type, x[i]);
}

/* backwardBias, src/CpuUtil.cpp:189-196 (sumArray adds left to right, :208-215). */
PXO_API void pxo_backward_bias(float* bias_updates, const float* delta, int batch, int n, int size)
{
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < n; ++i) {
            const float* a = delta + (size_t)size * (i + (size_t)b * n);
            float sum = 0.0f;
            for (int j = 0; j < size; ++j) sum += a[j];
            bias_updates[i] += sum;
        }
}

/* Batch normalisation with batch statistics.
 * eps_mode 1 follows batchNormForward(training = true), src/BatchNorm.cpp:44-67: meanCpu / varianceCpu
 * (src/CpuUtil.cpp:248-280: population variance), rolling = 0.99 * rolling + 0.01 * batch value (:52-56, here with the
 * factor as an argument), normalizeCpu (:282-293: (x - mean) / (sqrt(var) + eps)), scaleBias, addBias; save_scale
 * receives the variance.  eps_mode 0 is cudnnBatchNormalizationForwardTraining in spatial mode as documented by
 * cuDNN, which is what the CUDA layers call (include/cuda/ConvLayer.h:285-292): (x - mean) / sqrt(var + eps), the
 * saved value is 1 / sqrt(var + eps), and the running variance is fed var * n / (n - 1).  Sums in double. */
PXO_API void pxo_batchnorm_forward_training(const float* x, float* y, int batch, int channels, int spatial,
                                            const float* gamma, const float* beta, float* running_mean,
                                            float* running_var, float factor, float eps, int eps_mode,
                                            float* save_mean, float* save_scale)
{
    const double n = (double)batch * spatial;
    for (int c = 0; c < channels; ++c) {
        double s = 0.0;
        for (int b = 0; b < batch; ++b)
            for (int k = 0; k < spatial; ++k) s += x[((size_t)b * channels + c) * spatial + k];
        const float mean = (float)(s / n);
        double v = 0.0;
        for (int b = 0; b < batch; ++b)
            for (int k = 0; k < spatial; ++k) {
                const double d = (double)x[((size_t)b * channels + c) * spatial + k] - (double)mean;
                v += d * d;
            }
        const float var = (float)(v / n);
        float inv, fed;
        if (eps_mode == 1) { inv = 1.0f / (sqrtf(var) + eps); fed = var; save_scale[c] = var; }
        else { inv = 1.0f / sqrtf(var + eps); fed = n > 1.0 ? (float)(v / n * n / (n - 1.0)) : var; save_scale[c] = inv; }
        save_mean[c] = mean;
        if (running_mean) running_mean[c] = (1.0f - factor) * running_mean[c] + factor * mean;
        if (running_var) running_var[c] = (1.0f - factor) * running_var[c] + factor * fed;
        for (int b = 0; b < batch; ++b)
            for (int k = 0; k < spatial; ++k) {
                const size_t i = ((size_t)b * channels + c) * spatial + k;
                y[i] = gamma[c] * ((x[i] - mean) * inv) + beta[c];
            }
    }
}

/* batchNormBackward, src/BatchNorm.cpp:68-98 (eps_mode 1): biasUpdates += sum delta; scaleUpdates += sum delta * xNorm
 * with xNorm = (x - mean) / (sqrt(var) + eps); delta *= scale; meanDelta, varianceDelta, normalizeDelta of
 * src/CpuUtil.cpp:303-343, which use 1 / sqrt(var + eps).  eps_mode 0 is cudnnBatchNormalizationBackward as documented
 * by cuDNN (include/cuda/ConvLayer.h:327-332): the same sums with xhat = (x - mean) * saved inverse std,
 * dx = gamma * invstd / n * (n * dy - sum dy - xhat * sum dy * xhat).  Sums in double. */
PXO_API void pxo_batchnorm_backward(const float* x, const float* dy, float* dx, int batch, int channels, int spatial,
                                    const float* gamma, float* dgamma, float* dbeta, const float* save_mean,
                                    const float* save_scale, float eps, int eps_mode)
{
    const double n = (double)batch * spatial;
    for (int c = 0; c < channels; ++c) {
        const float mean = save_mean[c];
        float inv_fwd, inv_bwd;
        if (eps_mode == 1) { inv_fwd = 1.0f / (sqrtf(save_scale[c]) + eps); inv_bwd = 1.0f / sqrtf(save_scale[c] + eps); }
        else inv_fwd = inv_bwd = save_scale[c];
        double s1 = 0.0, s2 = 0.0;
        for (int b = 0; b < batch; ++b)
            for (int k = 0; k < spatial; ++k) {
                const size_t i = ((size_t)b * channels + c) * spatial + k;
                s1 += dy[i];
                s2 += (double)dy[i] * ((double)x[i] - (double)mean);
            }
        if (dbeta) dbeta[c] += (float)s1;
        if (dgamma) dgamma[c] += (float)(s2 * inv_fwd);
        const double g = gamma[c];
        const double mean_delta = -g * s1 * inv_bwd;
        const double var_delta = -0.5 * g * s2 * (double)inv_bwd * inv_bwd * inv_bwd;
        for (int b = 0; b < batch; ++b)
            for (int k = 0; k < spatial; ++k) {
                const size_t i = ((size_t)b * channels + c) * spatial + k;
                dx[i] = (float)(g * dy[i] * inv_bwd + var_delta * 2.0 * ((double)x[i] - mean) / n + mean_delta / n);
            }
    }
}

/* adamKernel, src/Adam.cu:26-38. */
PXO_API void pxo_adam(size_t n, float* x, const float* m, const float* v, float beta1, float beta2, float rate, float eps, int t)
{
    const float c1 = 1.0f - powf(beta1, (float)t), c2 = 1.0f - powf(beta2, (float)t);
    for (size_t i = 0; i < n; ++i) {
        const float mhat = m[i] / c1, vhat = v[i] / c2;
        x[i] += rate * mhat / (sqrtf(vhat) + eps);
    }
}

/* softmaxCrossEntropyKernel, src/SoftmaxKernel.cu:25-39. */
PXO_API void pxo_softmax_cross_entropy(size_t n, const float* pred, const float* truth, float* delta, float* error)
{
    for (size_t i = 0; i < n; ++i) {
        error[i] = truth[i] ? -logf(pred[i] + 1e-9f) : 0.0f;
        delta[i] = truth[i] - pred[i];
    }
}

/* MaxPoolLayer::backward, include/MaxPoolLayer.h:138-158. */
PXO_API void pxo_maxpool_backward(const float* delta, const int* indexes, float* grad, size_t size)
{
    for (size_t i = 0; i < size; ++i)
        if (indexes[i] >= 0) grad[indexes[i]] += delta[i];
}

/* UpsampleLayer::upsample with forward == false, include/UpsampleLayer.h:97-121: acc[in] += scale * out[o],
 * outputs visited in row-major order. */
PXO_API void pxo_upsample_backward(float* acc, const float* out, int batch, int c, int h, int w, int stride, float scale)
{
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k)
            for (int j = 0; j < h * stride; ++j)
                for (int i = 0; i < w * stride; ++i) {
                    size_t ii = (size_t)b * w * h * c + (size_t)k * w * h + (size_t)(j / stride) * w + i / stride;
                    size_t oi = (size_t)b * w * h * c * stride * stride + (size_t)k * w * h * stride * stride
                                + (size_t)j * w * stride + i;
                    acc[ii] += scale * out[oi];
                }
}

/* constrain(n, alpha, x, 1), src/CpuUtil.cpp:344-362. */
PXO_API void pxo_constrain(float* x, size_t n, float alpha)
{
    for (size_t i = 0; i < n; ++i) x[i] = fminf(alpha, fmaxf(-alpha, x[i]));
}

/* ------------------------------------------------------------------ */
/* Bias / batch-norm inference: src/CpuUtil.cpp, src/BatchNorm.cpp     */
/* ------------------------------------------------------------------ */

/* addBias, src/CpuUtil.cpp:178-187 */
PXO_API void pxo_add_bias(float* out, const float* bias, int batch, int n, int size)
{
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < size; ++j)
                out[((size_t)b * n + i) * size + j] += bias[i];
}

/* scaleBias, src/CpuUtil.cpp:293-300 (cblas_sscal per channel row == x *= s) */
PXO_API void pxo_scale_bias(float* out, const float* scales, int batch, int n, int size)
{
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < size; ++j)
                out[((size_t)b * n + i) * size + j] *= scales[i];
}

/*
 * normalizeCpu, src/CpuUtil.cpp:282-291.  eps_mode 1 is the CPU form
 * (x-mean)/(sqrt(var)+eps).  The reference calls the unqualified C `sqrt`, so
 * the denominator and the division are evaluated in double and the quotient is
 * rounded to float on the store; that is reproduced here.  eps_mode 0 is the
 * form the CUDA path gets from cudnnBatchNormalizationForwardInference,
 * (x-mean)/sqrt(var+eps) in fp32 (include/cuda/ConvLayer.h:294-299, epsilon = 1e-5).
 */
PXO_API void pxo_normalize(float* x, const float* mean, const float* var, int batch,
                           int filters, int spatial, float eps, int eps_mode)
{
    for (int b = 0; b < batch; ++b)
        for (int f = 0; f < filters; ++f) {
            double denom_cpu = sqrt((double)var[f]) + (double)eps;
            float denom_cudnn = sqrtf(var[f] + eps);
            for (int i = 0; i < spatial; ++i) {
                size_t idx = ((size_t)b * filters + f) * spatial + i;
                float centred = x[idx] - mean[f];
                x[idx] = eps_mode ? (float)((double)centred / denom_cpu) : centred / denom_cudnn;
            }
        }
}

/*
 * Conv epilogue, CPU order of operations: ConvLayer<CPU>::forward
 * include/ConvLayer.h:227-236 -> batchNormForward (src/BatchNorm.cpp:61-66:
 * normalize, scaleBias, addBias) or addBias alone, then the activation.
 * gamma == NULL means "no batch norm" (bias only).  bias2 is an additional
 * per-channel bias added after BN (NULL to skip); the reference has either
 * beta or a bias, the sweep configuration applies both.
 */
PXO_API void pxo_conv_epilogue(float* x, int batch, int channels, int spatial,
                               const float* gamma, const float* beta, const float* mean,
                               const float* var, float eps, int eps_mode,
                               const float* bias2, int act)
{
    if (gamma) {
        pxo_normalize(x, mean, var, batch, channels, spatial, eps, eps_mode);
        pxo_scale_bias(x, gamma, batch, channels, spatial);
        pxo_add_bias(x, beta, batch, channels, spatial);
    }
    if (bias2) pxo_add_bias(x, bias2, batch, channels, spatial);
    pxo_activate(act, x, (size_t)batch * channels * spatial);
}

/* ------------------------------------------------------------------ */
/* MaxPool: include/MaxPoolLayer.h:51-71 (geometry), :88-135 (forward) */
/* ------------------------------------------------------------------ */

PXO_API int pxo_maxpool_out_dim(int in, int kernel, int stride, int padding)
{
    return (in + padding - kernel) / stride + 1;   /* MaxPoolLayer.h:61-62 */
}

PXO_API void pxo_maxpool(const float* in, float* out, int* idx, int batch, int c,
                         int ih, int iw, int kernel, int stride, int padding)
{
    const int oh = pxo_maxpool_out_dim(ih, kernel, stride, padding);
    const int ow = pxo_maxpool_out_dim(iw, kernel, stride, padding);
    const int off = -padding / 2;                  /* C truncation, :92-93 */
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k)
            for (int i = 0; i < oh; ++i)
                for (int j = 0; j < ow; ++j) {
                    float best = -FLT_MAX;
                    int best_idx = -1;
                    for (int n = 0; n < kernel; ++n)
                        for (int m = 0; m < kernel; ++m) {
                            int cur_h = off + i * stride + n;
                            int cur_w = off + j * stride + m;
                            if (cur_h < 0 || cur_h >= ih || cur_w < 0 || cur_w >= iw) continue;
                            int index = cur_w + iw * (cur_h + ih * (k + c * b));
                            float v = in[index];
                            if (best_idx < 0 || v > best) { best_idx = index; best = v; }
                        }
                    size_t o = (size_t)j + (size_t)ow * (i + (size_t)oh * (k + (size_t)c * b));
                    out[o] = best;
                    if (idx) idx[o] = best_idx;
                }
}

/* ------------------------------------------------------------------ */
/* Upsample: include/UpsampleLayer.h:97-121 (forward branch)           */
/* ------------------------------------------------------------------ */
PXO_API void pxo_upsample(const float* in, float* out, int batch, int c, int h, int w,
                          int stride, float scale)
{
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k)
            for (int j = 0; j < h * stride; ++j)
                for (int i = 0; i < w * stride; ++i) {
                    size_t ii = (size_t)b * w * h * c + (size_t)k * w * h + (size_t)(j / stride) * w + i / stride;
                    size_t oi = (size_t)b * w * h * c * stride * stride + (size_t)k * w * h * stride * stride
                                + (size_t)j * w * stride + i;
                    out[oi] = scale * in[ii];
                }
}

/* ------------------------------------------------------------------ */
/* Shortcut: include/ShortcutLayer.h:113-141.  The two products and    */
/* the sum are rounded separately (no fused multiply-add).             */
/* ------------------------------------------------------------------ */
PXO_API void pxo_shortcut(int batch, int w1, int h1, int c1, const float* add,
                          int w2, int h2, int c2, float s1, float s2, float* out)
{
    int stride = w1 / w2; if (stride < 1) stride = 1;
    int sample = w2 / w1; if (sample < 1) sample = 1;
    int minw = w1 < w2 ? w1 : w2, minh = h1 < h2 ? h1 : h2, minc = c1 < c2 ? c1 : c2;
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < minc; ++k)
            for (int j = 0; j < minh; ++j)
                for (int i = 0; i < minw; ++i) {
                    size_t oi = (size_t)i * sample + (size_t)w2 * (j * sample + (size_t)h2 * (k + (size_t)c2 * b));
                    size_t ai = (size_t)i * stride + (size_t)w1 * (j * stride + (size_t)h1 * (k + (size_t)c1 * b));
                    volatile float p = s1 * out[oi];
                    volatile float q = s2 * add[ai];
                    out[oi] = p + q;
                }
}

/* ------------------------------------------------------------------ */
/* Route: include/RouteLayer.h:91-113 (per source, per image slab)     */
/* ------------------------------------------------------------------ */
PXO_API void pxo_route(int n_src, const float* const* src, const int* src_outputs,
                       int batch, float* out)
{
    size_t outputs = 0;
    for (int s = 0; s < n_src; ++s) outputs += (size_t)src_outputs[s];
    size_t offset = 0;
    for (int s = 0; s < n_src; ++s) {
        for (int b = 0; b < batch; ++b)
            memcpy(out + (size_t)b * outputs + offset, src[s] + (size_t)b * src_outputs[s],
                   (size_t)src_outputs[s] * sizeof(float));
        offset += (size_t)src_outputs[s];
    }
}

/* ------------------------------------------------------------------ */
/* YOLO head: include/YoloLayer.h:164-196 (activate), :637-698 decode  */
/* ------------------------------------------------------------------ */

/* entryIndex, include/YoloLayer.h:730-739 */
static size_t yolo_entry(int batch, int location, int entry, int area, int classes, size_t outputs)
{
    int n = location / area, loc = location % area;
    return (size_t)batch * outputs + (size_t)n * area * (4 + classes + 1) + (size_t)entry * area + loc;
}

PXO_API void pxo_yolo_activate(const float* in, float* out, int batch, int masks,
                               int classes, int area)
{
    size_t outputs = (size_t)area * masks * (classes + 5);
    if (out != in) memcpy(out, in, (size_t)batch * outputs * sizeof(float));
    for (int b = 0; b < batch; ++b)
        for (int n = 0; n < masks; ++n) {
            float* p = out + yolo_entry(b, n * area, 0, area, classes, outputs);
            for (int i = 0; i < 2 * area; ++i) p[i] = 1.0f / (1.0f + expf(-p[i]));
            p = out + yolo_entry(b, n * area, 4, area, classes, outputs);
            for (int i = 0; i < (1 + classes) * area; ++i) p[i] = 1.0f / (1.0f + expf(-p[i]));
        }
}

/* float -> int as x86-64 cvttss2si does it (the reference's host decode):
 * truncation, INT_MIN for NaN or out-of-range values. */
static int f2i_x86(float v)
{
    if (!(v > -2147483904.0f && v < 2147483648.0f)) return INT_MIN;
    return (int)v;
}

/*
 * YoloLayer::addDetects for one image, include/YoloLayer.h:659-698.
 * img_w/img_h > 0 selects scaledYoloBox (:601-635), otherwise yoloBox().rect()
 * (:637-651, src/DarkBox.cpp:84-123).  anchors are ints (YoloLayer.h:93).
 * Appends to dets[*count ...]; records beyond cap are counted but not stored.
 */
PXO_API void pxo_yolo_decode_image(const float* pred, int b, int masks, const int* mask,
                                   const int* anchors, int classes, int lw, int lh,
                                   int net_w, int net_h, int img_w, int img_h, float thr,
                                   pxo_detection* dets, long long cap, long long* count)
{
    const int area = lw * lh > 1 ? lw * lh : 1;
    const size_t outputs = (size_t)area * masks * (classes + 5);
    const int scaled = img_w > 0 && img_h > 0;
    for (int i = 0; i < area; ++i) {
        int row = i / lw, col = i % lw;
        for (int n = 0; n < masks; ++n) {
            float obj = pred[yolo_entry(b, n * area + i, 4, area, classes, outputs)];
            if (obj < thr) continue;
            size_t bi = yolo_entry(b, n * area + i, 0, area, classes, outputs);
            float bx, by, bw, bh;
            int a = mask[n];
            if (scaled) {
                int new_w, new_h;
                if (((float)net_w / img_w) < ((float)net_h / img_h)) {
                    new_w = net_w; new_h = (img_h * net_w) / img_w;
                } else {
                    new_h = net_h; new_w = (img_w * net_h) / img_h;
                }
                float x = (col + pred[bi]) / lw;
                x = (x - (net_w - new_w) / 2.0f / net_w) / ((float)new_w / net_w);
                float y = (row + pred[bi + area]) / lh;
                y = (y - (net_h - new_h) / 2.0f / net_h) / ((float)new_h / net_h);
                float width = expf(pred[bi + 2 * (size_t)area]) * anchors[2 * a] / net_w;
                width *= (float)net_w / new_w;
                float height = expf(pred[bi + 3 * (size_t)area]) * anchors[2 * a + 1] / net_h;
                height *= (float)net_h / new_h;
                int left = f2i_x86((x - width / 2) * img_w);    if (left < 0) left = 0;
                int right = f2i_x86((x + width / 2) * img_w);   if (right > img_w - 1) right = img_w - 1;
                int top = f2i_x86((y - height / 2) * img_h);    if (top < 0) top = 0;
                int bottom = f2i_x86((y + height / 2) * img_h); if (bottom > img_h - 1) bottom = img_h - 1;
                bx = (float)left; by = (float)top;
                bw = (float)(right - left); bh = (float)(bottom - top);
            } else {
                float x = (col + pred[bi]) / lw;
                float y = (row + pred[bi + area]) / lh;
                float w = expf(pred[bi + 2 * (size_t)area]) * anchors[2 * a] / net_w;
                float h = expf(pred[bi + 3 * (size_t)area]) * anchors[2 * a + 1] / net_h;
                bx = w > 0.0f ? x - w / 2.0f : x;    /* DarkBox::left,  DarkBox.cpp:84-91 */
                by = h > 0.0f ? y - h / 2.0f : y;    /* DarkBox::top,   DarkBox.cpp:102-109 */
                bw = w; bh = h;
            }
            for (int j = 0; j < classes; ++j) {
                float p = obj * pred[yolo_entry(b, n * area + i, 5 + j, area, classes, outputs)];
                if (p >= thr) {
                    if (*count < cap) {
                        pxo_detection* d = dets + *count;
                        d->x = bx; d->y = by; d->w = bw; d->h = bh; d->prob = p;
                        d->class_id = j; d->batch_id = b; d->source = i * masks + n;
                    }
                    ++*count;
                }
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* YOLOv1 detection head: DetectLayer::addDetects for one image,       */
/* include/DetectLayer.h:166-209.  predictions = that image's values:  */
/* [locations*classes scores][locations*num scales][locations*num*coords boxes]. */
/* ------------------------------------------------------------------ */
PXO_API void pxo_detect_decode_image(const float* predictions, int b, int side, int num, int classes,
                                     int coords, int squared, int width, int height, float thr,
                                     pxo_detection* dets, long long cap, long long* count)
{
    const int locations = side * side;
    for (int i = 0; i < locations; ++i) {
        int row = i / side, col = i % side;
        for (int n = 0; n < num; ++n) {
            int pindex = locations * classes + i * num + n;
            float scale = predictions[pindex];
            if (!isfinite(scale) || scale <= 0.0f) continue;
            int bindex = locations * (classes + num) + (i * num + n) * coords;
            float x = (predictions[bindex + 0] + col) / side * width;
            float y = (predictions[bindex + 1] + row) / side * height;
            float w = powf(predictions[bindex + 2], squared ? 2.0f : 1.0f) * width;
            float h = powf(predictions[bindex + 3], squared ? 2.0f : 1.0f) * height;
            int max_class = 0;
            float max_prob = -FLT_MAX;
            for (int j = 0; j < classes; ++j) {
                float prob = scale * predictions[i * classes + j];
                if (prob > max_prob) { max_class = j; max_prob = prob; }
            }
            if (max_prob >= thr) {
                if (*count < cap) {
                    pxo_detection* d = dets + *count;
                    d->x = w > 0.0f ? x - w / 2.0f : x;    /* DarkBox::left,  DarkBox.cpp:84-91 */
                    d->y = h > 0.0f ? y - h / 2.0f : y;    /* DarkBox::top,   DarkBox.cpp:102-109 */
                    d->w = w; d->h = h; d->prob = max_prob;
                    d->class_id = max_class; d->batch_id = b; d->source = i * num + n;
                }
                ++*count;
            }
        }
    }
}

/* AvgPoolLayer::forward, include/AvgPoolLayer.h:66-87: running float sum in index order, then one division. */
PXO_API void pxo_avgpool(const float* in, float* out, int batch, int channels, int area)
{
    if (area < 1) area = 1;
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < channels; ++k) {
            int oi = k + b * channels;
            out[oi] = 0.0f;
            for (int i = 0; i < area; ++i) out[oi] += in[i + (size_t)area * (k + (size_t)b * channels)];
            out[oi] /= area;
        }
}

/* ------------------------------------------------------------------ */
/* CenterNet head: include/CenterNetLayer.h:85-110, 181-247            */
/* ------------------------------------------------------------------ */
PXO_API void pxo_centernet_activate(const float* in, float* out, int batch, int classes,
                                    int area, float heatmap_bias)
{
    size_t outputs = (size_t)(classes + 4) * area;
    size_t heat = (size_t)classes * area;
    if (out != in) memcpy(out, in, (size_t)batch * outputs * sizeof(float));
    for (int b = 0; b < batch; ++b) {
        float* p = out + (size_t)b * outputs;
        for (size_t i = 0; i < heat; ++i) p[i] += heatmap_bias;
        for (size_t i = 0; i < heat; ++i) p[i] = 1.0f / (1.0f + expf(-p[i]));
    }
}

static int cn_local_max(const float* heat, int cls, int x, int y, int w, int h)
{
    const size_t area = (size_t)w * h;
    const float v = heat[cls * area + (size_t)y * w + x];
    int y0 = y - 1 > 0 ? y - 1 : 0, y1 = y + 1 < h - 1 ? y + 1 : h - 1;
    int x0 = x - 1 > 0 ? x - 1 : 0, x1 = x + 1 < w - 1 ? x + 1 : w - 1;
    for (int yy = y0; yy <= y1; ++yy)
        for (int xx = x0; xx <= x1; ++xx)
            if ((xx != x || yy != y) && heat[cls * area + (size_t)yy * w + xx] > v) return 0;
    return 1;
}

typedef struct { pxo_detection d; } cn_cand;

static int cn_cmp_desc_stable(const void* a, const void* b)
{
    const pxo_detection* p = (const pxo_detection*)a;
    const pxo_detection* q = (const pxo_detection*)b;
    if (p->prob > q->prob) return -1;
    if (p->prob < q->prob) return 1;
    /* std::stable_sort keeps emission order == ascending flat index */
    return (p->source > q->source) - (p->source < q->source);
}

/*
 * CenterNetLayer::addDetects for one image (include/CenterNetLayer.h:196-247).
 * heat/size/off point at this image's activated heatmap [classes,H,W], size
 * [2,H,W] and offset [2,H,W] planes.  Writes at most max_det records sorted by
 * score descending (ties: lower flat index (class*H+y)*W+x first) and returns
 * the number written; *n_candidates receives the count before truncation.
 */
PXO_API int pxo_centernet_decode_image(const float* heat, const float* size, const float* off,
                                       int b, int classes, int w, int h, int img_w, int img_h,
                                       float thr, int max_det, pxo_detection* out,
                                       int* n_candidates)
{
    const size_t area = (size_t)w * h;
    const float image_w = img_w > 0 ? (float)img_w : 1.0f;
    const float image_h = img_h > 0 ? (float)img_h : 1.0f;
    size_t cap = 1024, n = 0;
    pxo_detection* cand = (pxo_detection*)malloc(cap * sizeof(*cand));
    for (int c = 0; c < classes; ++c)
        for (int y = 0; y < h; ++y)
            for (int x = 0; x < w; ++x) {
                size_t index = (size_t)y * w + x;
                float score = heat[c * area + index];
                if (!isfinite(score) || score < thr || !cn_local_max(heat, c, x, y, w, h)) continue;
                float bw = size[index] / w;
                float bh = size[area + index] / h;
                float ox = off[index], oy = off[area + index];
                if (!isfinite(bw) || !isfinite(bh) || !isfinite(ox) || !isfinite(oy)
                    || bw <= 0.0f || bh <= 0.0f) continue;
                float cx = (x + ox) / w, cy = (y + oy) / h;
                if (n == cap) { cap *= 2; cand = (pxo_detection*)realloc(cand, cap * sizeof(*cand)); }
                pxo_detection* d = cand + n++;
                d->x = (cx - bw / 2.0f) * image_w;
                d->y = (cy - bh / 2.0f) * image_h;
                d->w = bw * image_w;
                d->h = bh * image_h;
                d->prob = score; d->class_id = c; d->batch_id = b;
                d->source = (int32_t)(c * area + index);
            }
    qsort(cand, n, sizeof(*cand), cn_cmp_desc_stable);
    if (n_candidates) *n_candidates = (int)n;
    int keep = n > (size_t)max_det ? max_det : (int)n;
    memcpy(out, cand, (size_t)keep * sizeof(*cand));
    free(cand);
    return keep;
}

/* ------------------------------------------------------------------ */
/* Softmax: src/Math.cpp:77-108, include/SoftmaxLayer.h:86-99          */
/* ------------------------------------------------------------------ */
PXO_API void pxo_softmax_one(const float* in, int n, float temp, float* out, int stride)
{
    float sum = 0.0f, largest = -FLT_MAX;
    for (int i = 0; i < n; ++i) if (in[i * stride] > largest) largest = in[i * stride];
    for (int i = 0; i < n; ++i) {
        float e = expf(in[i * stride] / temp - largest / temp);
        sum += e;
        out[i * stride] = e;
    }
    for (int i = 0; i < n; ++i) out[i * stride] /= sum;
}

PXO_API void pxo_softmax(const float* in, int n, int batch, int batch_offset, int groups,
                         int group_offset, int stride, float temp, float* out)
{
    for (int b = 0; b < batch; ++b)
        for (int g = 0; g < groups; ++g)
            pxo_softmax_one(in + (size_t)b * batch_offset + (size_t)g * group_offset, n, temp,
                            out + (size_t)b * batch_offset + (size_t)g * group_offset, stride);
}

/* SoftmaxLayer::addDetects, include/SoftmaxLayer.h:182-196: first maximum. */
PXO_API int pxo_softmax_detect(const float* pred, int classes, int b, int width, int height,
                               float thr, pxo_detection* out)
{
    int best = 0;
    for (int i = 1; i < classes; ++i) if (pred[best] < pred[i]) best = i;
    if (pred[best] >= thr) {
        out->x = 0; out->y = 0; out->w = (float)width; out->h = (float)height;
        out->prob = pred[best]; out->class_id = best; out->batch_id = b; out->source = best;
        return 1;
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* Region head: include/RegionLayer.h:271-300, 355-395;                */
/* flatten: src/CpuUtil.cpp:364-384                                    */
/* ------------------------------------------------------------------ */
PXO_API void pxo_flatten(float* x, int size, int layers, int batch, int forward)
{
    size_t total = (size_t)size * layers * batch;
    float* swap = (float*)calloc(total, sizeof(float));
    for (int b = 0; b < batch; ++b)
        for (int c = 0; c < layers; ++c)
            for (int i = 0; i < size; ++i) {
                size_t i1 = (size_t)b * layers * size + (size_t)c * size + i;
                size_t i2 = (size_t)b * layers * size + (size_t)i * layers + c;
                if (forward) swap[i2] = x[i1]; else swap[i1] = x[i2];
            }
    memcpy(x, swap, total * sizeof(float));
    free(swap);
}

PXO_API void pxo_region_forward(const float* in, float* out, int batch, int w, int h, int num,
                                int coords, int classes, int use_softmax)
{
    const int size = coords + 1 + classes;
    const size_t outputs = (size_t)w * h * num * size;
    if (out != in) memcpy(out, in, (size_t)batch * outputs * sizeof(float));
    pxo_flatten(out, w * h, size * num, batch, 1);
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < h * w * num; ++i) {
            size_t index = (size_t)i * size + (size_t)b * outputs;
            out[index + 4] = 1.0f / (1.0f + expf(-out[index + 4]));
            if (use_softmax)
                pxo_softmax_one(out + index + coords + 1, classes, 1.0f, out + index + coords + 1, 1);
        }
}

/*
 * RegionLayer::addDetects for one image, include/RegionLayer.h:355-395 with
 * lightBox (src/DarkBox.cpp:191-202).  The reference indexes predictions
 * WITHOUT the batch offset (RegionLayer.h:363-369), i.e. every image decodes
 * image 0's slots; that quirk is kept: pred is the start of the whole tensor.
 * biases are the float anchors.
 */
PXO_API void pxo_region_decode_image(const float* pred, int b, int w, int h, int num, int coords,
                                     int classes, const float* biases, int img_w, int img_h,
                                     float thr, pxo_detection* dets, long long cap,
                                     long long* count)
{
    const int size = coords + 1 + classes;
    for (int i = 0; i < h * w; ++i) {
        int row = i / w, col = i % w;
        for (int n = 0; n < num; ++n) {
            int index = i * num + n;
            float scale = pred[(size_t)index * size + coords];
            size_t bi = (size_t)index * size;
            float x = (col + 1.0f / (1.0f + expf(-pred[bi + 0]))) / w;
            float y = (row + 1.0f / (1.0f + expf(-pred[bi + 1]))) / h;
            float bw = expf(pred[bi + 2]) * biases[2 * n] / w;
            float bh = expf(pred[bi + 3]) * biases[2 * n + 1] / h;
            for (int j = 0; j < classes; ++j) {
                float p = scale * pred[bi + coords + 1 + j];
                if (p >= thr) {
                    if (*count < cap) {
                        float x1 = x * img_w, y1 = y * img_h, ww = bw * img_w, hh = bh * img_h;
                        pxo_detection* d = dets + *count;
                        d->x = x1 - ww / 2.0f; d->y = y1 - hh / 2.0f; d->w = ww; d->h = hh;
                        d->prob = p; d->class_id = j; d->batch_id = b; d->source = index;
                    }
                    ++*count;
                }
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* NMS: src/Box.cpp:25-145.                                            */
/* cv::Rect2f intersection and area follow OpenCV >= 4.5.4 (the        */
/* version CMakeLists.txt:86 requires), core/types.hpp operator&=.     */
/* ------------------------------------------------------------------ */
typedef struct { float x, y, w, h; } rectf;

static int rect_empty(rectf r) { return r.w <= 0 || r.h <= 0; }

static rectf rect_and(rectf a, rectf b)
{
    rectf z = { 0, 0, 0, 0 };
    if (rect_empty(a) || rect_empty(b)) return z;
    const rectf* rx_min = (a.x < b.x) ? &a : &b;
    const rectf* rx_max = (a.x < b.x) ? &b : &a;
    const rectf* ry_min = (a.y < b.y) ? &a : &b;
    const rectf* ry_max = (a.y < b.y) ? &b : &a;
    if ((rx_min->x < 0 && rx_min->x + rx_min->w < rx_max->x) ||
        (ry_min->y < 0 && ry_min->y + ry_min->h < ry_max->y)) return z;
    rectf r;
    r.w = fminf(rx_min->w - (rx_max->x - rx_min->x), rx_max->w);
    r.h = fminf(ry_min->h - (ry_max->y - ry_min->y), ry_max->h);
    r.x = rx_max->x;
    r.y = ry_max->y;
    if (rect_empty(r)) return z;
    return r;
}

static float rect_area(rectf r) { return r.w * r.h; }

/* boxIoU, src/Box.cpp:35-45 */
static float box_iou(rectf a, rectf b)
{
    float inter = rect_area(rect_and(a, b));
    float uni = fmaxf(0.0f, rect_area(a) + rect_area(b) - rect_area(rect_and(a, b)));
    float r = inter / uni;
    if (isnan(r) || isinf(r)) return 0.0f;
    return r;
}

/* normalizedRect, src/Box.cpp:47-54 */
static rectf rect_norm(const pxo_detection* d)
{
    float x1 = fminf(d->x, d->x + d->w), y1 = fminf(d->y, d->y + d->h);
    float x2 = fmaxf(d->x, d->x + d->w), y2 = fmaxf(d->y, d->y + d->h);
    rectf r = { x1, y1, fmaxf(0.0f, x2 - x1), fmaxf(0.0f, y2 - y1) };
    return r;
}

/* stable merge sort by prob descending (std::stable_sort, Box.cpp:60-62) */
static void stable_sort_desc(pxo_detection* a, pxo_detection* tmp, size_t n)
{
    if (n < 2) return;
    size_t m = n / 2;
    stable_sort_desc(a, tmp, m);
    stable_sort_desc(a + m, tmp, n - m);
    size_t i = 0, j = m, k = 0;
    while (i < m && j < n) tmp[k++] = (a[j].prob > a[i].prob) ? a[j++] : a[i++];
    while (i < m) tmp[k++] = a[i++];
    while (j < n) tmp[k++] = a[j++];
    memcpy(a, tmp, n * sizeof(*a));
}

PXO_API float pxo_box_iou(const pxo_detection* a, const pxo_detection* b)
{
    return box_iou(rect_norm(a), rect_norm(b));
}

/*
 * nms, src/Box.cpp:56-145.  out must hold n records; returns the number kept.
 * The reference's R-tree only pre-filters by bounding-box intersection; a scan
 * over the retained boxes of the group gives the same suppression decisions
 * because IoU > threshold >= 0 implies an intersecting box.  Only the first
 * 1024 members of each (image, class) group are examined (Box.cpp:104-108).
 */
PXO_API long long pxo_nms(const pxo_detection* dets, long long n, float threshold,
                          pxo_detection* out)
{
    if (n <= 0) return 0;
    pxo_detection* s = (pxo_detection*)malloc((size_t)n * sizeof(*s));
    pxo_detection* tmp = (pxo_detection*)malloc((size_t)n * sizeof(*s));
    unsigned char* discard = (unsigned char*)calloc((size_t)n, 1);
    memcpy(s, dets, (size_t)n * sizeof(*s));
    stable_sort_desc(s, tmp, (size_t)n);

    /* cross-class near-duplicate pass, Box.cpp:69-88 */
    for (long long i = 0; i < n; ++i) {
        if (discard[i]) continue;
        for (long long j = 0; j < i; ++j) {
            if (discard[j] || s[i].batch_id != s[j].batch_id || s[i].class_id == s[j].class_id) continue;
            if (box_iou(rect_norm(&s[i]), rect_norm(&s[j])) > 0.9f) { discard[i] = 1; break; }
        }
    }

    /* per-(image, class) greedy suppression, Box.cpp:94-133 */
    long long* kept = (long long*)malloc((size_t)n * sizeof(long long));
    unsigned char* seen = (unsigned char*)calloc((size_t)n, 1);
    for (long long g = 0; g < n; ++g) {
        if (seen[g]) continue;
        long long position = 0, nkept = 0;
        for (long long i = g; i < n; ++i) {
            if (s[i].batch_id != s[g].batch_id || s[i].class_id != s[g].class_id) continue;
            seen[i] = 1;
            if (position++ >= 1024) continue;
            if (discard[i]) continue;
            rectf box = rect_norm(&s[i]);
            int suppressed = 0;
            for (long long k = 0; k < nkept; ++k)
                if (box_iou(box, rect_norm(&s[kept[k]])) > threshold) { suppressed = 1; break; }
            if (suppressed) discard[i] = 1; else kept[nkept++] = i;
        }
    }

    long long m = 0;
    for (long long i = 0; i < n; ++i) if (!discard[i]) out[m++] = s[i];
    free(s); free(tmp); free(discard); free(kept); free(seen);
    return m;
}

/* ------------------------------------------------------------------ */
/* CPU convolution pieces for the timed CPU forward:                   */
/* im2ColCpuExt src/CpuUtil.cpp:74-105; GEMM call ConvLayer.h:212-225  */
/* ------------------------------------------------------------------ */
PXO_API void pxo_im2col(const float* im, int channels, int height, int width, int kh, int kw,
                        int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                        float* col)
{
    const int out_h = (height + 2 * pad_h - (dil_h * (kh - 1) + 1)) / stride_h + 1;
    const int out_w = (width + 2 * pad_w - (dil_w * (kw - 1) + 1)) / stride_w + 1;
    for (int c = 0; c < channels; ++c)
        for (int i = 0; i < kh; ++i)
            for (int j = 0; j < kw; ++j) {
                size_t row = (size_t)c * kh * kw + (size_t)i * kw + j;
                for (int oh = 0; oh < out_h; ++oh) {
                    int in_y = oh * stride_h - pad_h + i * dil_h;
                    for (int ow = 0; ow < out_w; ++ow) {
                        int in_x = ow * stride_w - pad_w + j * dil_w;
                        float v = 0.0f;
                        if (in_y >= 0 && in_y < height && in_x >= 0 && in_x < width)
                            v = im[(size_t)c * height * width + (size_t)in_y * width + in_x];
                        col[row * out_h * out_w + (size_t)oh * out_w + ow] = v;
                    }
                }
            }
}

typedef void (*pxo_sgemm_fn)(int order, int transa, int transb, int m, int n, int k, float alpha,
                             const float* a, int lda, const float* b, int ldb, float beta,
                             float* c, int ldc);

/*
 * ConvLayer<CPU>::forward GEMM part, include/ConvLayer.h:195-225, groups == 1:
 * per image im2ColCpuExt (always, also for 1x1 kernels) and
 * C = W[F, K*K*C] x col[K*K*C, OH*OW].  sgemm is a CBLAS-compatible sgemm
 * (RowMajor = 101, NoTrans = 111) supplied by the caller.
 */
PXO_API void pxo_conv_forward(pxo_sgemm_fn sgemm, const float* in, const float* weights,
                              float* out, float* column, int batch, int channels, int height,
                              int width, int filters, int kernel, int stride, int pad, int dilation)
{
    const int eff = dilation * (kernel - 1) + 1;
    const int out_h = (height + 2 * pad - eff) / stride + 1;
    const int out_w = (width + 2 * pad - eff) / stride + 1;
    const int m = filters, n = out_h * out_w, k = kernel * kernel * channels;
    for (int b = 0; b < batch; ++b) {
        const float* im = in + (size_t)b * channels * height * width;
        pxo_im2col(im, channels, height, width, kernel, kernel, pad, pad, stride, stride,
                   dilation, dilation, column);
        sgemm(101, 111, 111, m, n, k, 1.0f, weights, k, column, n, 0.0f,
              out + (size_t)b * m * n, n);
    }
}


/* ------------------------------------------------------------------ */
/* Detector losses as the reference's CUDA path computes them:         */
/* src/YoloKernels.cu:11-214, src/CenterNetKernels.cu:20-122.          */
/* Sums are taken in index order, in double, so that they can serve as */
/* the reference value for any order of float additions.               */
/* ------------------------------------------------------------------ */
static float loss_overlap(float x1, float w1, float x2, float w2)
{
    return fminf(x1 + w1 / 2.0f, x2 + w2 / 2.0f) - fmaxf(x1 - w1 / 2.0f, x2 - w2 / 2.0f);   /* :11-15 */
}

static float loss_box_iou(const float* a, const float* b)                                   /* :17-24 */
{
    float w = loss_overlap(a[0], a[2], b[0], b[2]);
    float h = loss_overlap(a[1], a[3], b[1], b[3]);
    float intersection = w > 0.0f && h > 0.0f ? w * h : 0.0f;
    float union_area = fmaxf(0.0f, a[2] * a[3] + b[2] * b[3] - intersection);
    return union_area > 0.0f ? intersection / union_area : 0.0f;
}

static void loss_decode_box(const float* out, float* box, int area, int x, int y, int anchor, const float* anchors,
                            int width, int height, int net_w, int net_h)                    /* :33-46 */
{
    box[0] = (x + out[0]) / width;
    box[1] = (y + out[area]) / height;
    box[2] = expf(out[2 * area]) * anchors[2 * anchor] / net_w;
    box[3] = expf(out[3 * area]) * anchors[2 * anchor + 1] / net_h;
}

static void loss_box_delta(const float* truth, const float* out, float* del, int area, int x, int y, int width,
                           int height, int net_w, int net_h, const float* anchors, int anchor, float coord_scale)
{                                                                                            /* :48-61 */
    float scale = coord_scale * (2.0f - truth[2] * truth[3]);
    float tx = truth[0] * width - x;
    float ty = truth[1] * height - y;
    float tw = logf(fmaxf(1e-9f, truth[2] * net_w / anchors[2 * anchor]));
    float th = logf(fmaxf(1e-9f, truth[3] * net_h / anchors[2 * anchor + 1]));
    del[0] = scale * (tx - out[0]);
    del[area] = scale * (ty - out[area]);
    del[2 * area] = scale * (tw - out[2 * area]);
    del[3 * area] = scale * (th - out[3 * area]);
}

/* yoloLossGpu, src/YoloKernels.cu:223-252: the region pass, the object pass, the squared norm of delta and the
 * loss components, in that order.  stats: 12 doubles, cost: 1 double, both added to. */
PXO_API void pxo_yolo_loss(const float* output, float* delta, const float* truths, const int* truth_counts, int max_truth,
                           const int* assigned_classes, const int* assigned_anchors, const float* assigned_boxes,
                           const int* masks, const float* anchors, double* stats, double* cost, int batch, int mask_count,
                           int classes, int width, int height, int net_w, int net_h, float ignore_thr, float truth_thr,
                           float coord_scale, float object_scale, float no_object_scale, float class_scale)
{
    const int area = width * height, entries = classes + 5;
    const int slots = batch * mask_count * area;
    for (int slot = 0; slot < slots; ++slot) {                                              /* :73-124 */
        int b = slot / (mask_count * area), within = slot % (mask_count * area);
        int ms = within / area, cell = within % area;
        int x = cell % width, y = cell / width;
        const float* out = output + (size_t)b * mask_count * entries * area + (size_t)ms * entries * area + cell;
        float* del = delta + (out - output);
        float pred[4];
        loss_decode_box(out, pred, area, x, y, masks[ms], anchors, width, height, net_w, net_h);
        float best_iou = -FLT_MAX;
        int best = -1;
        for (int t = 0; t < truth_counts[b]; ++t) {
            int ti = (b * max_truth + t) * 5;
            float iou = loss_box_iou(pred, truths + ti);
            if (iou > best_iou) { best_iou = iou; best = ti; }
        }
        float objectness = out[4 * area];
        stats[5] += objectness;
        if (best < 0 || best_iou < ignore_thr) del[4 * area] = -no_object_scale * objectness;
        if (best >= 0 && best_iou > truth_thr) {
            del[4 * area] = object_scale * (1.0f - objectness);
            int class_id = (int)truths[best + 4];
            for (int c = 0; c < classes; ++c)
                del[(5 + c) * area] = class_scale * ((c == class_id ? 1.0f : 0.0f) - out[(5 + c) * area]);
            loss_box_delta(truths + best, out, del, area, x, y, width, height, net_w, net_h, anchors, masks[ms], coord_scale);
        }
    }
    for (int slot = 0; slot < slots; ++slot) {                                              /* :126-168 */
        if (assigned_classes[slot] < 0) continue;
        int b = slot / (mask_count * area), within = slot % (mask_count * area);
        int ms = within / area, cell = within % area;
        int x = cell % width, y = cell / width;
        const float* out = output + (size_t)b * mask_count * entries * area + (size_t)ms * entries * area + cell;
        float* del = delta + (out - output);
        const float* truth = assigned_boxes + (size_t)slot * 4;
        int anchor = assigned_anchors[slot];
        float pred[4];
        loss_decode_box(out, pred, area, x, y, anchor, anchors, width, height, net_w, net_h);
        float iou = loss_box_iou(pred, truth);
        loss_box_delta(truth, out, del, area, x, y, width, height, net_w, net_h, anchors, anchor, coord_scale);
        stats[4] += out[4 * area];
        del[4 * area] = object_scale * (1.0f - out[4 * area]);
        int class_id = assigned_classes[slot];
        for (int c = 0; c < classes; ++c) {
            float truth_class = c == class_id ? 1.0f : 0.0f;
            del[(5 + c) * area] = class_scale * (truth_class - out[(5 + c) * area]);
            if (truth_class != 0.0f) stats[3] += fminf(1.0f, out[(5 + c) * area]);
        }
        stats[0] += iou;
        if (iou > 0.5f) stats[1] += 1.0;
        if (iou > 0.75f) stats[2] += 1.0;
        stats[6] += 1.0;
        stats[7] += 1.0;
    }
    const size_t outputs = (size_t)slots * entries;                                         /* :170-182 */
    for (size_t i = 0; i < outputs; ++i) *cost += (double)(delta[i] * delta[i]);
    for (int slot = 0; slot < slots; ++slot) {                                              /* :184-214 */
        int b = slot / (mask_count * area), within = slot % (mask_count * area);
        int ms = within / area, cell = within % area;
        const float* del = delta + (size_t)b * mask_count * entries * area + (size_t)ms * entries * area + cell;
        float box = 0.0f;
        for (int k = 0; k < 4; ++k) box += del[k * area] * del[k * area];
        stats[8] += box;
        float object = del[4 * area];
        stats[object >= 0.0f ? 9 : 10] += (double)(object * object);
        float cls = 0.0f;
        for (int c = 0; c < classes; ++c) cls += del[(5 + c) * area] * del[(5 + c) * area];
        stats[11] += cls;
    }
}

/* centerNetLossGpu, src/CenterNetKernels.cu:20-139.  costs: 3 doubles, added to. */
PXO_API void pxo_centernet_loss(const float* output, float* delta, const float* target_heat, const float* target_size,
                                const float* target_offset, const float* target_mask, double* costs, int batch,
                                int classes, int area, float normalizer, float alpha, float beta, float size_weight)
{
    const size_t outputs = (size_t)(classes + 4) * area, heat = (size_t)classes * area;
    for (size_t i = 0; i < (size_t)batch * heat; ++i) {                                     /* :20-61 */
        size_t b = i / heat, at = b * outputs + i % heat;
        float prediction = fminf(fmaxf(output[at], 1e-4f), 1.0f - 1e-4f);
        float truth = target_heat[i];
        float loss;
        if (truth >= 1.0f - 1e-6f) {
            float one_minus = 1.0f - prediction;
            loss = -powf(one_minus, alpha) * logf(prediction);
            delta[at] = normalizer * (powf(one_minus, alpha + 1.0f) - alpha * prediction * powf(one_minus, alpha) * logf(prediction));
        } else {
            float weight = powf(1.0f - truth, beta);
            loss = -weight * powf(prediction, alpha) * logf(1.0f - prediction);
            delta[at] = normalizer * weight * (alpha * powf(prediction, alpha) * (1.0f - prediction) * logf(1.0f - prediction)
                                               - powf(prediction, alpha + 1.0f));
        }
        costs[0] += loss;
    }
    for (size_t i = 0; i < (size_t)batch * area; ++i) {                                     /* :63-122 */
        if (target_mask[i] == 0.0f) continue;
        size_t b = i / area, cell = i % area;
        for (int channel = 0; channel < 2; ++channel) {
            size_t map = (size_t)channel * area + cell;
            size_t si = b * outputs + heat + map, oi = b * outputs + heat + 2 * (size_t)area + map;
            float size_error = target_size[b * 2 * area + map] - output[si];
            float offset_error = target_offset[b * 2 * area + map] - output[oi];
            costs[1] += fabsf(size_error);
            costs[2] += fabsf(offset_error);
            delta[si] = size_weight * normalizer * (float)((size_error > 0.0f) - (size_error < 0.0f));
            delta[oi] = normalizer * (float)((offset_error > 0.0f) - (offset_error < 0.0f));
        }
    }
}
