/*
 * ref_cuda_glue.cu -- extern "C" doorway into the reference's own CUDA epilogue kernels.
 *
 * TEST / BASELINE INFRASTRUCTURE ONLY.  Compiled together with the reference's unmodified
 * src/{Activation,Adam,BiasKernels,MaxPoolKernels,UpsampleKernels,ShortcutKernel,YoloKernels,
 * CenterNetKernels,CudaUtils}.cu (read in place from the reference tree, never copied) into
 * oracle/_ref/libpxref_cuda.so.  The forwarding functions let tests compare the new kernels with
 * the reference's kernels on the same device; the *_replay functions issue the exact call
 * sequence of the reference's Layer<Device::CUDA>::forward bodies so that it can be timed.
 */
#include <cstddef>
#include <cuda_runtime.h>
#include <cudnn.h>

#include "Activation.cuh"
#include "Adam.cuh"
#include "BiasKernels.cuh"
#include "CenterNetKernels.cuh"
#include "CudaUtils.cuh"
#include "MaxPoolKernels.cuh"
#include "ShortcutKernel.cuh"
#include "UpsampleKernels.cuh"
#include "YoloKernels.cuh"

#define API extern "C" __attribute__((visibility("default")))

namespace {
cudnnHandle_t g_cudnn = nullptr;
cudnnTensorDescriptor_t g_y = nullptr, g_sbmv = nullptr;

int ensure_cudnn()
{
    if (g_cudnn) return 0;
    if (cudnnCreate(&g_cudnn) != CUDNN_STATUS_SUCCESS) return 1;
    cudnnCreateTensorDescriptor(&g_y);
    cudnnCreateTensorDescriptor(&g_sbmv);
    return 0;
}
}  // namespace

template <typename F>
static int guarded(F f)
{
    try { f(); } catch (...) { return 1; }
    return 0;
}

API int pxrefcu_activate(int type, float* x, std::size_t n)
{
    return guarded([&] { px::activate(static_cast<ActivationType>(type), x, n); });
}

API int pxrefcu_add_bias(float* out, const float* bias, int batch, int n, int size)
{
    return guarded([&] { px::addBiasGpu(out, bias, batch, n, size); });
}

API int pxrefcu_maxpool(const float* in, float* out, int* idx, int batch, int c, int ih, int iw, int oh, int ow,
                        int kernel, int stride, int padding)
{
    return guarded([&] { px::maxPoolForwardGpu(in, out, idx, batch, c, ih, iw, oh, ow, kernel, stride, padding); });
}

API int pxrefcu_upsample(const float* in, int w, int h, int c, int batch, int stride, float scale, float* out)
{
    return guarded([&] { px::upsampleGpu(in, w, h, c, batch, stride, 1, scale, nullptr, out); });
}

API int pxrefcu_shortcut(int batch, int w1, int h1, int c1, const float* add, int w2, int h2, int c2, float s1,
                         float s2, float* out)
{
    return guarded([&] { px::shortcutGpu(batch, w1, h1, c1, add, w2, h2, c2, s1, s2, out); });
}

API int pxrefcu_yolo_activate(const float* in, float* out, int batch, int masks, int classes, int area)
{
    return guarded([&] { px::yoloActivateGpu(in, out, batch, masks, classes, area); });
}

API int pxrefcu_centernet_activate(const float* in, float* out, int batch, int classes, int area, float bias)
{
    return guarded([&] { px::centerNetActivateGpu(in, out, batch, classes, area, bias); });
}

API int pxrefcu_gradient(int type, const float* x, std::size_t n, float* delta)
{
    return guarded([&] { px::gradient(static_cast<ActivationType>(type), x, n, delta); });
}

API int pxrefcu_backward_bias(float* bias_updates, const float* delta, int batch, int n, int size)
{
    return guarded([&] { px::backwardBiasGpu(bias_updates, delta, batch, n, size); });
}

API int pxrefcu_maxpool_backward(const float* delta, const int* indexes, float* grad, int size)
{
    return guarded([&] { px::maxPoolBackwardGpu(delta, indexes, grad, size); });
}

API int pxrefcu_upsample_backward(int w, int h, int c, int batch, int stride, float scale, float* acc, float* out)
{
    return guarded([&] { px::upsampleGpu(nullptr, w, h, c, batch, stride, 0, scale, acc, out); });
}

API int pxrefcu_constrain(int n, float alpha, float* x)
{
    return guarded([&] { px::constrainGpu(n, alpha, x); });
}

API int pxrefcu_mul(int n, float* x, float* y)
{
    return guarded([&] { px::mulGpu(n, x, y); });
}

API int pxrefcu_adam(int n, float* x, float* m, float* v, float beta1, float beta2, float rate, float eps, int t)
{
    return guarded([&] { px::adamGpu(n, x, m, v, beta1, beta2, rate, eps, t); });
}

API int pxrefcu_random(float* p, std::size_t n, float a, float b)
{
    return guarded([&] { px::randomGpu(p, n, a, b); });
}

API int pxrefcu_random_normal(float* p, std::size_t n, float mean, float stddev)
{
    return guarded([&] { px::randomNormalGpu(p, n, mean, stddev); });
}

API int pxrefcu_yolo_loss(const float* output, float* delta, const float* truths, const int* truth_counts,
                          const int* assigned_classes, const int* assigned_anchors, const float* assigned_boxes,
                          const int* masks, const float* anchors, float* stats, float* cost, const void* unused,
                          int max_truth, int batch, int mask_count, int anchor_count, int classes, int width, int height,
                          int net_w, int net_h, float ignore_thr, float truth_thr, float coord_scale, float object_scale,
                          float no_object_scale, float class_scale)
{
    (void)unused;
    return guarded([&] {
        px::yoloLossGpu(output, delta, truths, truth_counts, max_truth, assigned_classes, assigned_anchors, assigned_boxes,
                        masks, anchors, stats, cost, batch, mask_count, anchor_count, classes, width, height, net_w, net_h,
                        ignore_thr, truth_thr, coord_scale, object_scale, no_object_scale, class_scale);
    });
}

API int pxrefcu_centernet_loss(const float* output, float* delta, const float* target_heat, const float* target_size,
                               const float* target_offset, const float* target_mask, float* costs, int batch, int classes,
                               int area, float normalizer, float alpha, float beta, float size_weight)
{
    return guarded([&] {
        px::centerNetLossGpu(output, delta, target_heat, target_size, target_offset, target_mask, costs, batch, classes,
                             area, normalizer, alpha, beta, size_weight);
    });
}

API void pxrefcu_gridsize(unsigned n, unsigned* xyz)
{
    const dim3 d = px::cudaGridsize(n);
    xyz[0] = d.x; xyz[1] = d.y; xyz[2] = d.z;
}

API int pxrefcu_fill(float* p, std::size_t n, float v)
{
    return guarded([&] { px::fillGpu(p, n, v); });
}

/* cudnnBatchNormalizationForwardInference exactly as include/cuda/ConvLayer.h:294-299 calls it:
 * spatial mode, alpha 1, beta 0, in place, epsilon 1e-5, NCHW float descriptors. */
API int pxrefcu_batchnorm_inference(float* x, const float* gamma, const float* beta, const float* mean,
                                    const float* var, int batch, int channels, int height, int width)
{
    if (ensure_cudnn()) return 1;
    if (cudnnSetTensor4dDescriptor(g_y, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, batch, channels, height, width)
        != CUDNN_STATUS_SUCCESS) return 2;
    if (cudnnSetTensor4dDescriptor(g_sbmv, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, 1, channels, 1, 1)
        != CUDNN_STATUS_SUCCESS) return 2;
    float alpha = 1.0f, zero = 0.0f;
    auto st = cudnnBatchNormalizationForwardInference(g_cudnn, CUDNN_BATCHNORM_SPATIAL, &alpha, &zero, g_y, x, g_y, x,
                                                      g_sbmv, gamma, beta, mean, var, 0.00001);
    return st == CUDNN_STATUS_SUCCESS ? 0 : 3;
}

/*
 * The epilogue part of ConvLayer<Device::CUDA>::forward (include/cuda/ConvLayer.h:266-308) as the
 * reference runs it when inferring, minus the convolution itself: Layer::forward's two fills
 * (include/Layer.h:377-383), BN inference or addBiasGpu, the preActivation_ device copy, the
 * activation.  `out` plays output_ (already holding the conv result; the fill of output_ is issued
 * on `scratch` so the data survives), `delta` and `preact` are the layer's other buffers.
 */
API int pxrefcu_conv_epilogue_replay(float* out, float* delta, float* preact, float* scratch, int batch, int channels,
                                     int height, int width, const float* gamma, const float* beta, const float* mean,
                                     const float* var, const float* bias, int act)
{
    const std::size_t n = static_cast<std::size_t>(batch) * channels * height * width;
    return guarded([&] {
        px::fillGpu(delta, n, 0.0f);
        px::fillGpu(scratch, n, 0.0f);
        if (gamma) {
            if (pxrefcu_batchnorm_inference(out, gamma, beta, mean, var, batch, channels, height, width)) throw 1;
        } else {
            px::addBiasGpu(out, bias, batch, channels, height * width);
        }
        if (cudaMemcpy(preact, out, n * sizeof(float), cudaMemcpyDeviceToDevice) != cudaSuccess) throw 2;
        px::activate(static_cast<ActivationType>(act), out, n);
    });
}

/* MaxPoolLayer<Device::CUDA>::forward, include/cuda/MaxPoolLayer.h:36-42 (+ base-class fills). */
API int pxrefcu_maxpool_replay(const float* in, float* out, float* delta, int* idx, int batch, int c, int ih, int iw,
                               int oh, int ow, int kernel, int stride, int padding)
{
    const std::size_t n = static_cast<std::size_t>(batch) * c * oh * ow;
    return guarded([&] {
        px::fillGpu(delta, n, 0.0f);
        px::fillGpu(out, n, 0.0f);
        px::maxPoolForwardGpu(in, out, idx, batch, c, ih, iw, oh, ow, kernel, stride, padding);
    });
}

/* UpsampleLayer<Device::CUDA>::forward, include/cuda/UpsampleLayer.h:33-40 (+ fills). */
API int pxrefcu_upsample_replay(const float* in, float* out, float* delta, int batch, int c, int h, int w, int stride,
                                float scale)
{
    const std::size_t n = static_cast<std::size_t>(batch) * c * h * w * stride * stride;
    return guarded([&] {
        px::fillGpu(delta, n, 0.0f);
        px::fillGpu(out, n, 0.0f);
        px::upsampleGpu(in, w, h, c, batch, stride, 1, scale, nullptr, out);
    });
}

/* ShortcutLayer<Device::CUDA>::forward, include/cuda/ShortcutLayer.h:23-34 (+ fills). */
API int pxrefcu_shortcut_replay(const float* in, const float* from, float* out, float* delta, int batch, int c, int h,
                                int w, float alpha, float beta, int act)
{
    const std::size_t n = static_cast<std::size_t>(batch) * c * h * w;
    return guarded([&] {
        px::fillGpu(delta, n, 0.0f);
        px::fillGpu(out, n, 0.0f);
        if (cudaMemcpy(out, in, n * sizeof(float), cudaMemcpyDeviceToDevice) != cudaSuccess) throw 2;
        px::shortcutGpu(batch, w, h, c, from, w, h, c, alpha, beta, out);
        px::activate(static_cast<ActivationType>(act), out, n);
    });
}

/* RouteLayer<Device::CUDA>::forward, include/cuda/RouteLayer.h:21-44: one blocking device copy per
 * (source, image) (+ fills). */
API int pxrefcu_route_replay(int n_src, const float* const* srcs, const int* src_outputs, float* out, float* delta,
                             int batch)
{
    std::size_t outputs = 0;
    for (int s = 0; s < n_src; ++s) outputs += src_outputs[s];
    return guarded([&] {
        px::fillGpu(delta, outputs * batch, 0.0f);
        px::fillGpu(out, outputs * batch, 0.0f);
        std::size_t offset = 0;
        for (int s = 0; s < n_src; ++s) {
            for (int i = 0; i < batch; ++i) {
                if (cudaMemcpy(out + i * outputs + offset, srcs[s] + static_cast<std::size_t>(i) * src_outputs[s],
                               src_outputs[s] * sizeof(float), cudaMemcpyDeviceToDevice) != cudaSuccess) throw 2;
            }
            offset += src_outputs[s];
        }
    });
}

/* YoloLayer<Device::CUDA>::forward when inferring, include/cuda/YoloLayer.h:70-78 (+ fills), followed
 * by addDetects' full-tensor device-to-host copy (include/cuda/YoloLayer.h:168-177) into `host`. */
API int pxrefcu_yolo_replay(const float* in, float* out, float* delta, float* host, int batch, int masks, int classes,
                            int area)
{
    const std::size_t n = static_cast<std::size_t>(batch) * masks * (classes + 5) * area;
    return guarded([&] {
        px::fillGpu(delta, n, 0.0f);
        px::fillGpu(out, n, 0.0f);
        px::yoloActivateGpu(in, out, batch, masks, classes, area);
        if (host && cudaMemcpy(host, out, n * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) throw 2;
    });
}
