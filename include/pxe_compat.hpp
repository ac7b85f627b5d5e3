/*
 * pxe_compat.hpp -- link-compatible tier.
 *
 * The free functions of the reference's src/Activation.cu, BiasKernels.cu, MaxPoolKernels.cu,
 * UpsampleKernels.cu, ShortcutKernel.cu, CudaUtils.cu, YoloKernels.cu and CenterNetKernels.cu -- forward,
 * backward and loss -- declared with the reference's exact C++ signatures (namespace px, same
 * parameter types and order), so that the reference links against libpxe.so instead of those
 * eight object files with no source change.
 * Each one forwards to the C ABI in pxe.h on the legacy default stream and, like the
 * reference's PX_CUDA_CHECK_LAST, throws on failure (std::runtime_error here; the reference
 * throws px::CudaError, which also derives from std::exception).
 *
 * Unlike the reference's versions, none of these synchronises the device
 * (src/UpsampleKernels.cu:60 and src/ShortcutKernel.cu:62 call cudaDeviceSynchronize).
 */
#pragma once
#include <cstddef>
#include <cstdint>

#include <vector_types.h>

/* include/ActivationTypes.h:19-30 -- must stay value- and name-identical for the mangled
 * name of px::activate to match. */
#ifndef PXE_HAVE_ACTIVATION_TYPES
enum ActivationType : int
{
    LEAKY = 0,
    LINEAR,
    LOGGY,
    LOGISTIC,
    MISH,
    RELU,
    SOFTPLUS,
    SWISH,
    TANH,
};
#endif

namespace px {

/* include/Activation.cuh:26 */
void activate(ActivationType type, float* x, std::size_t n);
/* include/BiasKernels.cuh:21 */
void addBiasGpu(float* output, const float* biases, int batch, int n, int size);
/* include/MaxPoolKernels.cuh:5 */
void maxPoolForwardGpu(const float* input, float* output, int* indexes, int batch, int channels, int inputHeight,
                       int inputWidth, int outputHeight, int outputWidth, int kernel, int stride, int padding);
/* include/UpsampleKernels.cuh:21 (forward != 0: out = scale * in; forward == 0: acc += scale * out, summed per input) */
void upsampleGpu(const float* in, int w, int h, int c, int batch, int stride, int forward, float scale, float* acc,
                 float* out);
/* include/ShortcutKernel.cuh:21 */
void shortcutGpu(int batch, int w1, int h1, int c1, const float* add, int w2, int h2, int c2, float s1, float s2,
                 float* out);
/* include/YoloKernels.cuh:7 */
void yoloActivateGpu(const float* input, float* output, int batch, int masks, int classes, int area);
/* include/CenterNetKernels.cuh:5 */
void centerNetActivateGpu(const float* input, float* output, int batch, int classes, int area, float heatmapBias);
/* include/CudaUtils.cuh:29-30 */
void fillGpu(float* ptr, std::size_t n, float value);
void fillGpu(int* ptr, std::size_t n, int value);
/* include/Activation.cuh:27 */
void gradient(ActivationType type, const float* x, std::size_t n, float* delta);
/* include/BiasKernels.cuh:22 */
void backwardBiasGpu(float* biasUpdates, const float* delta, int batch, int n, int size);
/* include/MaxPoolKernels.cuh:7 */
void maxPoolBackwardGpu(const float* delta, const int* indexes, float* grad, int size);
/* include/CudaUtils.cuh:27-33.  cudaGridsize: the launch grid for n threads in blocks of CUDA_BLOCK_SIZE = 512,
 * folded into two dimensions beyond 65535 blocks (src/CudaUtils.cu:28-43); the reference's own kernels that
 * stay in a build (Adam, the loss launchers) size their launches with it. */
void constrainGpu(int n, float alpha, float* x);
dim3 cudaGridsize(std::uint32_t n);
void mulGpu(int n, float* x, float* y);
void randomGpu(float* ptr, std::size_t n, float a = 0.f, float b = 1.f);
void randomNormalGpu(float* ptr, std::size_t n, float mean = 0.f, float stddev = 1.f);
/* include/YoloKernels.cuh:10-19 */
void yoloLossGpu(const float* output, float* delta, const float* truths, const int* truthCounts, int maxTruth,
                 const int* assignedClasses, const int* assignedAnchors, const float* assignedBoxes, const int* masks,
                 const float* anchors, float* stats, float* cost, int batch, int maskCount, int anchorCount, int classes,
                 int width, int height, int networkWidth, int networkHeight, float ignoreThreshold,
                 float truthThreshold, float coordScale, float objectScale, float noObjectScale, float classScale);
/* include/CenterNetKernels.cuh:8-13 */
void centerNetLossGpu(const float* output, float* delta, const float* targetHeatmap, const float* targetSize,
                      const float* targetOffset, const float* targetMask, float* costs, int batch, int classes, int area,
                      float normalizer, float focalAlpha, float focalBeta, float sizeWeight);
/* include/Adam.cuh:21 */
void adamGpu(int n, float* x, float* m, float* v, float beta1, float beta2, float rate, float eps, int t);
/* include/SoftmaxKernel.cuh:21 */
void softmaxCrossEntropy(int n, const float* pred, const float* truth, float* delta, float* error);

}   // namespace px
