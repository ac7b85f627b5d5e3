/*
 * pxe_compat.hpp -- link-compatible tier.
 *
 * The eight free functions PixieNN's CUDA layers call between convolutions, declared with the
 * reference's exact C++ signatures (namespace px, same parameter types and order), so that the
 * reference links against libpxe.so instead of its own src/*.cu objects with no source change.
 * Each one forwards to the C ABI in pxe.h on the legacy default stream and, like the
 * reference's PX_CUDA_CHECK_LAST, throws on failure (std::runtime_error here; the reference
 * throws px::CudaError, which also derives from std::exception).
 *
 * Unlike the reference's versions, none of these synchronises the device
 * (src/UpsampleKernels.cu:60 and src/ShortcutKernel.cu:62 call cudaDeviceSynchronize).
 */
#pragma once
#include <cstddef>

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
/* include/UpsampleKernels.cuh:21 (forward != 0 only; the backward mode is training code) */
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

}   // namespace px
