// Link-compatible tier: the reference's px:: free functions (same mangled names) on top of the
// C ABI.  See include/pxe_compat.hpp.
#include <stdexcept>
#include <string>

#include "pxe_common.cuh"
#include "pxe_compat.hpp"

namespace {

void check(int rc, const char* what)
{
    if (rc != PXE_OK) throw std::runtime_error(std::string(what) + ": " + pxe_last_error_string());
}

template <typename T>
__global__ void fill_kernel(T* ptr, size_t n, T value)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        ptr[i] = value;
}

template <typename T>
void fill(T* ptr, size_t n, T value)
{
    if (n == 0) return;
    pxe::DeviceInfo di;
    check(pxe::device_info(&di), "fillGpu");
    fill_kernel<T><<<pxe::grid_for((long long)n, 256 * 4, di.sm_count, 16), 256>>>(ptr, n, value);
    if (cudaPeekAtLastError() != cudaSuccess) throw std::runtime_error("fillGpu: launch failed");
}

}  // namespace

#define PXE_EXPORT __attribute__((visibility("default")))

namespace px {

PXE_EXPORT void activate(ActivationType type, float* x, std::size_t n)
{
    check(pxe_activate(nullptr, (int)type, x, n), "activate");
}

PXE_EXPORT void addBiasGpu(float* output, const float* biases, int batch, int n, int size)
{
    check(pxe_add_bias(nullptr, output, biases, batch, n, size), "addBiasGpu");
}

PXE_EXPORT void maxPoolForwardGpu(const float* input, float* output, int* indexes, int batch, int channels,
                                  int inputHeight, int inputWidth, int outputHeight, int outputWidth, int kernel,
                                  int stride, int padding)
{
    if (pxe_maxpool_out_dim(inputHeight, kernel, stride, padding) != outputHeight ||
        pxe_maxpool_out_dim(inputWidth, kernel, stride, padding) != outputWidth)
        throw std::runtime_error("maxPoolForwardGpu: output extent does not match (in + padding - kernel)/stride + 1");
    check(pxe_maxpool(nullptr, input, 0, output, 0, indexes, batch, channels, inputHeight, inputWidth, kernel, stride,
                      padding), "maxPoolForwardGpu");
}

PXE_EXPORT void upsampleGpu(const float* in, int w, int h, int c, int batch, int stride, int forward, float scale,
                            float* acc, float* out)
{
    (void)acc;
    if (!forward) throw std::runtime_error("upsampleGpu: the backward mode is not part of the inference path");
    check(pxe_upsample(nullptr, in, 0, out, 0, batch, c, h, w, stride, scale), "upsampleGpu");
}

PXE_EXPORT void shortcutGpu(int batch, int w1, int h1, int c1, const float* add, int w2, int h2, int c2, float s1,
                            float s2, float* out)
{
    if (w1 == w2 && h1 == h2 && c1 == c2)
        check(pxe_shortcut(nullptr, out, 0, add, 0, out, 0, nullptr, 0, batch, c1, h1, w1, s1, s2, PXE_ACT_LINEAR),
              "shortcutGpu");
    else
        check(pxe_shortcut_general(nullptr, batch, w1, h1, c1, add, w2, h2, c2, s1, s2, out), "shortcutGpu");
}

PXE_EXPORT void yoloActivateGpu(const float* input, float* output, int batch, int masks, int classes, int area)
{
    check(pxe_yolo_activate(nullptr, input, output, batch, masks, classes, area), "yoloActivateGpu");
}

PXE_EXPORT void centerNetActivateGpu(const float* input, float* output, int batch, int classes, int area,
                                     float heatmapBias)
{
    check(pxe_centernet_activate(nullptr, input, output, batch, classes, area, heatmapBias), "centerNetActivateGpu");
}

PXE_EXPORT void fillGpu(float* ptr, std::size_t n, float value) { fill<float>(ptr, n, value); }
PXE_EXPORT void fillGpu(int* ptr, std::size_t n, int value) { fill<int>(ptr, n, value); }

}  // namespace px
