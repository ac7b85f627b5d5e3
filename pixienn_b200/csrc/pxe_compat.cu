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
        pxe::gst(ptr + i, value);
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
    if (!forward) {
        check(pxe_upsample_backward(nullptr, acc, out, batch, c, h, w, stride, scale), "upsampleGpu");
        return;
    }
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

PXE_EXPORT void gradient(ActivationType type, const float* x, std::size_t n, float* delta)
{
    check(pxe_activation_gradient(nullptr, (int)type, x, n, delta), "gradient");
}

PXE_EXPORT void backwardBiasGpu(float* biasUpdates, const float* delta, int batch, int n, int size)
{
    check(pxe_backward_bias(nullptr, biasUpdates, delta, batch, n, size), "backwardBiasGpu");
}

PXE_EXPORT void maxPoolBackwardGpu(const float* delta, const int* indexes, float* grad, int size)
{
    if (size < 0) throw std::runtime_error("maxPoolBackwardGpu: negative size");
    check(pxe_maxpool_backward(nullptr, delta, indexes, grad, (std::size_t)size), "maxPoolBackwardGpu");
}

PXE_EXPORT void constrainGpu(int n, float alpha, float* x)
{
    if (n < 0) throw std::runtime_error("constrainGpu: negative size");
    check(pxe_constrain(nullptr, x, (std::size_t)n, alpha), "constrainGpu");
}

PXE_EXPORT void mulGpu(int n, float* x, float* y)
{
    if (n < 0) throw std::runtime_error("mulGpu: negative size");
    check(pxe_mul(nullptr, x, y, (std::size_t)n), "mulGpu");
}

PXE_EXPORT void randomGpu(float* ptr, std::size_t n, float a, float b)
{
    check(pxe_random_uniform(nullptr, ptr, n, a, b), "randomGpu");
}

PXE_EXPORT void randomNormalGpu(float* ptr, std::size_t n, float mean, float stddev)
{
    check(pxe_random_normal(nullptr, ptr, n, mean, stddev), "randomNormalGpu");
}

PXE_EXPORT void yoloLossGpu(const float* output, float* delta, const float* truths, const int* truthCounts, int maxTruth,
                            const int* assignedClasses, const int* assignedAnchors, const float* assignedBoxes,
                            const int* masks, const float* anchors, float* stats, float* cost, int batch, int maskCount,
                            int anchorCount, int classes, int width, int height, int networkWidth, int networkHeight,
                            float ignoreThreshold, float truthThreshold, float coordScale, float objectScale,
                            float noObjectScale, float classScale)
{
    (void)anchorCount;
    pxe_yolo_loss_desc d{};
    d.output = output; d.delta = delta; d.truths = truths; d.truth_counts = truthCounts; d.max_truth = maxTruth;
    d.assigned_classes = assignedClasses; d.assigned_anchors = assignedAnchors; d.assigned_boxes = assignedBoxes;
    d.masks = masks; d.anchors = anchors; d.stats = stats; d.cost = cost;
    d.batch = batch; d.mask_count = maskCount; d.classes = classes; d.width = width; d.height = height;
    d.network_width = networkWidth; d.network_height = networkHeight;
    d.ignore_threshold = ignoreThreshold; d.truth_threshold = truthThreshold; d.coord_scale = coordScale;
    d.object_scale = objectScale; d.no_object_scale = noObjectScale; d.class_scale = classScale;
    check(pxe_yolo_loss(nullptr, &d), "yoloLossGpu");
}

PXE_EXPORT void centerNetLossGpu(const float* output, float* delta, const float* targetHeatmap, const float* targetSize,
                                 const float* targetOffset, const float* targetMask, float* costs, int batch,
                                 int classes, int area, float normalizer, float focalAlpha, float focalBeta,
                                 float sizeWeight)
{
    check(pxe_centernet_loss(nullptr, output, delta, targetHeatmap, targetSize, targetOffset, targetMask, costs, batch,
                             classes, area, normalizer, focalAlpha, focalBeta, sizeWeight), "centerNetLossGpu");
}

PXE_EXPORT void adamGpu(int n, float* x, float* m, float* v, float beta1, float beta2, float rate, float eps, int t)
{
    if (n < 0) throw std::runtime_error("adamGpu: negative size");
    check(pxe_adam_update(nullptr, (std::size_t)n, x, m, v, beta1, beta2, rate, eps, t), "adamGpu");
}

PXE_EXPORT void softmaxCrossEntropy(int n, const float* pred, const float* truth, float* delta, float* error)
{
    if (n < 0) throw std::runtime_error("softmaxCrossEntropy: negative size");
    check(pxe_softmax_cross_entropy(nullptr, (std::size_t)n, pred, truth, delta, error), "softmaxCrossEntropy");
}

// Launch grid for n threads in blocks of 512: one row of blocks up to 65535, a near-square arrangement beyond
// (src/CudaUtils.cu:28-43).  The second dimension is what keeps launches of more than 33.5 M threads legal.
PXE_EXPORT dim3 cudaGridsize(std::uint32_t n)
{
    constexpr std::uint32_t kBlock = 512;
    const std::uint32_t blocks = (n - 1) / kBlock + 1;
    std::uint32_t x = blocks, y = 1;
    if (x > 65535) {
        x = (std::uint32_t)ceil(sqrt((double)blocks));
        y = (n - 1) / (x * kBlock) + 1;
    }
    return dim3(x, y, 1);
}

}  // namespace px
