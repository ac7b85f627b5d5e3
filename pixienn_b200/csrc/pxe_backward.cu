// The element-wise kernels PixieNN's CUDA layers call on the way back through the graph and when they set
// weights up: activation gradients, bias gradients, max-pool and upsample backward, gradient clipping, the
// element-wise product Adam uses, and the uniform / normal fills.  They replace
//   px::gradient            src/Activation.cu:84-92, 135-143 (functors: include/Activation.h:40-228)
//   px::backwardBiasGpu     src/BiasKernels.cu:39-111
//   px::maxPoolBackwardGpu  src/MaxPoolKernels.cu:45-49, 61-65
//   px::upsampleGpu (forward == 0)   src/UpsampleKernels.cu:25-63
//   px::constrainGpu, px::mulGpu, px::randomGpu, px::randomNormalGpu, px::cudaGridsize   src/CudaUtils.cu:28-146
// so that a build of the reference can drop those source files and link this library instead.  None of them
// synchronises the device (the reference's backwardBiasGpu and upsampleGpu do).
//
// Sums: the reference accumulates with atomicAdd (max-pool and upsample backward) or in a fixed 512-way split
// (bias gradient), so its own results depend on thread timing in the last bits.  Here every sum is taken in a
// fixed order -- the same call gives the same bits every time -- and agrees with the reference to rounding.
#include <stdint.h>

#include "pxe_common.cuh"

namespace pxe {
namespace {

// ---------------------------------------------------------------- activation gradients
// delta[i] *= f'(x[i]) with the reference functors' expressions (precise math library).
__device__ __forceinline__ float softplus_apply(float x)
{
    if (x > 20.0f) return x;
    if (x < -20.0f) return expf(x);
    return logf(expf(x) + 1.0f);
}
__device__ __forceinline__ float softplus_gradient(float x)
{
    if (x > 20.0f) return 1.0f;
    if (x < -20.0f) return expf(x);
    return 1.0f / (1.0f + expf(-x));
}

template <int ACT>
__device__ __forceinline__ float act_gradient(float x)
{
    if (ACT == PXE_ACT_LEAKY) return x > 0.0f ? 1.0f : 0.1f;
    if (ACT == PXE_ACT_LINEAR) return 1.0f;
    if (ACT == PXE_ACT_LOGGY) { const float y = (x + 1.0f) / 2.0f; return 2.0f * (1.0f - y) * y; }
    if (ACT == PXE_ACT_LOGISTIC) { const float y = 1.0f / (1.0f + expf(-x)); return y * (1.0f - y); }
    if (ACT == PXE_ACT_SOFTPLUS) return softplus_gradient(x);
    if (ACT == PXE_ACT_MISH) {
        const float sp = softplus_apply(x), grad_sp = softplus_gradient(x);
        const float tsp = tanhf(sp);
        const float grad_tsp = (1.0f - tsp * tsp) * grad_sp;
        return x * grad_tsp + tsp;
    }
    if (ACT == PXE_ACT_RELU) return x > 0.0f ? 1.0f : 0.0f;
    if (ACT == PXE_ACT_SWISH) { const float val = 1.0f / (1.0f + expf(-1.0f * x)); return x * val + 1.0f * val * (1.0f - x * val); }
    if (ACT == PXE_ACT_TANH) { const float y = tanhf(x); return 1.0f - y * y; }
    return 1.0f;
}

template <int ACT, bool VEC>
__global__ void __launch_bounds__(256)
gradient_kernel(const float* __restrict__ x, float* __restrict__ delta, size_t n)
{
    const size_t stride = (size_t)gridDim.x * 256;
    if (VEC) {
        const size_t n4 = n >> 2;
        for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
            const float4 xv = gld(reinterpret_cast<const float4*>(x) + i);
            float4 d = gld(reinterpret_cast<float4*>(delta) + i);
            d.x *= act_gradient<ACT>(xv.x); d.y *= act_gradient<ACT>(xv.y);
            d.z *= act_gradient<ACT>(xv.z); d.w *= act_gradient<ACT>(xv.w);
            gst(reinterpret_cast<float4*>(delta) + i, d);
        }
        for (size_t i = (n4 << 2) + (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride)
            gst(delta + i, gld(delta + i) * (act_gradient<ACT>(gld(x + i))));
    } else {
        for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) gst(delta + i, gld(delta + i) * (act_gradient<ACT>(gld(x + i))));
    }
}

template <int ACT>
int launch_gradient(cudaStream_t s, const float* x, float* delta, size_t n, int sm_count)
{
    const bool vec = aligned16(x) && aligned16(delta);
    const unsigned grid = grid_for((long long)((n + 3) / 4), 256, sm_count, 16);
    if (vec) gradient_kernel<ACT, true><<<grid, 256, 0, s>>>(x, delta, n);
    else gradient_kernel<ACT, false><<<grid, 256, 0, s>>>(x, delta, n);
    PXE_LAUNCH_OK("gradient_kernel");
    return PXE_OK;
}

// ---------------------------------------------------------------- bias gradient
// bias_updates[f] += sum over images and positions of delta[b, f, :].  One block per filter; every thread sums
// its strided share image by image, the block combines the 256 partial sums in a fixed tree.
__global__ void __launch_bounds__(256)
backward_bias_kernel(float* bias_updates, const float* __restrict__ delta, int batch, int n, int size)
{
    __shared__ float part[256];
    const int f = blockIdx.x;
    float sum = 0.0f;
    for (int b = 0; b < batch; ++b) {
        const float* row = delta + ((size_t)b * n + f) * size;
        for (int i = threadIdx.x; i < size; i += 256) sum += gld(row + i);
    }
    part[threadIdx.x] = sum;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) gst(bias_updates + f, gld(bias_updates + f) + part[0]);
}

// size == 1 (connected layers): one thread per output, images summed in order (src/BiasKernels.cu:39-53).
__global__ void __launch_bounds__(256)
backward_bias_conn_kernel(float* bias_updates, const float* __restrict__ delta, int batch, int n)
{
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float sum = 0.0f;
    for (int b = 0; b < batch; ++b) sum += gld(delta + ((size_t)b * n + i));
    gst(bias_updates + i, gld(bias_updates + i) + sum);
}

// ---------------------------------------------------------------- max-pool backward
// grad[indexes[i]] += delta[i].  Two outputs can name the same input only when the windows overlap
// (stride < kernel); the adds go through atomicAdd as in the reference (src/MaxPoolKernels.cu:45-49).
__global__ void __launch_bounds__(256)
maxpool_backward_kernel(const float* __restrict__ delta, const int* __restrict__ indexes, float* grad, size_t size)
{
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < size; i += (size_t)gridDim.x * 256) {
        const int at = gld(indexes + i);
        if (at >= 0 && gcheck(grad + at)) atomicAdd(grad + at, gld(delta + i));
    }
}

// ---------------------------------------------------------------- upsample backward
// acc[b, c, y, x] += sum over the stride x stride outputs of that input of scale * out[...], rows then columns.
// One thread per input element: no atomics, the same bits on every run (the reference adds the stride^2 terms
// with atomicAdd in whatever order its threads arrive, src/UpsampleKernels.cu:25-52).
__global__ void __launch_bounds__(256)
upsample_backward_kernel(float* acc, const float* __restrict__ out, size_t n_in, int w, int h, int stride, float scale)
{
    const int ow = w * stride;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n_in; i += (size_t)gridDim.x * 256) {
        const int x = (int)(i % w);
        const size_t r = i / w;
        const int y = (int)(r % h);
        const size_t plane = r / h;                                  // b * c + channel
        const float* src = out + (plane * h * stride + (size_t)y * stride) * ow + (size_t)x * stride;
        float sum = 0.0f;
        for (int dy = 0; dy < stride; ++dy)
            for (int dx = 0; dx < stride; ++dx) sum += scale * gld(src + ((size_t)dy * ow + dx));
        gst(acc + i, gld(acc + i) + sum);
    }
}

// ---------------------------------------------------------------- clip / product
__global__ void __launch_bounds__(256)
constrain_kernel(float* x, size_t n, float alpha)
{
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256)
        gst(x + i, fminf(alpha, fmaxf(-alpha, gld(x + i))));                    // src/CudaUtils.cu:122-129
}

__global__ void __launch_bounds__(256)
mul_kernel(const float* __restrict__ x, float* y, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) gst(y + i, gld(x + i) * gld(y + i));
}

// ---------------------------------------------------------------- random fills
// The reference draws element i from thrust::default_random_engine (the minimal-standard generator,
// x <- 48271 x mod 2^31-1, seed 1) advanced i steps (src/CudaUtils.cu:53-60, 103-109).  The state after i + 1
// steps is 48271^(i+1) mod (2^31-1): a modular power, so every element is independent of the others, as there.
__device__ __forceinline__ uint32_t minstd_after(uint64_t steps)
{
    const uint64_t M = 2147483647ull;
    uint64_t result = 1, base = 48271ull;
    while (steps) {
        if (steps & 1ull) result = result * base % M;
        base = base * base % M;
        steps >>= 1;
    }
    return (uint32_t)result;
}

// Uniform on [a, b): the engine's value mapped to [0, 1) as (x - 1) / 2^31 (its range is 1 .. 2^31-2).
__global__ void __launch_bounds__(256)
random_uniform_kernel(float* out, size_t n, float a, float b)
{
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const float u = (float)(minstd_after(i + 1) - 1u) / 2147483648.0f;
        gst(out + i, u * (b - a) + a);
    }
}

// Normal(mean, stddev) by inversion of the same uniform: mean + stddev * sqrt(2) * erfinv(2u - 1), with u taken at
// the centre of the engine's step so that it never reaches 0 or 1.
__global__ void __launch_bounds__(256)
random_normal_kernel(float* out, size_t n, float mean, float stddev)
{
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const float u = ((float)(minstd_after(i + 1) - 1u) + 0.5f) / 2147483648.0f;
        gst(out + i, mean + stddev * 1.41421356f * erfinvf(2.0f * u - 1.0f));
    }
}

// ---------------------------------------------------------------- Adam step, softmax cross-entropy
// adamKernel (src/Adam.cu:26-38): x += rate * (m / (1 - beta1^t)) / (sqrt(v / (1 - beta2^t)) + eps), the same
// expressions in the same order; every thread evaluates the two powers itself, as the reference's does.
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ x, const float* __restrict__ m, const float* __restrict__ v, size_t n, float beta1,
            float beta2, float rate, float eps, int t)
{
    const float c1 = 1.0f - powf(beta1, t), c2 = 1.0f - powf(beta2, t);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float mhat = gld(m + i) / c1;
        const float vhat = gld(v + i) / c2;
        gst(x + i, gld(x + i) + (rate * mhat / (sqrtf(vhat) + eps)));
    }
}

// softmaxCrossEntropyKernel (src/SoftmaxKernel.cu:25-39): error[i] = truth[i] ? -log(pred[i] + 1e-9) : 0,
// delta[i] = truth[i] - pred[i].  (The reference has every thread loop over all n elements; the values are these.)
__global__ void __launch_bounds__(256)
softmax_cross_entropy_kernel(const float* __restrict__ pred, const float* __restrict__ truth, float* __restrict__ delta,
                             float* __restrict__ error, size_t n)
{
    constexpr float epsilon = 1e-9f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float t = gld(truth + i), p = gld(pred + i);
        gst(error + i, t ? -logf(p + epsilon) : 0.0f);
        gst(delta + i, t - p);
    }
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" int pxe_activation_gradient(pxe_stream_t stream, int act, const float* x, size_t n, float* delta)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(x && delta, "activation_gradient: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (act) {
    case PXE_ACT_LEAKY: return launch_gradient<PXE_ACT_LEAKY>(s, x, delta, n, di.sm_count);
    case PXE_ACT_LINEAR: return PXE_OK;                              // delta *= 1
    case PXE_ACT_LOGGY: return launch_gradient<PXE_ACT_LOGGY>(s, x, delta, n, di.sm_count);
    case PXE_ACT_LOGISTIC: return launch_gradient<PXE_ACT_LOGISTIC>(s, x, delta, n, di.sm_count);
    case PXE_ACT_MISH: return launch_gradient<PXE_ACT_MISH>(s, x, delta, n, di.sm_count);
    case PXE_ACT_RELU: return launch_gradient<PXE_ACT_RELU>(s, x, delta, n, di.sm_count);
    case PXE_ACT_SOFTPLUS: return launch_gradient<PXE_ACT_SOFTPLUS>(s, x, delta, n, di.sm_count);
    case PXE_ACT_SWISH: return launch_gradient<PXE_ACT_SWISH>(s, x, delta, n, di.sm_count);
    case PXE_ACT_TANH: return launch_gradient<PXE_ACT_TANH>(s, x, delta, n, di.sm_count);
    default: return set_error(PXE_ERR_BAD_ARG, "activation_gradient: unknown activation %d", act);
    }
}

extern "C" int pxe_backward_bias(pxe_stream_t stream, float* bias_updates, const float* delta, int batch, int n, int size)
{
    PXE_REQUIRE(bias_updates && delta, "backward_bias: null pointer");
    PXE_REQUIRE(batch > 0 && n > 0 && size > 0, "backward_bias: non-positive shape");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (size == 1) {
        backward_bias_conn_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(bias_updates, delta, batch, n);
        PXE_LAUNCH_OK("backward_bias_conn_kernel");
    } else {
        backward_bias_kernel<<<(unsigned)n, 256, 0, s>>>(bias_updates, delta, batch, n, size);
        PXE_LAUNCH_OK("backward_bias_kernel");
    }
    return PXE_OK;
}

extern "C" int pxe_maxpool_backward(pxe_stream_t stream, const float* delta, const int* indexes, float* grad, size_t size)
{
    if (size == 0) return PXE_OK;
    PXE_REQUIRE(delta && indexes && grad, "maxpool_backward: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    maxpool_backward_kernel<<<grid_for((long long)size, 256, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        delta, indexes, grad, size);
    PXE_LAUNCH_OK("maxpool_backward_kernel");
    return PXE_OK;
}

extern "C" int pxe_upsample_backward(pxe_stream_t stream, float* acc, const float* out, int batch, int channels, int height,
                                     int width, int stride, float scale)
{
    PXE_REQUIRE(acc && out, "upsample_backward: null pointer");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0 && stride > 0, "upsample_backward: non-positive shape");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    const size_t n_in = (size_t)batch * channels * height * width;
    upsample_backward_kernel<<<grid_for((long long)n_in, 256, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        acc, out, n_in, width, height, stride, scale);
    PXE_LAUNCH_OK("upsample_backward_kernel");
    return PXE_OK;
}

extern "C" int pxe_constrain(pxe_stream_t stream, float* x, size_t n, float alpha)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(x != nullptr, "constrain: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    constrain_kernel<<<grid_for((long long)n, 256, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, n, alpha);
    PXE_LAUNCH_OK("constrain_kernel");
    return PXE_OK;
}

extern "C" int pxe_mul(pxe_stream_t stream, const float* x, float* y, size_t n)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(x && y, "mul: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    mul_kernel<<<grid_for((long long)n, 256, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n);
    PXE_LAUNCH_OK("mul_kernel");
    return PXE_OK;
}

extern "C" int pxe_random_uniform(pxe_stream_t stream, float* out, size_t n, float a, float b)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(out != nullptr, "random_uniform: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    random_uniform_kernel<<<grid_for((long long)n, 256, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(out, n, a, b);
    PXE_LAUNCH_OK("random_uniform_kernel");
    return PXE_OK;
}

extern "C" int pxe_random_normal(pxe_stream_t stream, float* out, size_t n, float mean, float stddev)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(out != nullptr, "random_normal: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    random_normal_kernel<<<grid_for((long long)n, 256, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(out, n, mean, stddev);
    PXE_LAUNCH_OK("random_normal_kernel");
    return PXE_OK;
}

extern "C" int pxe_adam_update(pxe_stream_t stream, size_t n, float* x, const float* m, const float* v, float beta1,
                               float beta2, float rate, float eps, int t)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(x && m && v, "adam_update: null pointer");
    PXE_REQUIRE(t >= 1, "adam_update: step %d (the first step is 1)", t);
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    adam_kernel<<<grid_for((long long)n, 256 * 4, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, m, v, n, beta1, beta2,
                                                                                                            rate, eps, t);
    PXE_LAUNCH_OK("adam_kernel");
    return PXE_OK;
}

extern "C" int pxe_softmax_cross_entropy(pxe_stream_t stream, size_t n, const float* pred, const float* truth, float* delta,
                                         float* error)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(pred && truth && delta && error, "softmax_cross_entropy: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    softmax_cross_entropy_kernel<<<grid_for((long long)n, 256 * 4, di.sm_count, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        pred, truth, delta, error, n);
    PXE_LAUNCH_OK("softmax_cross_entropy_kernel");
    return PXE_OK;
}
