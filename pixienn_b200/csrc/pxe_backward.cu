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
#include <cooperative_groups.h>
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
// bias_updates[f] += sum over images and positions of delta[b, f, :].  A thread-block cluster per filter: its blocks
// take consecutive segments of the filter's planes, every thread sums its strided share image by image, a block
// combines its 256 partial sums in a fixed tree, and the cluster's first block adds the blocks' sums in rank order out
// of their shared memory (distributed shared memory: no scratch buffer, no atomics, the same bits every run).  One
// block per filter, as the reference launches it, leaves a 64-filter layer on 64 of the machine's 148 SMs.
namespace cg = cooperative_groups;

template <bool VEC>
__global__ void __launch_bounds__(256)
backward_bias_kernel(float* bias_updates, const float* __restrict__ delta, int batch, int n, int size, int segment)
{
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned ranks = cluster.num_blocks(), rank = cluster.block_rank();
    __shared__ float part[256];
    __shared__ float block_sum;
    const int f = blockIdx.x / ranks;
    const int lo = (int)rank * segment, hi = min(size, lo + segment);
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    // the segment of every image as one index space, four loads in flight per thread
    const int per_image = hi > lo ? (VEC ? (hi - lo) / 4 : hi - lo) : 0;
    const int total = batch * per_image;                       // the host checks that batch * size fits an int
    const float* base = delta + (size_t)f * size + lo;
    const size_t image_stride = (size_t)n * size;
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * 256) {
        float4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int id = i0 + k * 256;
            v[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (id < total) {
                const int b = id / per_image, i = id - b * per_image;
                if (VEC) v[k] = gld(reinterpret_cast<const float4*>(base + b * image_stride) + i);
                else v[k].x = gld(base + b * image_stride + i);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) { s0 += v[k].x; s1 += v[k].y; s2 += v[k].z; s3 += v[k].w; }
    }
    part[threadIdx.x] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) block_sum = part[0];
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        float total = 0.0f;
        for (unsigned r = 0; r < ranks; ++r) total += *cluster.map_shared_rank(&block_sum, r);
        gst(bias_updates + f, gld(bias_updates + f) + total);
    }
    cluster.sync();                                    // the other blocks' shared memory stays until it has been read
}

// size == 1 (connected layers; the reference: one thread per output, src/BiasKernels.cu:39-53).  A block is 32
// outputs x 8 phases of the batch, a cluster's blocks take consecutive parts of the batch; phases, then blocks, are
// added in a fixed order.
__global__ void __launch_bounds__(256)
backward_bias_conn_kernel(float* bias_updates, const float* __restrict__ delta, int batch, int n, int segment)
{
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned ranks = cluster.num_blocks(), rank = cluster.block_rank();
    __shared__ float part[8][32];
    __shared__ float block_sum[32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int i = (int)(blockIdx.x / ranks) * 32 + tx;
    const int lo = (int)rank * segment, hi = min(batch, lo + segment);
    float sum = 0.0f;
    if (i < n)
        for (int b = lo + ty; b < hi; b += 8) sum += gld(delta + ((size_t)b * n + i));
    part[ty][tx] = sum;
    __syncthreads();
    if (ty == 0) {
        float t = part[0][tx];
        for (int k = 1; k < 8; ++k) t += part[k][tx];
        block_sum[tx] = t;
    }
    cluster.sync();
    if (rank == 0 && ty == 0 && i < n) {
        float total = 0.0f;
        for (unsigned r = 0; r < ranks; ++r) total += *cluster.map_shared_rank(&block_sum[tx], r);
        gst(bias_updates + i, gld(bias_updates + i) + total);
    }
    cluster.sync();
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
// VEC: the tensors are 16-byte aligned, so four elements move per access; the last n % 4 go one by one.
template <bool VEC>
__global__ void __launch_bounds__(256)
constrain_kernel(float* x, size_t n, float alpha)
{
    const size_t stride = (size_t)gridDim.x * 256, first = (size_t)blockIdx.x * 256 + threadIdx.x;
    const size_t n4 = VEC ? n >> 2 : 0;
    for (size_t i = first; i < n4; i += stride) {
        float4 v = gld(reinterpret_cast<const float4*>(x) + i);
        v.x = fminf(alpha, fmaxf(-alpha, v.x)); v.y = fminf(alpha, fmaxf(-alpha, v.y));
        v.z = fminf(alpha, fmaxf(-alpha, v.z)); v.w = fminf(alpha, fmaxf(-alpha, v.w));
        gst(reinterpret_cast<float4*>(x) + i, v);
    }
    for (size_t i = (n4 << 2) + first; i < n; i += stride)
        gst(x + i, fminf(alpha, fmaxf(-alpha, gld(x + i))));                    // src/CudaUtils.cu:122-129
}

template <bool VEC>
__global__ void __launch_bounds__(256)
mul_kernel(const float* __restrict__ x, float* y, size_t n)
{
    const size_t stride = (size_t)gridDim.x * 256, first = (size_t)blockIdx.x * 256 + threadIdx.x;
    const size_t n4 = VEC ? n >> 2 : 0;
    for (size_t i = first; i < n4; i += stride) {
        const float4 a = gld(reinterpret_cast<const float4*>(x) + i);
        float4 b = gld(reinterpret_cast<const float4*>(y) + i);
        b.x = a.x * b.x; b.y = a.y * b.y; b.z = a.z * b.z; b.w = a.w * b.w;
        gst(reinterpret_cast<float4*>(y) + i, b);
    }
    for (size_t i = (n4 << 2) + first; i < n; i += stride) gst(y + i, gld(x + i) * gld(y + i));
}

// ---------------------------------------------------------------- random fills
// The reference draws element i from thrust::default_random_engine (the minimal-standard generator,
// x <- 48271 x mod 2^31-1, seed 1) advanced i steps (src/CudaUtils.cu:53-60, 103-109).  The state after i + 1
// steps is 48271^(i+1) mod (2^31-1): a modular power, so every element is independent of the others, as there.
// a * b mod 2^31-1 for a, b below the modulus: 2^31 = 1 (mod 2^31-1), so the high part of the product folds onto the low
__device__ __forceinline__ uint32_t minstd_mul(uint32_t a, uint32_t b)
{
    const uint64_t M = 2147483647ull;
    const uint64_t p = (uint64_t)a * b;
    uint64_t r = (p & M) + (p >> 31);
    r = (r & M) + (r >> 31);
    return (uint32_t)(r >= M ? r - M : r);
}

__device__ __forceinline__ uint32_t minstd_after(uint64_t steps)
{
    uint32_t result = 1, base = 48271u;
    while (steps) {
        if (steps & 1ull) result = minstd_mul(result, base);
        base = minstd_mul(base, base);
        steps >>= 1;
    }
    return result;
}

// A thread's elements are a whole grid apart: it raises the generator to its first element's power once and then
// jumps from one element to the next with one multiplication by 48271^(grid stride).

// Uniform on [a, b): the engine's value mapped to [0, 1) as (x - 1) / 2^31 (its range is 1 .. 2^31-2).
__global__ void __launch_bounds__(256)
random_uniform_kernel(float* out, size_t n, float a, float b)
{
    const size_t first = (size_t)blockIdx.x * 256 + threadIdx.x, stride = (size_t)gridDim.x * 256;
    if (first >= n) return;
    uint32_t state = minstd_after(first + 1);
    const uint32_t jump = minstd_after(stride);
    for (size_t i = first; i < n; i += stride) {
        const float u = (float)(state - 1u) / 2147483648.0f;
        gst(out + i, u * (b - a) + a);
        state = minstd_mul(state, jump);
    }
}

// Normal(mean, stddev) by inversion of the same uniform: mean + stddev * sqrt(2) * erfinv(2u - 1), with u taken at
// the centre of the engine's step so that it never reaches 0 or 1.
__global__ void __launch_bounds__(256)
random_normal_kernel(float* out, size_t n, float mean, float stddev)
{
    const size_t first = (size_t)blockIdx.x * 256 + threadIdx.x, stride = (size_t)gridDim.x * 256;
    if (first >= n) return;
    uint32_t state = minstd_after(first + 1);
    const uint32_t jump = minstd_after(stride);
    for (size_t i = first; i < n; i += stride) {
        const float u = ((float)(state - 1u) + 0.5f) / 2147483648.0f;
        gst(out + i, mean + stddev * 1.41421356f * erfinvf(2.0f * u - 1.0f));
        state = minstd_mul(state, jump);
    }
}

// ---------------------------------------------------------------- Adam step, softmax cross-entropy
// adamKernel (src/Adam.cu:26-38): x += rate * (m / (1 - beta1^t)) / (sqrt(v / (1 - beta2^t)) + eps), the same
// expressions in the same order; every thread evaluates the two powers itself, as the reference's does.
template <bool VEC>
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ x, const float* __restrict__ m, const float* __restrict__ v, size_t n, float beta1,
            float beta2, float rate, float eps, int t)
{
    const float c1 = 1.0f - powf(beta1, t), c2 = 1.0f - powf(beta2, t);
    const size_t stride = (size_t)gridDim.x * blockDim.x, first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n4 = VEC ? n >> 2 : 0;
    auto step = [&](float xv, float mv, float vv) {
        const float mhat = mv / c1;
        const float vhat = vv / c2;
        return xv + (rate * mhat / (sqrtf(vhat) + eps));
    };
    for (size_t i = first; i < n4; i += stride) {
        const float4 mv = gld(reinterpret_cast<const float4*>(m) + i), vv = gld(reinterpret_cast<const float4*>(v) + i);
        float4 xv = gld(reinterpret_cast<const float4*>(x) + i);
        xv.x = step(xv.x, mv.x, vv.x); xv.y = step(xv.y, mv.y, vv.y); xv.z = step(xv.z, mv.z, vv.z); xv.w = step(xv.w, mv.w, vv.w);
        gst(reinterpret_cast<float4*>(x) + i, xv);
    }
    for (size_t i = (n4 << 2) + first; i < n; i += stride) gst(x + i, step(gld(x + i), gld(m + i), gld(v + i)));
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
    PXE_REQUIRE((long long)batch * size < (1LL << 31), "backward_bias: batch * size = %lld does not fit 31 bits", (long long)batch * size);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // blocks per filter (a cluster, at most 8): enough to put a few blocks on every SM, each with 8192 terms or more
    const long long work = size == 1 ? (long long)batch * 32 : (long long)batch * size;
    const long long groups = size == 1 ? (n + 31) / 32 : n;
    int ranks = 1;
    while (ranks < 8 && groups * ranks < 592 && work / (ranks * 2) >= 8192) ranks *= 2;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ranks; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3((unsigned)(groups * ranks)); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (size == 1) {
        const int segment = (batch + ranks - 1) / ranks;
        PXE_CUDA_OK(cudaLaunchKernelEx(&cfg, backward_bias_conn_kernel, bias_updates, delta, batch, n, segment));
    } else {
        int segment = (size + ranks - 1) / ranks;
        segment = (segment + 3) & ~3;
        const bool vec = size % 4 == 0 && aligned16(delta);
        if (vec) PXE_CUDA_OK(cudaLaunchKernelEx(&cfg, backward_bias_kernel<true>, bias_updates, delta, batch, n, size, segment));
        else PXE_CUDA_OK(cudaLaunchKernelEx(&cfg, backward_bias_kernel<false>, bias_updates, delta, batch, n, size, segment));
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
    const unsigned grid = grid_for((long long)n, 256 * 4, di.sm_count, 16);
    if (aligned16(x)) constrain_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, n, alpha);
    else constrain_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, n, alpha);
    PXE_LAUNCH_OK("constrain_kernel");
    return PXE_OK;
}

extern "C" int pxe_mul(pxe_stream_t stream, const float* x, float* y, size_t n)
{
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(x && y, "mul: null pointer");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    const unsigned grid = grid_for((long long)n, 256 * 4, di.sm_count, 16);
    if (aligned16(x) && aligned16(y)) mul_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n);
    else mul_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n);
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
    const unsigned grid = grid_for((long long)n, 256 * 4, di.sm_count, 16);
    if (aligned16(x) && aligned16(m) && aligned16(v))
        adam_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, m, v, n, beta1, beta2, rate, eps, t);
    else
        adam_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, m, v, n, beta1, beta2, rate, eps, t);
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
