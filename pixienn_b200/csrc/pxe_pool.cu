// Max pooling (px::maxPoolForwardGpu, src/MaxPoolKernels.cu:10-59) and the SPP block
// (stride-1 pools of one input with several kernel sizes) as single-read kernels.
//
// Semantics kept bit for bit: output extent (in + padding - kernel)/stride + 1, window origin
// -padding/2 (C truncation), taps outside the input are skipped, the first tap is always taken
// and later taps replace it only when strictly greater (so the first maximum wins and a NaN in
// the first tap sticks), the index is the flat position in a dense [B,C,H,W] input.
#include "pxe_common.cuh"

namespace pxe {
namespace {

constexpr int kThreads = 256;

struct PoolParams {
    const float* x; float* y; int* idx;
    long long xbs, ybs;
    int C, H, W, OH, OW;
    int kernel, stride, offset;
    uint32_t total;                  // outputs in this launch
    FastDiv div_ow, div_oh, div_c;
};

template <bool WITH_INDEX>
__global__ void __launch_bounds__(kThreads)
maxpool_kernel(const PoolParams p)
{
    for (uint32_t o = blockIdx.x * kThreads + threadIdx.x; o < p.total; o += gridDim.x * kThreads) {
        uint32_t t, ow, oh, c, b;
        p.div_ow.divmod(o, t, ow);
        p.div_oh.divmod(t, t, oh);
        p.div_c.divmod(t, b, c);
        const float* plane = p.x + (long long)b * p.xbs + (long long)c * p.H * p.W;
        const int y0 = p.offset + (int)oh * p.stride;
        const int x0 = p.offset + (int)ow * p.stride;
        float best = -FLT_MAX;
        int best_idx = -1;
        for (int ky = 0; ky < p.kernel; ++ky) {
            const int iy = y0 + ky;
            if (iy < 0 || iy >= p.H) continue;
            for (int kx = 0; kx < p.kernel; ++kx) {
                const int ix = x0 + kx;
                if (ix < 0 || ix >= p.W) continue;
                const float v = plane[iy * p.W + ix];
                if (best_idx < 0 || v > best) {
                    best = v;
                    best_idx = ix + p.W * (iy + p.H * ((int)c + p.C * (int)b));
                }
            }
        }
        p.y[(long long)b * p.ybs + ((long long)c * p.OH + oh) * p.OW + ow] = best;
        if (WITH_INDEX) p.idx[((long long)b * p.C + c) * p.OH * p.OW + (long long)oh * p.OW + ow] = best_idx;
    }
}

// ---------------------------------------------------------------------------------------------
// SPP: one block per (image, channel) plane.  The plane is staged in shared memory once and every
// requested stride-1 pool is evaluated from it, each result going to its own destination
// (typically a channel slot of the concat buffer the following route layer would have built).
// ---------------------------------------------------------------------------------------------
constexpr int kMaxPools = 4;

struct SppParams {
    const float* x; long long xbs;
    int C, H, W;
    int n_pools;
    int kernel[kMaxPools];
    int offset[kMaxPools];
    float* y[kMaxPools];
    long long ybs[kMaxPools];
    // optional conv epilogue applied while the plane is staged (pxe_spp_epilogue): v = act(a[c]*v + b[c]),
    // also stored to yid (the identity slot of the SPP concat) when that is set
    const float* a; const float* b; int act;
    float* yid; long long yidbs;
};

// the activations exactly as the fused epilogue kernels evaluate them (fast-math forms)
__device__ __forceinline__ float activate_fast_dyn(int act, float x)
{
    switch (act) {
    case PXE_ACT_LEAKY: return activate<PXE_ACT_LEAKY, true>(x);
    case PXE_ACT_LOGGY: return activate<PXE_ACT_LOGGY, true>(x);
    case PXE_ACT_LOGISTIC: return activate<PXE_ACT_LOGISTIC, true>(x);
    case PXE_ACT_MISH: return activate<PXE_ACT_MISH, true>(x);
    case PXE_ACT_RELU: return activate<PXE_ACT_RELU, true>(x);
    case PXE_ACT_SOFTPLUS: return activate<PXE_ACT_SOFTPLUS, true>(x);
    case PXE_ACT_SWISH: return activate<PXE_ACT_SWISH, true>(x);
    case PXE_ACT_TANH: return activate<PXE_ACT_TANH, true>(x);
    default: return x;
    }
}

// A k x k maximum is the maximum over rows of the k-wide row maxima: each pool runs as a row pass into a second
// shared-memory plane and a column pass over it, 2k reads per output instead of k*k (54 instead of 275 for the
// 5 / 9 / 13 block).  The reference's scan (src/MaxPoolKernels.cu:26-40: the first tap is taken as it is, a later
// tap replaces it only when strictly greater) is reproduced exactly: both passes ignore NaNs the way "v > best"
// does, and a window whose FIRST tap is a NaN yields that NaN, as the scan would.
__global__ void __launch_bounds__(kThreads)
spp_kernel(const SppParams p)
{
    extern __shared__ float tile[];
    const int plane = blockIdx.x;
    const int b = plane / p.C, c = plane - b * p.C;
    const int HW = p.H * p.W;
    float* rowmax = tile + HW;
    const float* src = p.x + (long long)b * p.xbs + (long long)c * HW;
    if (p.a || p.act != PXE_ACT_LINEAR || p.yid) {
        const float ca = p.a ? p.a[c] : 1.0f, cb = p.a ? p.b[c] : 0.0f;
        float* yid = p.yid ? p.yid + (long long)b * p.yidbs + (long long)c * HW : nullptr;
        for (int i = threadIdx.x; i < HW; i += kThreads) {
            float v = src[i];
            if (p.a) v = fmaf(ca, v, cb);
            v = activate_fast_dyn(p.act, v);
            tile[i] = v;
            if (yid) yid[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < HW; i += kThreads) tile[i] = src[i];
    }
    __syncthreads();
    for (int k = 0; k < p.n_pools; ++k) {
        const int K = p.kernel[k], off = p.offset[k];
        for (int i = threadIdx.x; i < HW; i += kThreads) {
            const int oy = i / p.W, ox = i - oy * p.W;
            const int xa = ox + off < 0 ? 0 : ox + off;
            const int xb = ox + off + K < p.W ? ox + off + K : p.W;
            float m = -INFINITY;
            for (int ix = xa; ix < xb; ++ix) {
                const float v = tile[oy * p.W + ix];
                m = v > m ? v : m;
            }
            rowmax[i] = m;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < HW; i += kThreads) {
            const int oy = i / p.W, ox = i - oy * p.W;
            const int ya = oy + off < 0 ? 0 : oy + off;
            const int yb = oy + off + K < p.H ? oy + off + K : p.H;
            const int xa = ox + off < 0 ? 0 : ox + off;
            float m = -INFINITY;
            for (int iy = ya; iy < yb; ++iy) {
                const float v = rowmax[iy * p.W + ox];
                m = v > m ? v : m;
            }
            const float first = tile[ya * p.W + xa];
            if (first != first) m = first;
            p.y[k][(long long)b * p.ybs[k] + (long long)c * HW + i] = m;
        }
        __syncthreads();
    }
}

// Global average pool (include/AvgPoolLayer.h:66-87; cuDNN average pooling over the whole plane on the CUDA
// path, include/cuda/AvgPoolLayer.h:35-75): one warp per (image, channel) plane, lanes stride the plane,
// shuffle reduction, one division by max(1, H*W).  The reference's CPU loop adds the plane's values in index
// order; the tree order here differs from it by rounding only.
__global__ void __launch_bounds__(256)
avgpool_kernel(const float* x, long long xbs, float* y, long long ybs, int batch, int channels, int area)
{
    const int lane = threadIdx.x & 31;
    const long long plane = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (plane >= (long long)batch * channels) return;
    const int b = (int)(plane / channels), c = (int)(plane - (long long)b * channels);
    const float* src = x + (long long)b * xbs + (long long)c * area;
    float sum = 0.0f;
    for (int i = lane; i < area; i += 32) sum += src[i];
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) y[(long long)b * ybs + c] = sum / (float)(area > 1 ? area : 1);
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" int pxe_maxpool_out_dim(int in, int kernel, int stride, int padding)
{
    if (stride <= 0) return 0;
    return (in + padding - kernel) / stride + 1;     // include/MaxPoolLayer.h:61-62
}

extern "C" int pxe_maxpool(pxe_stream_t stream, const float* x, long long x_batch_stride, float* y,
                           long long y_batch_stride, int* indexes, int batch, int channels, int height,
                           int width, int kernel, int stride, int padding)
{
    PXE_REQUIRE(x && y, "maxpool: null pointer");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0, "maxpool: non-positive shape");
    PXE_REQUIRE(kernel > 0 && stride > 0 && padding >= 0, "maxpool: bad kernel/stride/padding %d/%d/%d", kernel, stride, padding);
    const int oh = pxe_maxpool_out_dim(height, kernel, stride, padding);
    const int ow = pxe_maxpool_out_dim(width, kernel, stride, padding);
    PXE_REQUIRE(oh > 0 && ow > 0, "maxpool: empty output %dx%d", oh, ow);
    const long long chw = (long long)channels * height * width, ochw = (long long)channels * oh * ow;
    PXE_REQUIRE(x_batch_stride == 0 || x_batch_stride >= chw, "maxpool: x_batch_stride too small");
    PXE_REQUIRE(y_batch_stride == 0 || y_batch_stride >= ochw, "maxpool: y_batch_stride too small");
    PXE_REQUIRE((long long)batch * chw < (1LL << 31), "maxpool: int32 argmax indices need fewer than 2^31 input elements");

    // the common 2x2 / stride 2 case runs through the vectorised pooled-store path
    if (kernel == 2 && stride == 2 && padding <= 1 && !indexes) {
        pxe_epilogue_desc d{};
        d.x = x; d.x_batch_stride = x_batch_stride;
        d.batch = batch; d.channels = channels; d.height = height; d.width = width;
        d.act = PXE_ACT_LINEAR;
        d.pool_kernel = 2; d.pool_stride = 2; d.pool_padding = padding;
        d.y_pool = y; d.y_pool_batch_stride = y_batch_stride;
        return pxe_conv_epilogue(stream, &d);
    }

    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    PoolParams p{};
    p.x = x; p.y = y; p.idx = indexes;
    p.xbs = x_batch_stride ? x_batch_stride : chw;
    p.ybs = y_batch_stride ? y_batch_stride : ochw;
    p.C = channels; p.H = height; p.W = width; p.OH = oh; p.OW = ow;
    p.kernel = kernel; p.stride = stride; p.offset = -padding / 2;
    PXE_REQUIRE((long long)batch * ochw < (1LL << 32), "maxpool: too many outputs for one launch");
    p.total = (uint32_t)((long long)batch * ochw);
    p.div_ow = FastDiv((uint32_t)ow); p.div_oh = FastDiv((uint32_t)oh); p.div_c = FastDiv((uint32_t)channels);
    unsigned grid = grid_for(p.total, kThreads, di.sm_count, 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (indexes) maxpool_kernel<true><<<grid, kThreads, 0, s>>>(p);
    else maxpool_kernel<false><<<grid, kThreads, 0, s>>>(p);
    PXE_LAUNCH_OK("maxpool_kernel");
    return PXE_OK;
}

namespace {
int spp_launch(pxe_stream_t stream, const float* x, long long x_batch_stride, int batch, int channels,
               int height, int width, int n_pools, const int* kernels, float* const* ys,
               const long long* y_batch_strides, const float* a, const float* b, int act, float* y_identity,
               long long y_identity_batch_stride, bool fused)
{
    PXE_REQUIRE(x && kernels && ys && y_batch_strides, "spp: null pointer");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0, "spp: non-positive shape");
    PXE_REQUIRE(n_pools > 0 && n_pools <= kMaxPools, "spp: n_pools %d outside 1..%d", n_pools, kMaxPools);
    const long long chw = (long long)channels * height * width;
    PXE_REQUIRE(x_batch_stride == 0 || x_batch_stride >= chw, "spp: x_batch_stride too small");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    SppParams p{};
    p.x = x; p.xbs = x_batch_stride ? x_batch_stride : chw;
    p.C = channels; p.H = height; p.W = width; p.n_pools = n_pools;
    p.a = a; p.b = b; p.act = act; p.yid = y_identity;
    p.yidbs = y_identity_batch_stride ? y_identity_batch_stride : chw;
    for (int k = 0; k < n_pools; ++k) {
        PXE_REQUIRE(kernels[k] > 0 && ys[k] != nullptr, "spp: bad pool %d", k);
        PXE_REQUIRE(y_batch_strides[k] == 0 || y_batch_strides[k] >= chw, "spp: y_batch_stride %d too small", k);
        p.kernel[k] = kernels[k];
        p.offset[k] = -(kernels[k] - 1) / 2;           // default padding kernel-1, origin -padding/2
        p.y[k] = ys[k];
        p.ybs[k] = y_batch_strides[k] ? y_batch_strides[k] : chw;
    }
    const size_t smem = 2 * (size_t)height * width * sizeof(float);      // the plane and its row maxima
    if (smem > 48 * 1024 || (long long)batch * channels > 0x7fffffffLL) {
        if (fused)
            return set_error(PXE_ERR_UNSUPPORTED, "spp_epilogue: a %d x %d plane does not fit shared memory; run "
                             "pxe_conv_epilogue and pxe_spp", height, width);
        // plane too large to stage: one generic stride-1 pool per kernel size
        for (int k = 0; k < n_pools; ++k) {
            rc = pxe_maxpool(stream, x, x_batch_stride, ys[k], y_batch_strides[k], nullptr, batch, channels,
                             height, width, kernels[k], 1, kernels[k] - 1);
            if (rc != PXE_OK) return rc;
        }
        return PXE_OK;
    }
    spp_kernel<<<(unsigned)(batch * channels), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
    PXE_LAUNCH_OK("spp_kernel");
    return PXE_OK;
}
}  // namespace

extern "C" int pxe_spp(pxe_stream_t stream, const float* x, long long x_batch_stride, int batch, int channels,
                       int height, int width, int n_pools, const int* kernels, float* const* ys,
                       const long long* y_batch_strides)
{
    return spp_launch(stream, x, x_batch_stride, batch, channels, height, width, n_pools, kernels, ys, y_batch_strides,
                      nullptr, nullptr, PXE_ACT_LINEAR, nullptr, 0, false);
}

extern "C" int pxe_spp_epilogue(pxe_stream_t stream, const float* x, long long x_batch_stride, int batch, int channels,
                                int height, int width, const float* a, const float* b, int act, float* y_identity,
                                long long y_identity_batch_stride, int n_pools, const int* kernels, float* const* ys,
                                const long long* y_batch_strides)
{
    PXE_REQUIRE((a == nullptr) == (b == nullptr), "spp_epilogue: a and b come together");
    PXE_REQUIRE(valid_activation(act), "spp_epilogue: unknown activation %d", act);
    const long long chw = (long long)channels * height * width;
    PXE_REQUIRE(y_identity_batch_stride == 0 || y_identity_batch_stride >= chw, "spp_epilogue: y_identity_batch_stride too small");
    return spp_launch(stream, x, x_batch_stride, batch, channels, height, width, n_pools, kernels, ys, y_batch_strides,
                      a, b, act, y_identity, y_identity_batch_stride, true);
}

extern "C" int pxe_avgpool(pxe_stream_t stream, const float* x, long long x_batch_stride, float* y,
                           long long y_batch_stride, int batch, int channels, int height, int width)
{
    PXE_REQUIRE(x && y, "avgpool: null pointer");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0, "avgpool: non-positive shape");
    const long long area = (long long)height * width, chw = area * channels;
    PXE_REQUIRE(area <= 0x7fffffffLL, "avgpool: plane too large");
    PXE_REQUIRE(x_batch_stride == 0 || x_batch_stride >= chw, "avgpool: x_batch_stride too small");
    PXE_REQUIRE(y_batch_stride == 0 || y_batch_stride >= channels, "avgpool: y_batch_stride too small");
    const long long planes = (long long)batch * channels;
    PXE_REQUIRE((planes + 7) / 8 <= 0x7fffffffLL, "avgpool: too many planes");
    avgpool_kernel<<<(unsigned)((planes + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, x_batch_stride ? x_batch_stride : chw, y, y_batch_stride ? y_batch_stride : channels, batch, channels, (int)area);
    PXE_LAUNCH_OK("avgpool_kernel");
    return PXE_OK;
}
