// Data-movement layers between convolutions: nearest-neighbour upsample, shortcut (residual
// add), and route (channel concat).  Each kernel can read from and write to a channel slot of a
// wider buffer (a batch stride larger than C*H*W), which is what removes the reference's
// separate concat copies (include/cuda/RouteLayer.h:21-44).
#include "pxe_common.cuh"

namespace pxe {
namespace {

constexpr int kThreads = 256;

// ------------------------------------------------------------------------------------ upsample
struct UpParams {
    const float* x; float* y;
    long long xbs, ybs;
    int C, H, W, stride;
    float scale;
    uint32_t total;
    FastDiv div_w, div_h, div_c;   // over the unit space (see kernels)
};

// Stride 2, VI input columns per thread (4: float4 in, two float4 per output row;
// 2: float2 in, one float4 per output row; 1: scalar in, one float2 per output row).  out = scale * in, assigned
// (include/UpsampleLayer.h:113; the CUDA kernel's "+=" lands on a zero-filled buffer).
template <int VI>
__global__ void __launch_bounds__(kThreads)
upsample2_vec_kernel(const UpParams p)
{
    const int WV = p.W / VI;
    for (uint32_t u = blockIdx.x * kThreads + threadIdx.x; u < p.total; u += gridDim.x * kThreads) {
        uint32_t t, wv, h, c, b;
        p.div_w.divmod(u, t, wv);
        p.div_h.divmod(t, t, h);
        p.div_c.divmod(t, b, c);
        (void)WV;
        const float* src = p.x + (long long)b * p.xbs + ((long long)c * p.H + h) * p.W + (long long)wv * VI;
        float* dst = p.y + (long long)b * p.ybs + ((long long)c * p.H * 2 + 2 * h) * (p.W * 2) + (long long)wv * VI * 2;
        const int ow = p.W * 2;
        if (VI == 4) {
            float4 v = gldv<float4>(src);
            v.x *= p.scale; v.y *= p.scale; v.z *= p.scale; v.w *= p.scale;
            const float4 lo = make_float4(v.x, v.x, v.y, v.y), hi = make_float4(v.z, v.z, v.w, v.w);
            gstv(dst, lo);
            gstv(dst + 4, hi);
            gstv(dst + ow, lo);
            gstv(dst + ow + 4, hi);
        } else if (VI == 2) {
            float2 v = gldv<float2>(src);
            v.x *= p.scale; v.y *= p.scale;
            const float4 o = make_float4(v.x, v.x, v.y, v.y);
            gstv(dst, o);
            gstv(dst + ow, o);
        } else {
            // odd widths (13, 19): one input element per thread, the output rows are still 8-byte aligned
            const float v = gld(src) * p.scale;
            const float2 o = make_float2(v, v);
            gstv(dst, o);
            gstv(dst + ow, o);
        }
    }
}

// Any stride / alignment: one thread per output element.
__global__ void __launch_bounds__(kThreads)
upsample_scalar_kernel(const UpParams p)
{
    const int OW = p.W * p.stride;
    for (uint32_t o = blockIdx.x * kThreads + threadIdx.x; o < p.total; o += gridDim.x * kThreads) {
        uint32_t t, ow, oh, c, b;
        p.div_w.divmod(o, t, ow);
        p.div_h.divmod(t, t, oh);
        p.div_c.divmod(t, b, c);
        const int ih = (int)oh / p.stride, iw = (int)ow / p.stride;
        const float v = gld(p.x + ((long long)b * p.xbs + ((long long)c * p.H + ih) * p.W + iw));
        gst(p.y + ((long long)b * p.ybs + ((long long)c * p.H * p.stride + oh) * OW + ow), p.scale * v);
    }
}

// ------------------------------------------------------------------------------------ shortcut
// px::shortcutGpu's general index rule (src/ShortcutKernel.cu:25-42) for unequal shapes.
struct ScParams {
    const float* add; float* out;
    int minw, minh, minc, stride, sample, batch, w1, h1, c1, w2, h2, c2;
    float s1, s2;
    uint32_t total;
};

__global__ void __launch_bounds__(kThreads)
shortcut_general_kernel(const ScParams p)
{
    for (uint32_t id0 = blockIdx.x * kThreads + threadIdx.x; id0 < p.total; id0 += gridDim.x * kThreads) {
        uint32_t id = id0;
        const int i = id % p.minw; id /= p.minw;
        const int j = id % p.minh; id /= p.minh;
        const int k = id % p.minc; id /= p.minc;
        const int b = id % p.batch;
        const long long oi = i * p.sample + (long long)p.w2 * (j * p.sample + (long long)p.h2 * (k + (long long)p.c2 * b));
        const long long ai = i * p.stride + (long long)p.w1 * (j * p.stride + (long long)p.h1 * (k + (long long)p.c1 * b));
        gst(p.out + oi, fmaf(p.s1, gld(p.out + oi), p.s2 * gld(p.add + ai)));
    }
}

// ------------------------------------------------------------------------------------ concat
constexpr int kMaxSources = 8;

struct CatParams {
    const float* src[kMaxSources];
    long long sbs[kMaxSources];
    long long len[kMaxSources];       // elements per image of source s (channels*H*W)
    long long dst_off[kMaxSources];   // element offset of the slot inside one output image
    float* y; long long ybs;
    int batch;
    int vec[kMaxSources];             // 1: float4 path valid for this source
};

__global__ void __launch_bounds__(kThreads)
concat_kernel(const CatParams p)
{
    const int s = blockIdx.y;
    const long long len = p.len[s];
    if (p.vec[s]) {
        const long long nv = len / 4;
        const long long total = nv * p.batch;
        for (long long u = (long long)blockIdx.x * kThreads + threadIdx.x; u < total; u += (long long)gridDim.x * kThreads) {
            const long long b = u / nv, r = u - b * nv;
            const float4 v = gldv<float4>(p.src[s] + b * p.sbs[s] + r * 4);
            gstv(p.y + b * p.ybs + p.dst_off[s] + r * 4, v);
        }
    } else {
        const long long total = len * p.batch;
        for (long long u = (long long)blockIdx.x * kThreads + threadIdx.x; u < total; u += (long long)gridDim.x * kThreads) {
            const long long b = u / len, r = u - b * len;
            gst(p.y + (b * p.ybs + p.dst_off[s] + r), gld(p.src[s] + (b * p.sbs[s] + r)));
        }
    }
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" int pxe_upsample(pxe_stream_t stream, const float* x, long long x_batch_stride, float* y,
                            long long y_batch_stride, int batch, int channels, int height, int width,
                            int stride, float scale)
{
    PXE_REQUIRE(x && y, "upsample: null pointer");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0 && stride > 0, "upsample: non-positive shape");
    const long long chw = (long long)channels * height * width;
    const long long ochw = chw * stride * stride;
    PXE_REQUIRE(x_batch_stride == 0 || x_batch_stride >= chw, "upsample: x_batch_stride too small");
    PXE_REQUIRE(y_batch_stride == 0 || y_batch_stride >= ochw, "upsample: y_batch_stride too small");
    PXE_REQUIRE((long long)batch * ochw < (1LL << 32), "upsample: too many outputs for one launch");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    UpParams p{};
    p.x = x; p.y = y;
    p.xbs = x_batch_stride ? x_batch_stride : chw;
    p.ybs = y_batch_stride ? y_batch_stride : ochw;
    p.C = channels; p.H = height; p.W = width; p.stride = stride; p.scale = scale;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool out16 = aligned16(y) && p.ybs % 4 == 0;
    int vi = 0;
    if (stride == 2 && out16) {
        if (width % 4 == 0 && aligned16(x) && p.xbs % 4 == 0) vi = 4;
        else if (width % 2 == 0 && aligned8(x) && p.xbs % 2 == 0) vi = 2;
    }
    if (stride == 2 && vi == 0 && aligned8(y) && p.ybs % 2 == 0) vi = 1;
    if (vi) {
        p.total = (uint32_t)((long long)batch * chw / vi);
        p.div_w = FastDiv((uint32_t)(width / vi)); p.div_h = FastDiv((uint32_t)height); p.div_c = FastDiv((uint32_t)channels);
        unsigned grid = grid_for(p.total, kThreads, di.sm_count, 16);
        if (vi == 4) upsample2_vec_kernel<4><<<grid, kThreads, 0, s>>>(p);
        else if (vi == 2) upsample2_vec_kernel<2><<<grid, kThreads, 0, s>>>(p);
        else upsample2_vec_kernel<1><<<grid, kThreads, 0, s>>>(p);
    } else {
        p.total = (uint32_t)((long long)batch * ochw);
        p.div_w = FastDiv((uint32_t)(width * stride)); p.div_h = FastDiv((uint32_t)(height * stride));
        p.div_c = FastDiv((uint32_t)channels);
        unsigned grid = grid_for(p.total, kThreads, di.sm_count, 16);
        upsample_scalar_kernel<<<grid, kThreads, 0, s>>>(p);
    }
    PXE_LAUNCH_OK("upsample kernel");
    return PXE_OK;
}

extern "C" int pxe_shortcut(pxe_stream_t stream, const float* x, long long x_batch_stride, const float* from,
                            long long from_batch_stride, float* y, long long y_batch_stride, float* y2,
                            long long y2_batch_stride, int batch, int channels, int height, int width,
                            float alpha, float beta, int act)
{
    PXE_REQUIRE(x && from && y, "shortcut: null pointer");
    PXE_REQUIRE(valid_activation(act), "shortcut: unknown activation %d", act);
    // y = act(alpha*x + beta*from): the residual stage of the fused epilogue with an identity front
    pxe_epilogue_desc d{};
    d.x = x; d.x_batch_stride = x_batch_stride;
    d.y = y; d.y_batch_stride = y_batch_stride;
    d.y2 = y2; d.y2_batch_stride = y2_batch_stride;
    d.batch = batch; d.channels = channels; d.height = height; d.width = width;
    d.act = PXE_ACT_LINEAR;
    d.residual = from; d.residual_batch_stride = from_batch_stride;
    d.res_alpha = alpha; d.res_beta = beta; d.res_act = act;
    return pxe_conv_epilogue(stream, &d);
}

extern "C" int pxe_shortcut_general(pxe_stream_t stream, int batch, int w1, int h1, int c1, const float* add,
                                    int w2, int h2, int c2, float s1, float s2, float* out)
{
    PXE_REQUIRE(add && out, "shortcut_general: null pointer");
    PXE_REQUIRE(batch > 0 && w1 > 0 && h1 > 0 && c1 > 0 && w2 > 0 && h2 > 0 && c2 > 0, "shortcut_general: non-positive shape");
    ScParams p{};
    p.add = add; p.out = out;
    p.minw = w1 < w2 ? w1 : w2; p.minh = h1 < h2 ? h1 : h2; p.minc = c1 < c2 ? c1 : c2;
    p.stride = w1 / w2 < 1 ? 1 : w1 / w2;
    p.sample = w2 / w1 < 1 ? 1 : w2 / w1;
    p.batch = batch; p.w1 = w1; p.h1 = h1; p.c1 = c1; p.w2 = w2; p.h2 = h2; p.c2 = c2;
    p.s1 = s1; p.s2 = s2;
    const long long total = (long long)batch * p.minw * p.minh * p.minc;
    PXE_REQUIRE(total < (1LL << 32), "shortcut_general: too many elements for one launch");
    p.total = (uint32_t)total;
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    shortcut_general_kernel<<<grid_for(total, kThreads, di.sm_count, 16), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    PXE_LAUNCH_OK("shortcut_general_kernel");
    return PXE_OK;
}

extern "C" int pxe_concat(pxe_stream_t stream, int n_src, const float* const* srcs,
                          const long long* src_batch_strides, const int* src_channels, float* y,
                          long long y_batch_stride, int batch, int height, int width)
{
    PXE_REQUIRE(srcs && src_batch_strides && src_channels && y, "concat: null pointer");
    PXE_REQUIRE(n_src > 0 && n_src <= kMaxSources, "concat: n_src %d outside 1..%d", n_src, kMaxSources);
    PXE_REQUIRE(batch > 0 && height > 0 && width > 0, "concat: non-positive shape");
    const long long hw = (long long)height * width;
    CatParams p{};
    long long off = 0, longest = 0;
    for (int s = 0; s < n_src; ++s) {
        PXE_REQUIRE(srcs[s] != nullptr && src_channels[s] > 0, "concat: bad source %d", s);
        p.src[s] = srcs[s];
        p.len[s] = hw * src_channels[s];
        p.sbs[s] = src_batch_strides[s] ? src_batch_strides[s] : p.len[s];
        PXE_REQUIRE(p.sbs[s] >= p.len[s], "concat: source %d batch stride too small", s);
        p.dst_off[s] = off;
        off += p.len[s];
        if (p.len[s] > longest) longest = p.len[s];
    }
    p.ybs = y_batch_stride ? y_batch_stride : off;
    PXE_REQUIRE(p.ybs >= off, "concat: y_batch_stride too small");
    p.y = y; p.batch = batch;
    for (int s = 0; s < n_src; ++s)
        p.vec[s] = p.len[s] % 4 == 0 && aligned16(p.src[s]) && p.sbs[s] % 4 == 0 && aligned16(y) && p.ybs % 4 == 0
                   && p.dst_off[s] % 4 == 0;
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    dim3 grid(grid_for(longest * batch / 4 + 1, kThreads, di.sm_count, 8), (unsigned)n_src);
    concat_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    PXE_LAUNCH_OK("concat_kernel");
    return PXE_OK;
}
