// The epilogue path for channels-last (NHWC) tensors.
//
// Why a second layout: with fp32 NCHW tensors (what the reference hands cuDNN, include/Cudnn.h:103-108,
// include/cuda/ConvLayer.h:278-283) cuDNN wraps its NHWC tensor-core convolution kernels in layout conversions on
// every layer -- on a YOLOv3-608 forward those conversions are 31 % of the time, more than every kernel of this
// library together.  Given channels-last input and filters the same cuDNN call converts nothing (the 75
// convolutions of YOLOv3-608 at 64 images: 28.0 ms NCHW, 16.1 ms NHWC on B200).  These kernels keep the rest of
// the path in that layout: the fused conv epilogue (batch-norm inference folded to one multiply-add, bias,
// activation, optional residual add, optional second store), upsample, max pool, and the transposition that
// hands a head to the NCHW decoders.
//
// A tensor is addressed as pixel * pixel_stride + channel: pixel = (image * H + row) * W + col, and
// pixel_stride is the channel count of the buffer it lives in, so a channel slot of a wider concat buffer is
// the same thing as a dense tensor with a larger stride (the NHWC form of a route: include/cuda/RouteLayer.h:21-44).
// Per-channel coefficients come from a table folded once per layer (pxe_fold_bn): weights do not change
// between inference calls, so the square roots of include/cuda/ConvLayer.h:294-299 are not redone per launch.
#include <initializer_list>

#include "pxe_common.cuh"

namespace pxe {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__global__ void fold_bn_kernel(const float* gamma, const float* beta, const float* mean, const float* var,
                               const float* bias, float eps, int eps_mode, int channels, float* a, float* b)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float fa = 1.0f, fb = 0.0f;
    if (gamma) {
        const float v = gld(var + c);
        const float denom = eps_mode == PXE_BN_EPS_CPU ? (sqrtf(v) + eps) : sqrtf(v + eps);
        fa = gld(gamma + c) / denom;
        fb = gld(beta + c) - gld(mean + c) * fa;
    }
    if (bias) fb += gld(bias + c);
    gst(a + c, fa);
    gst(b + c, fb);
}

struct NhwcParams {
    const float* x; float* y; float* y2; const float* res;
    long long xps, yps, y2ps, rps;       // pixel strides, floats
    const float* a; const float* b;      // folded coefficients, or null
    int C, act, res_act;
    float ralpha, rbeta;
    uint32_t units, chunk;               // vectors (or elements) in total / per block
    FastDiv div_cv;                      // vectors (or elements) per pixel
    int fixed_channels;                  // vectors per pixel are a power of two that divides the block size
};

template <int ACT, bool AFFINE>
__device__ __forceinline__ float nhwc_apply(float v, float a, float b)
{
    if (AFFINE) v = fmaf(a, v, b);
    return activate<ACT, true>(v);
}

// VW = 4: C % 4 == 0 and every pointer / stride keeps 16-byte alignment; VW = 1: anything.
template <int ACT, bool AFFINE, bool RES, int VW>
__global__ void __launch_bounds__(kThreads, 5)
epilogue_nhwc_kernel(const NhwcParams p)
{
    const uint32_t lo = blockIdx.x * p.chunk;
    if (lo >= p.units) return;
    uint32_t hi = lo + p.chunk;
    if (hi > p.units) hi = p.units;
    // with a residual every vector holds two loads in flight: half the unroll keeps the bytes in flight per
    // thread (64) and the register count of the plain form, so that more blocks are resident
    constexpr int UN = RES ? kUnroll / 2 : kUnroll;
    const uint32_t step = kThreads * UN;
    // When the vectors of one pixel divide the block size (every power-of-two channel count up to 1024), a
    // thread meets the same four channels in every vector it handles: its coefficients are loaded once.
    // p.chunk and step are multiples of kThreads, so u % cv == threadIdx.x % cv throughout.
    const bool fixed = VW == 4 && AFFINE && p.fixed_channels;
    float4 fa = make_float4(1.f, 1.f, 1.f, 1.f), fb = make_float4(0.f, 0.f, 0.f, 0.f);
    if (fixed) {
        const uint32_t c4 = threadIdx.x & (p.div_cv.d - 1);
        fa = gldv<float4>(p.a + 4 * c4);
        fb = gldv<float4>(p.b + 4 * c4);
    }
    for (uint32_t r0 = lo; r0 < hi; r0 += step) {
        if (VW == 4) {
            float4 v[UN], r[UN];
            uint32_t pix[UN], ch[UN];
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = r0 + threadIdx.x + k * kThreads;
                if (u < hi) {
                    uint32_t cv;
                    p.div_cv.divmod(u, pix[k], cv);
                    ch[k] = cv * 4;
                    v[k] = gldv<float4>(p.x + (long long)pix[k] * p.xps + ch[k]);
                    if (RES) r[k] = gldv<float4>(p.res + (long long)pix[k] * p.rps + ch[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = r0 + threadIdx.x + k * kThreads;
                if (u < hi) {
                    float4 ca = fa, cb = fb;
                    if (AFFINE && !fixed) {                      // cache hits: the table is a few KB
                        ca = gldv<float4>(p.a + ch[k]);
                        cb = gldv<float4>(p.b + ch[k]);
                    }
                    float4 o;
                    o.x = nhwc_apply<ACT, AFFINE>(v[k].x, ca.x, cb.x);
                    o.y = nhwc_apply<ACT, AFFINE>(v[k].y, ca.y, cb.y);
                    o.z = nhwc_apply<ACT, AFFINE>(v[k].z, ca.z, cb.z);
                    o.w = nhwc_apply<ACT, AFFINE>(v[k].w, ca.w, cb.w);
                    if (RES) {
                        // alpha*v + beta*r as the reference's kernel evaluates it (src/ShortcutKernel.cu:41)
                        o.x = activate_dyn(p.res_act, fmaf(p.ralpha, o.x, p.rbeta * r[k].x));
                        o.y = activate_dyn(p.res_act, fmaf(p.ralpha, o.y, p.rbeta * r[k].y));
                        o.z = activate_dyn(p.res_act, fmaf(p.ralpha, o.z, p.rbeta * r[k].z));
                        o.w = activate_dyn(p.res_act, fmaf(p.ralpha, o.w, p.rbeta * r[k].w));
                    }
                    if (p.y) gstv(p.y + (long long)pix[k] * p.yps + ch[k], o);
                    if (p.y2) gstv(p.y2 + (long long)pix[k] * p.y2ps + ch[k], o);
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = r0 + threadIdx.x + k * kThreads;
                if (u < hi) {
                    uint32_t pix, c;
                    p.div_cv.divmod(u, pix, c);
                    float o = nhwc_apply<ACT, AFFINE>(gld(p.x + ((long long)pix * p.xps + c)), AFFINE ? gld(p.a + c) : 1.0f, AFFINE ? gld(p.b + c) : 0.0f);
                    if (RES) o = activate_dyn(p.res_act, fmaf(p.ralpha, o, p.rbeta * gld(p.res + ((long long)pix * p.rps + c))));
                    if (p.y) gst(p.y + ((long long)pix * p.yps + c), o);
                    if (p.y2) gst(p.y2 + ((long long)pix * p.y2ps + c), o);
                }
            }
        }
    }
}

template <int ACT, bool AFFINE, bool RES>
int launch_nhwc(cudaStream_t s, NhwcParams& p, long long n_elems, bool vec)
{
    const int vw = vec ? 4 : 1;
    p.units = (uint32_t)(n_elems / vw);
    p.div_cv = FastDiv((uint32_t)(p.C / vw));
    const uint32_t cv = (uint32_t)(p.C / vw);
    p.fixed_channels = vec && (cv & (cv - 1)) == 0 && cv <= (uint32_t)kThreads;
    p.chunk = kThreads * kUnroll * 2;                    // two rounds per block: short blocks, many waves
    const unsigned grid = (unsigned)((p.units + p.chunk - 1) / p.chunk);
    if (vec) epilogue_nhwc_kernel<ACT, AFFINE, RES, 4><<<grid, kThreads, 0, s>>>(p);
    else epilogue_nhwc_kernel<ACT, AFFINE, RES, 1><<<grid, kThreads, 0, s>>>(p);
    PXE_LAUNCH_OK("epilogue_nhwc_kernel");
    return PXE_OK;
}

template <int ACT>
int dispatch_nhwc(cudaStream_t s, NhwcParams& p, long long n, bool vec)
{
    const bool affine = p.a != nullptr, res = p.res != nullptr;
    if (affine) return res ? launch_nhwc<ACT, true, true>(s, p, n, vec) : launch_nhwc<ACT, true, false>(s, p, n, vec);
    return res ? launch_nhwc<ACT, false, true>(s, p, n, vec) : launch_nhwc<ACT, false, false>(s, p, n, vec);
}

// Epilogue + 2x2 stride-2 max pool, NHWC: the four taps of a window are four pixels with the same channel
// vector, so a thread handles one channel vector of one pooled pixel -- four loads, one pooled store and
// (when the full-resolution tensor is wanted too) four stores.  Window origin (2*oh, 2*ow), taps past the
// edge skipped, first maximum in (ky, kx) order wins (src/MaxPoolKernels.cu:26-40).
struct NhwcPoolParams {
    NhwcParams e;
    float* ypool; long long pps;
    int H, W, OH, OW;
    FastDiv div_ow, div_oh;
};

template <int ACT, bool AFFINE, int VW>
__global__ void __launch_bounds__(kThreads, 4)
epilogue_pool_nhwc_kernel(const NhwcPoolParams q)
{
    const NhwcParams& p = q.e;
    for (uint32_t u = blockIdx.x * kThreads + threadIdx.x; u < p.units; u += gridDim.x * kThreads) {
        uint32_t opix, cv, bh, ow, b, oh;
        p.div_cv.divmod(u, opix, cv);
        q.div_ow.divmod(opix, bh, ow);
        q.div_oh.divmod(bh, b, oh);
        const uint32_t c = cv * VW;
        const int iy = 2 * (int)oh, ix = 2 * (int)ow;
        const bool row1 = iy + 1 < q.H, col1 = ix + 1 < q.W;
        const long long pix00 = ((long long)b * q.H + iy) * q.W + ix;
        const long long tap[4] = {pix00, pix00 + 1, pix00 + q.W, pix00 + q.W + 1};
        const bool on[4] = {true, col1, row1, row1 && col1};
        float v[4][VW];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            if (!on[t]) continue;
            const float* src = p.x + tap[t] * p.xps + c;
            if (VW == 4) {
                const float4 f = gldv<float4>(src);
                v[t][0] = f.x; v[t][1] = f.y; v[t][2] = f.z; v[t][3] = f.w;
            } else {
                v[t][0] = gld(src);
            }
        }
        float ca[VW], cb[VW];
#pragma unroll
        for (int j = 0; j < VW; ++j) { ca[j] = AFFINE ? gld(p.a + (c + j)) : 1.0f; cb[j] = AFFINE ? gld(p.b + (c + j)) : 0.0f; }
        float m[VW];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            if (!on[t]) continue;
#pragma unroll
            for (int j = 0; j < VW; ++j) {
                v[t][j] = nhwc_apply<ACT, AFFINE>(v[t][j], ca[j], cb[j]);
                m[j] = (t == 0 || v[t][j] > m[j]) ? v[t][j] : m[j];
            }
            if (p.y) {
                float* dst = p.y + tap[t] * p.yps + c;
                if (VW == 4) gstv(dst, make_float4(v[t][0], v[t][1], v[t][2], v[t][3]));
                else gst(dst, v[t][0]);
            }
        }
        float* dst = q.ypool + (long long)opix * q.pps + c;
        if (VW == 4) gstv(dst, make_float4(m[0], m[1], m[2], m[3]));
        else gst(dst, m[0]);
    }
}

template <int ACT>
int launch_pool_nhwc(cudaStream_t s, NhwcPoolParams& q, bool vec, int sm_count)
{
    const bool affine = q.e.a != nullptr;
    const unsigned grid = grid_for(q.e.units, kThreads, sm_count, 32);
    if (vec) {
        if (affine) epilogue_pool_nhwc_kernel<ACT, true, 4><<<grid, kThreads, 0, s>>>(q);
        else epilogue_pool_nhwc_kernel<ACT, false, 4><<<grid, kThreads, 0, s>>>(q);
    } else {
        if (affine) epilogue_pool_nhwc_kernel<ACT, true, 1><<<grid, kThreads, 0, s>>>(q);
        else epilogue_pool_nhwc_kernel<ACT, false, 1><<<grid, kThreads, 0, s>>>(q);
    }
    PXE_LAUNCH_OK("epilogue_pool_nhwc_kernel");
    return PXE_OK;
}

// Nearest-neighbour upsample (src/UpsampleKernels.cu:25-63): thread per input vector, stride*stride stores.
template <int VW>
__global__ void __launch_bounds__(kThreads)
upsample_nhwc_kernel(const float* in, long long ips, float* out, long long ops, uint32_t units, FastDiv div_cv,
                     FastDiv div_w, FastDiv div_h, int H, int W, int stride, float scale)
{
    for (uint32_t u = blockIdx.x * kThreads + threadIdx.x; u < units; u += gridDim.x * kThreads) {
        uint32_t pix, cv, bh, col, b, row;
        div_cv.divmod(u, pix, cv);
        div_w.divmod(pix, bh, col);
        div_h.divmod(bh, b, row);
        const uint32_t c = cv * VW;
        const long long OW = (long long)W * stride;
        const long long obase = ((long long)b * H * stride + (long long)row * stride) * OW + (long long)col * stride;
        if (VW == 4) {
            float4 v = gldv<float4>(in + (long long)pix * ips + c);
            v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
            for (int dy = 0; dy < stride; ++dy)
                for (int dx = 0; dx < stride; ++dx)
                    gstv(out + (obase + dy * OW + dx) * ops + c, v);
        } else {
            const float v = gld(in + ((long long)pix * ips + c)) * scale;
            for (int dy = 0; dy < stride; ++dy)
                for (int dx = 0; dx < stride; ++dx) gst(out + ((obase + dy * OW + dx) * ops + c), v);
        }
    }
}

// Max pool with the reference's geometry (src/MaxPoolKernels.cu:10-43): window origin
// (oh*stride - padding/2, ow*stride - padding/2), taps outside the map skipped, the first maximum in
// (ky, kx) scan order wins, -FLT_MAX when no tap is valid.  Thread per output vector.
template <int VW>
__global__ void __launch_bounds__(kThreads)
maxpool_nhwc_kernel(const float* in, long long ips, float* out, long long ops, uint32_t units, FastDiv div_cv,
                    FastDiv div_ow, FastDiv div_oh, int H, int W, int kernel, int stride, int offset)
{
    for (uint32_t u = blockIdx.x * kThreads + threadIdx.x; u < units; u += gridDim.x * kThreads) {
        uint32_t opix, cv, bh, ow, b, oh;
        div_cv.divmod(u, opix, cv);
        div_ow.divmod(opix, bh, ow);
        div_oh.divmod(bh, b, oh);
        const uint32_t c = cv * VW;
        float m[VW];
#pragma unroll
        for (int j = 0; j < VW; ++j) m[j] = -FLT_MAX;
        for (int ky = 0; ky < kernel; ++ky) {
            const int iy = (int)oh * stride + offset + ky;
            if (iy < 0 || iy >= H) continue;
            for (int kx = 0; kx < kernel; ++kx) {
                const int ix = (int)ow * stride + offset + kx;
                if (ix < 0 || ix >= W) continue;
                const float* src = in + (((long long)b * H + iy) * W + ix) * ips + c;
                if (VW == 4) {
                    const float4 v = gldv<float4>(src);
                    m[0] = v.x > m[0] ? v.x : m[0]; m[1] = v.y > m[1] ? v.y : m[1];
                    m[2] = v.z > m[2] ? v.z : m[2]; m[3] = v.w > m[3] ? v.w : m[3];
                } else {
                    m[0] = gld(src) > m[0] ? gld(src) : m[0];
                }
            }
        }
        float* dst = out + (long long)opix * ops + c;
        if (VW == 4) gstv(dst, make_float4(m[0], m[1], m[2], m[3]));
        else gst(dst, m[0]);
    }
}

// [B, H*W, C] (pixel stride ips) -> [B, C, H*W] (batch stride obs): 32x32 tiles through shared memory.
__global__ void __launch_bounds__(256)
nhwc_to_nchw_kernel(const float* in, long long ips, float* out, long long obs, int C, int HW)
{
    __shared__ float tile[32][33];
    const int b = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;       // 32 x 8
    for (int j = ty; j < 32; j += 8) {
        const int pix = p0 + j, c = c0 + tx;
        if (pix < HW && c < C) tile[j][tx] = gld(in + (((long long)b * HW + pix) * ips + c));
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int c = c0 + j, pix = p0 + tx;
        if (pix < HW && c < C) gst(out + ((long long)b * obs + (long long)c * HW + pix), tile[tx][j]);
    }
}

long long dense_or(long long stride, long long dense) { return stride == 0 ? dense : stride; }

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" int pxe_fold_bn(pxe_stream_t stream, const float* gamma, const float* beta, const float* mean,
                           const float* var, const float* bias, float eps, int eps_mode, int channels, float* a,
                           float* b)
{
    PXE_REQUIRE(a && b && channels > 0, "fold_bn: null output or non-positive channel count");
    if (gamma) PXE_REQUIRE(beta && mean && var, "fold_bn: gamma given but beta/mean/var missing");
    PXE_REQUIRE(eps_mode == PXE_BN_EPS_CUDNN || eps_mode == PXE_BN_EPS_CPU, "fold_bn: bad eps_mode %d", eps_mode);
    fold_bn_kernel<<<(channels + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(gamma, beta, mean, var, bias, eps,
                                                                                      eps_mode, channels, a, b);
    PXE_LAUNCH_OK("fold_bn_kernel");
    return PXE_OK;
}

extern "C" int pxe_conv_epilogue_nhwc(pxe_stream_t stream, const pxe_epilogue_nhwc_desc* dp)
{
    PXE_REQUIRE(dp != nullptr, "conv_epilogue_nhwc: null descriptor");
    const pxe_epilogue_nhwc_desc& d = *dp;
    PXE_REQUIRE(d.x && (d.y || d.pool_kernel), "conv_epilogue_nhwc: x or y is null");
    PXE_REQUIRE(d.pixels > 0 && d.channels > 0, "conv_epilogue_nhwc: non-positive shape");
    PXE_REQUIRE(valid_activation(d.act), "conv_epilogue_nhwc: unknown activation %d", d.act);
    PXE_REQUIRE((d.a == nullptr) == (d.b == nullptr), "conv_epilogue_nhwc: a and b go together");
    if (d.residual) PXE_REQUIRE(valid_activation(d.res_act), "conv_epilogue_nhwc: unknown residual activation %d", d.res_act);
    const long long C = d.channels;
    for (long long ps : {d.x_pixel_stride, d.y_pixel_stride, d.y2_pixel_stride, d.residual_pixel_stride})
        PXE_REQUIRE(ps == 0 || ps >= C, "conv_epilogue_nhwc: a pixel stride is smaller than the channel count");
    NhwcParams p{};
    p.xps = dense_or(d.x_pixel_stride, C); p.yps = dense_or(d.y_pixel_stride, C);
    p.y2ps = dense_or(d.y2_pixel_stride, C); p.rps = dense_or(d.residual_pixel_stride, C);
    p.a = d.a; p.b = d.b; p.C = d.channels; p.act = d.act;
    p.ralpha = d.res_alpha; p.rbeta = d.res_beta; p.res_act = d.res_act;
    auto ok16 = [](const float* ptr, long long ps) { return !ptr || (aligned16(ptr) && ps % 4 == 0); };
    const bool vec = C % 4 == 0 && ok16(d.x, p.xps) && ok16(d.y, p.yps) && ok16(d.y2, p.y2ps) && ok16(d.residual, p.rps)
                     && ok16(d.a, 4) && ok16(d.b, 4);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d.pool_kernel) {
        PXE_REQUIRE(d.y_pool != nullptr, "conv_epilogue_nhwc: pooling requested but y_pool is null");
        if (d.pool_kernel != 2 || d.pool_stride != 2 || d.pool_padding < 0 || d.pool_padding > 1)
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue_nhwc: fused pooling supports kernel 2 / stride 2 / padding 0|1 only (got %d/%d/%d)",
                             d.pool_kernel, d.pool_stride, d.pool_padding);
        if (d.residual || d.y2)
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue_nhwc: fused pooling cannot be combined with residual or y2");
        PXE_REQUIRE(d.batch > 0 && d.height > 0 && d.width > 0 && (long long)d.batch * d.height * d.width == d.pixels,
                    "conv_epilogue_nhwc: batch * height * width must equal pixels when pooling");
        NhwcPoolParams q{};
        q.e = p;
        q.e.x = d.x; q.e.y = d.y;
        q.H = d.height; q.W = d.width;
        q.OH = pxe_maxpool_out_dim(d.height, 2, 2, d.pool_padding);
        q.OW = pxe_maxpool_out_dim(d.width, 2, 2, d.pool_padding);
        PXE_REQUIRE(q.OH > 0 && q.OW > 0, "conv_epilogue_nhwc: empty pooled output");
        if (d.y && (2 * q.OH < d.height || 2 * q.OW < d.width))
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue_nhwc: padding 0 with an odd extent leaves full-resolution rows uncovered");
        q.ypool = d.y_pool; q.pps = dense_or(d.y_pool_pixel_stride, C);
        PXE_REQUIRE(q.pps >= C, "conv_epilogue_nhwc: y_pool pixel stride smaller than the channel count");
        const bool pvec = vec && aligned16(d.y_pool) && q.pps % 4 == 0;
        const int vw = pvec ? 4 : 1;
        const long long units = (long long)d.batch * q.OH * q.OW * (C / vw);
        PXE_REQUIRE(units < (1LL << 32), "conv_epilogue_nhwc: pooled tensor too large for one launch");
        q.e.units = (uint32_t)units;
        q.e.div_cv = FastDiv((uint32_t)(C / vw));
        q.div_ow = FastDiv((uint32_t)q.OW); q.div_oh = FastDiv((uint32_t)q.OH);
        DeviceInfo di;
        int rc = device_info(&di);
        if (rc != PXE_OK) return rc;
        switch (d.act) {
        case PXE_ACT_LEAKY: return launch_pool_nhwc<PXE_ACT_LEAKY>(s, q, pvec, di.sm_count);
        case PXE_ACT_LINEAR: return launch_pool_nhwc<PXE_ACT_LINEAR>(s, q, pvec, di.sm_count);
        case PXE_ACT_LOGGY: return launch_pool_nhwc<PXE_ACT_LOGGY>(s, q, pvec, di.sm_count);
        case PXE_ACT_LOGISTIC: return launch_pool_nhwc<PXE_ACT_LOGISTIC>(s, q, pvec, di.sm_count);
        case PXE_ACT_MISH: return launch_pool_nhwc<PXE_ACT_MISH>(s, q, pvec, di.sm_count);
        case PXE_ACT_RELU: return launch_pool_nhwc<PXE_ACT_RELU>(s, q, pvec, di.sm_count);
        case PXE_ACT_SOFTPLUS: return launch_pool_nhwc<PXE_ACT_SOFTPLUS>(s, q, pvec, di.sm_count);
        case PXE_ACT_SWISH: return launch_pool_nhwc<PXE_ACT_SWISH>(s, q, pvec, di.sm_count);
        default: return launch_pool_nhwc<PXE_ACT_TANH>(s, q, pvec, di.sm_count);
        }
    }
    // unit indices are 32-bit: at most 2^31 elements per launch, larger tensors go in slices of whole pixels
    const long long per = ((1LL << 31) / C) > 0 ? ((1LL << 31) / C) : 1;
    for (long long p0 = 0; p0 < d.pixels; p0 += per) {
        const long long np = d.pixels - p0 < per ? d.pixels - p0 : per;
        p.x = d.x + p0 * p.xps; p.y = d.y + p0 * p.yps;
        p.y2 = d.y2 ? d.y2 + p0 * p.y2ps : nullptr;
        p.res = d.residual ? d.residual + p0 * p.rps : nullptr;
        int rc;
        switch (d.act) {
        case PXE_ACT_LEAKY: rc = dispatch_nhwc<PXE_ACT_LEAKY>(s, p, np * C, vec); break;
        case PXE_ACT_LINEAR: rc = dispatch_nhwc<PXE_ACT_LINEAR>(s, p, np * C, vec); break;
        case PXE_ACT_LOGGY: rc = dispatch_nhwc<PXE_ACT_LOGGY>(s, p, np * C, vec); break;
        case PXE_ACT_LOGISTIC: rc = dispatch_nhwc<PXE_ACT_LOGISTIC>(s, p, np * C, vec); break;
        case PXE_ACT_MISH: rc = dispatch_nhwc<PXE_ACT_MISH>(s, p, np * C, vec); break;
        case PXE_ACT_RELU: rc = dispatch_nhwc<PXE_ACT_RELU>(s, p, np * C, vec); break;
        case PXE_ACT_SOFTPLUS: rc = dispatch_nhwc<PXE_ACT_SOFTPLUS>(s, p, np * C, vec); break;
        case PXE_ACT_SWISH: rc = dispatch_nhwc<PXE_ACT_SWISH>(s, p, np * C, vec); break;
        default: rc = dispatch_nhwc<PXE_ACT_TANH>(s, p, np * C, vec); break;
        }
        if (rc != PXE_OK) return rc;
    }
    return PXE_OK;
}

extern "C" int pxe_upsample_nhwc(pxe_stream_t stream, const float* in, long long in_pixel_stride, float* out,
                                 long long out_pixel_stride, int batch, int channels, int height, int width,
                                 int stride, float scale)
{
    PXE_REQUIRE(in && out, "upsample_nhwc: null pointer");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0 && stride > 0, "upsample_nhwc: non-positive shape");
    const long long ips = dense_or(in_pixel_stride, channels), ops = dense_or(out_pixel_stride, channels);
    PXE_REQUIRE(ips >= channels && ops >= channels, "upsample_nhwc: pixel stride smaller than the channel count");
    const long long pixels = (long long)batch * height * width;
    PXE_REQUIRE(pixels * channels < (1LL << 32), "upsample_nhwc: tensor too large");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    const bool vec = channels % 4 == 0 && aligned16(in) && aligned16(out) && ips % 4 == 0 && ops % 4 == 0;
    const int vw = vec ? 4 : 1;
    const uint32_t units = (uint32_t)(pixels * channels / vw);
    const unsigned grid = grid_for(units, kThreads, di.sm_count, 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const FastDiv dcv((uint32_t)(channels / vw)), dw((uint32_t)width), dh((uint32_t)height);
    if (vec) upsample_nhwc_kernel<4><<<grid, kThreads, 0, s>>>(in, ips, out, ops, units, dcv, dw, dh, height, width, stride, scale);
    else upsample_nhwc_kernel<1><<<grid, kThreads, 0, s>>>(in, ips, out, ops, units, dcv, dw, dh, height, width, stride, scale);
    PXE_LAUNCH_OK("upsample_nhwc_kernel");
    return PXE_OK;
}

extern "C" int pxe_maxpool_nhwc(pxe_stream_t stream, const float* in, long long in_pixel_stride, float* out,
                                long long out_pixel_stride, int batch, int channels, int height, int width,
                                int kernel, int stride, int padding)
{
    PXE_REQUIRE(in && out, "maxpool_nhwc: null pointer");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0 && kernel > 0 && stride > 0 && padding >= 0,
                "maxpool_nhwc: bad shape");
    const int oh = pxe_maxpool_out_dim(height, kernel, stride, padding), ow = pxe_maxpool_out_dim(width, kernel, stride, padding);
    PXE_REQUIRE(oh > 0 && ow > 0, "maxpool_nhwc: empty output");
    const long long ips = dense_or(in_pixel_stride, channels), ops = dense_or(out_pixel_stride, channels);
    PXE_REQUIRE(ips >= channels && ops >= channels, "maxpool_nhwc: pixel stride smaller than the channel count");
    const long long opixels = (long long)batch * oh * ow;
    PXE_REQUIRE(opixels * channels < (1LL << 32) && (long long)batch * height * width * ips < (1LL << 62), "maxpool_nhwc: tensor too large");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    const bool vec = channels % 4 == 0 && aligned16(in) && aligned16(out) && ips % 4 == 0 && ops % 4 == 0;
    const int vw = vec ? 4 : 1;
    const uint32_t units = (uint32_t)(opixels * channels / vw);
    const unsigned grid = grid_for(units, kThreads, di.sm_count, 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const FastDiv dcv((uint32_t)(channels / vw)), dow((uint32_t)ow), doh((uint32_t)oh);
    if (vec) maxpool_nhwc_kernel<4><<<grid, kThreads, 0, s>>>(in, ips, out, ops, units, dcv, dow, doh, height, width, kernel, stride, -(padding / 2));
    else maxpool_nhwc_kernel<1><<<grid, kThreads, 0, s>>>(in, ips, out, ops, units, dcv, dow, doh, height, width, kernel, stride, -(padding / 2));
    PXE_LAUNCH_OK("maxpool_nhwc_kernel");
    return PXE_OK;
}

extern "C" int pxe_nhwc_to_nchw(pxe_stream_t stream, const float* in, long long in_pixel_stride, float* out,
                                long long out_batch_stride, int batch, int channels, int height, int width)
{
    PXE_REQUIRE(in && out && in != out, "nhwc_to_nchw: null or aliased pointers");
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0, "nhwc_to_nchw: non-positive shape");
    PXE_REQUIRE(batch <= 65535, "nhwc_to_nchw: batch exceeds 65535");
    const long long hw = (long long)height * width;
    PXE_REQUIRE(hw <= 0x7fffffffLL && (channels + 31) / 32 <= 65535, "nhwc_to_nchw: tensor too large");
    const long long ips = dense_or(in_pixel_stride, channels), obs = dense_or(out_batch_stride, hw * channels);
    PXE_REQUIRE(ips >= channels && obs >= hw * channels, "nhwc_to_nchw: stride too small");
    dim3 grid((unsigned)((hw + 31) / 32), (unsigned)((channels + 31) / 32), (unsigned)batch);
    nhwc_to_nchw_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(in, ips, out, obs, channels, (int)hw);
    PXE_LAUNCH_OK("nhwc_to_nchw_kernel");
    return PXE_OK;
}
