// Batch normalisation in training mode, forward and backward, on dense NCHW tensors.  The reference's CUDA layers
// hand both to cuDNN (cudnnBatchNormalizationForwardTraining: include/cuda/ConvLayer.h:285-292,
// include/cuda/BatchNormLayer.h:59-71, include/cuda/ConnLayer.h:198-203; cudnnBatchNormalizationBackward:
// include/cuda/ConvLayer.h:327-332, include/cuda/BatchNormLayer.h:108-118, include/cuda/ConnLayer.h:233-238) and
// surround them with full-tensor copies (x_.copy(output_) before, preActivation_.copy(output_) and the in-place
// activation after: include/cuda/ConvLayer.h:286, 306-307); its CPU twins are batchNormForward / batchNormBackward
// (src/BatchNorm.cpp:24-98) over the loops of src/CpuUtil.cpp:198-343.
//
// Forward here is two passes over x and no copy: per-channel sums (a fixed split of every channel over blocks,
// combined in a fixed order, so the same call gives the same bits every time), then one pass that writes the
// normalised tensor and, if asked, the activated layer output beside it -- 4 + 4 + 4 (+ 4) bytes per element where
// the reference's sequence moves 36.  Backward is the same shape: per-channel sums of dy and dy * (x - mean), then
// dx = k1 * dy + k2 * x + k3 with three per-channel constants.
//
// eps_mode picks whose arithmetic is reproduced.  PXE_BN_EPS_CUDNN (what the CUDA layers get from cuDNN):
// y = gamma * (x - mean) / sqrt(var + eps) + beta, the saved scale is 1 / sqrt(var + eps), the running variance is
// fed the unbiased estimate var * n / (n - 1).  PXE_BN_EPS_CPU (src/BatchNorm.cpp, src/CpuUtil.cpp:264-300):
// y = gamma * (x - mean) / (sqrt(var) + eps) + beta, the saved scale is the population variance itself, and that is
// also what the running variance is fed; backward then uses 1 / sqrt(var + eps) for dx and 1 / (sqrt(var) + eps)
// for the normalised input in the scale gradient, as src/CpuUtil.cpp:303-343 and src/BatchNorm.cpp:84-97 do.
#include <stdint.h>

#include "pxe_common.cuh"

namespace pxe {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxPlaneSplits = 64;
constexpr int kSplitElements = 8192;        // a block's share of one plane

struct Split { int per_plane; int chunk; };

Split plane_split(long long hw)
{
    long long p = (hw + kSplitElements - 1) / kSplitElements;
    if (p < 1) p = 1;
    if (p > kMaxPlaneSplits) p = kMaxPlaneSplits;
    long long chunk = (hw + p - 1) / p;
    chunk = (chunk + 3) & ~3LL;                 // vector loads never cross a chunk
    Split s;
    s.chunk = (int)chunk;
    s.per_plane = (int)((hw + chunk - 1) / chunk);
    return s;
}

struct ReduceParams {
    const float* x; const float* dy;            // dy only in the backward form
    const float* mean;                          // backward: the saved batch mean
    float2* partial;                            // [C][splits]
    int B, C, HW, per_plane, chunk;
    int items;                                  // B * per_plane pieces of a channel, dealt out to the splits in turn
};

// Sums over one piece (image b, elements lo..hi of the plane) by `threads` cooperating threads, thread `t` of them.
// BACKWARD false: (x - K) and (x - K)^2; BACKWARD true: dy and dy * (x - mean).
template <bool BACKWARD, bool VEC>
__device__ __forceinline__ void bn_piece_sums(const ReduceParams& p, int c, int item, float shift, int t, int threads,
                                              float& s1, float& s2)
{
    const int b = item / p.per_plane, part = item - b * p.per_plane;
    const long long base = ((long long)b * p.C + c) * p.HW;
    const int lo = part * p.chunk;
    const int hi = min(lo + p.chunk, p.HW);
    if (VEC) {
        const float4* x4 = reinterpret_cast<const float4*>(p.x + base);
        const float4* d4 = BACKWARD ? reinterpret_cast<const float4*>(p.dy + base) : nullptr;
        // four vectors per thread in flight (two of each tensor in the backward form)
        constexpr int U = BACKWARD ? 2 : 4;
        for (int i0 = lo / 4 + t; i0 < hi / 4; i0 += U * threads) {
            float4 v[U], d[U];
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const int i = i0 + j * threads;
                const bool in = i < hi / 4;
                v[j] = in ? gld(x4 + i) : make_float4(shift, shift, shift, shift);
                if (BACKWARD) d[j] = in ? gld(d4 + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const float a0 = v[j].x - shift, a1 = v[j].y - shift, a2 = v[j].z - shift, a3 = v[j].w - shift;
                if (BACKWARD) {
                    s1 += (d[j].x + d[j].y) + (d[j].z + d[j].w);
                    s2 += fmaf(d[j].x, a0, d[j].y * a1) + fmaf(d[j].z, a2, d[j].w * a3);
                } else {
                    s1 += (a0 + a1) + (a2 + a3);
                    s2 += fmaf(a0, a0, a1 * a1) + fmaf(a2, a2, a3 * a3);
                }
            }
        }
    } else {
        for (int i = lo + t; i < hi; i += threads) {
            const float a = gld(p.x + (base + i)) - shift;
            if (BACKWARD) {
                const float d = gld(p.dy + (base + i));
                s1 += d;
                s2 = fmaf(d, a, s2);
            } else {
                s1 += a;
                s2 = fmaf(a, a, s2);
            }
        }
    }
}

// Block (c, s) adds up the pieces s, s + splits, ... of channel c.  The shift K of the forward form is the
// channel's first element (it keeps the variance free of the cancellation a plain sum of squares has when
// |mean| >> sigma).  WARP_PIECES: pieces are small (planes of a few hundred elements), so each warp takes whole
// pieces of its own instead of the block sharing one.
template <bool BACKWARD, bool VEC, bool WARP_PIECES>
__global__ void __launch_bounds__(kThreads)
bn_reduce_kernel(const ReduceParams p)
{
    const int c = blockIdx.x, s = blockIdx.y, splits = gridDim.y;
    const float shift = BACKWARD ? gld(p.mean + c) : gld(p.x + ((long long)c * p.HW));
    float s1 = 0.0f, s2 = 0.0f;
    if (WARP_PIECES) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int item = s + splits * warp; item < p.items; item += splits * (kThreads / 32))
            bn_piece_sums<BACKWARD, VEC>(p, c, item, shift, lane, 32, s1, s2);
    } else {
        for (int item = s; item < p.items; item += splits)
            bn_piece_sums<BACKWARD, VEC>(p, c, item, shift, (int)threadIdx.x, kThreads, s1, s2);
    }
    __shared__ float2 warp_sums[kThreads / 32];
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = make_float2(s1, s2);
    __syncthreads();
    if (threadIdx.x == 0) {
        float t1 = 0.0f, t2 = 0.0f;
        for (int w = 0; w < kThreads / 32; ++w) { t1 += warp_sums[w].x; t2 += warp_sums[w].y; }
        gst(p.partial + ((long long)c * splits + s), make_float2(t1, t2));
    }
}

struct ForwardFinal {
    const float* x; const float2* partial;
    const float *gamma, *beta;
    float *running_mean, *running_var, *save_mean, *save_scale;
    float2* coeff;                              // [C]: y = coeff.x * x + coeff.y
    float factor, eps; int eps_mode;
    int C, HW, splits; long long n;             // n = batch * HW
};

__global__ void bn_forward_final_kernel(const ForwardFinal p)
{
    // a warp per channel: the lanes take the channel's partial sums side by side (a single thread walking them pays one
    // memory latency per partial: 10 us for 43 of them), then one shuffle tree in double precision
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (c >= p.C) return;
    double s1 = 0.0, s2 = 0.0;
    for (int s = lane; s < p.splits; s += 32) {
        const float2 t = gld(p.partial + ((long long)c * p.splits + s));
        s1 += t.x; s2 += t.y;
    }
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane != 0) return;
    const double n = (double)p.n;
    const float mean = (float)((double)gld(p.x + ((long long)c * p.HW)) + s1 / n);
    double var_d = (s2 - s1 * s1 / n) / n;
    if (var_d < 0.0) var_d = 0.0;
    const float var = (float)var_d;
    float inv, fed;
    if (p.eps_mode == PXE_BN_EPS_CPU) {
        inv = 1.0f / (sqrtf(var) + p.eps);
        fed = var;
        gst(p.save_scale + c, var);
    } else {
        inv = 1.0f / sqrtf(var + p.eps);
        fed = p.n > 1 ? (float)(var_d * n / (n - 1.0)) : var;
        gst(p.save_scale + c, inv);
    }
    gst(p.save_mean + c, mean);
    if (p.running_mean) gst(p.running_mean + c, (1.0f - p.factor) * gld(p.running_mean + c) + p.factor * mean);
    if (p.running_var) gst(p.running_var + c, (1.0f - p.factor) * gld(p.running_var + c) + p.factor * fed);
    const float a = gld(p.gamma + c) * inv;
    gst(p.coeff + c, make_float2(a, gld(p.beta + c) - mean * a));
}

struct BackwardFinal {
    const float2* partial;
    const float *gamma, *save_mean, *save_scale;
    float *dgamma, *dbeta;
    float4* coeff;                              // [C]: dx = coeff.x * dy + coeff.y * x + coeff.z
    float eps; int eps_mode;
    int C, splits; long long n;
};

__global__ void bn_backward_final_kernel(const BackwardFinal p)
{
    // a warp per channel: the lanes take the channel's partial sums side by side (a single thread walking them pays one
    // memory latency per partial: 10 us for 43 of them), then one shuffle tree in double precision
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (c >= p.C) return;
    double s1 = 0.0, s2 = 0.0;
    for (int s = lane; s < p.splits; s += 32) {
        const float2 t = gld(p.partial + ((long long)c * p.splits + s));
        s1 += t.x; s2 += t.y;
    }
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane != 0) return;
    float inv_fwd, inv_bwd;
    if (p.eps_mode == PXE_BN_EPS_CPU) {
        const float var = gld(p.save_scale + c);
        inv_fwd = 1.0f / (sqrtf(var) + p.eps);
        inv_bwd = 1.0f / sqrtf(var + p.eps);
    } else {
        inv_fwd = inv_bwd = gld(p.save_scale + c);
    }
    if (p.dbeta) gst(p.dbeta + c, gld(p.dbeta + c) + (float)s1);
    if (p.dgamma) gst(p.dgamma + c, gld(p.dgamma + c) + (float)(s2 * (double)inv_fwd));
    const double n = (double)p.n;
    const float g = gld(p.gamma + c), mean = gld(p.save_mean + c);
    const float k1 = g * inv_bwd;
    const float k2 = (float)(-(double)g * inv_bwd * inv_bwd * inv_bwd * s2 / n);
    const float k3 = (float)(-(double)g * inv_bwd * s1 / n);
    gst(p.coeff + c, make_float4(k1, k2, k3 - k2 * mean, 0.0f));
}

struct ApplyParams {
    const float* x; const float* dy;
    float* y; float* y_act;
    const float2* coeff2; const float4* coeff4;
    int act;
    uint32_t units;                 // vectors (VEC) or elements
    uint32_t HW;
    FastDiv div_hw, div_c;          // elements per plane; channels
};

__device__ __forceinline__ uint32_t channel_of(const ApplyParams& p, uint32_t element)
{
    const uint32_t plane = p.div_hw.div(element);
    return plane - p.div_c.div(plane) * p.div_c.d;
}

// VEC: the tensor is dense and 16-byte aligned with a multiple of four elements; a vector may straddle two planes
// (odd plane sizes), in which case each component looks its own channel up.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
bn_forward_apply_kernel(const ApplyParams p)
{
    if (VEC) {
        // two vectors per thread in flight
        const uint32_t stride = gridDim.x * kThreads;
        for (uint32_t u0 = blockIdx.x * kThreads + threadIdx.x; u0 < p.units; u0 += 2 * stride) {
            float4 in[2];
#pragma unroll
            for (int j = 0; j < 2; ++j)
                if (u0 + j * stride < p.units) in[j] = gld(reinterpret_cast<const float4*>(p.x) + (p.units - 1 - (u0 + j * stride)));
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (u0 + j * stride >= p.units) break;
                // back to front: the statistics pass went front to back, so the end of x is what L2 still holds
                const uint32_t u = p.units - 1 - (u0 + j * stride);
                const uint32_t e = 4u * u;
                const uint32_t plane = p.div_hw.div(e);
                const uint32_t c = plane - p.div_c.div(plane) * p.div_c.d;
                const bool whole = e + 3 < (plane + 1) * p.HW;
                const float2 k0 = gld(p.coeff2 + c);
                float4 v = in[j];
                v.x = fmaf(k0.x, v.x, k0.y);
                if (whole) {
                    v.y = fmaf(k0.x, v.y, k0.y); v.z = fmaf(k0.x, v.z, k0.y); v.w = fmaf(k0.x, v.w, k0.y);
                } else {
                    const float2 k1 = gld(p.coeff2 + channel_of(p, e + 1)), k2 = gld(p.coeff2 + channel_of(p, e + 2)), k3 = gld(p.coeff2 + channel_of(p, e + 3));
                    v.y = fmaf(k1.x, v.y, k1.y); v.z = fmaf(k2.x, v.z, k2.y); v.w = fmaf(k3.x, v.w, k3.y);
                }
                gst(reinterpret_cast<float4*>(p.y) + u, v);
                if (p.y_act) {
                    v.x = activate_dyn(p.act, v.x); v.y = activate_dyn(p.act, v.y);
                    v.z = activate_dyn(p.act, v.z); v.w = activate_dyn(p.act, v.w);
                    gst(reinterpret_cast<float4*>(p.y_act) + u, v);
                }
            }
        }
        return;
    }
    for (uint32_t u = blockIdx.x * kThreads + threadIdx.x; u < p.units; u += gridDim.x * kThreads) {
        const float2 k = gld(p.coeff2 + channel_of(p, u));
        const float v = fmaf(k.x, gld(p.x + u), k.y);
        gst(p.y + u, v);
        if (p.y_act) gst(p.y_act + u, activate_dyn(p.act, v));
    }
}

__device__ __forceinline__ float bn_dx(const float4 k, float d, float v) { return fmaf(k.x, d, fmaf(k.y, v, k.z)); }

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
bn_backward_apply_kernel(const ApplyParams p)
{
    for (uint32_t uf = blockIdx.x * kThreads + threadIdx.x; uf < p.units; uf += gridDim.x * kThreads) {
        const uint32_t u = p.units - 1 - uf;           // back to front, as in the forward pass
        if (VEC) {
            const uint32_t e = 4u * u;
            const uint32_t plane = p.div_hw.div(e);
            const uint32_t c = plane - p.div_c.div(plane) * p.div_c.d;
            const bool whole = e + 3 < (plane + 1) * p.HW;
            const float4 k0 = gld(p.coeff4 + c);
            const float4 v = gld(reinterpret_cast<const float4*>(p.x) + u);
            const float4 d = gld(reinterpret_cast<const float4*>(p.dy) + u);
            float4 o;
            o.x = bn_dx(k0, d.x, v.x);
            if (whole) {
                o.y = bn_dx(k0, d.y, v.y); o.z = bn_dx(k0, d.z, v.z); o.w = bn_dx(k0, d.w, v.w);
            } else {
                o.y = bn_dx(gld(p.coeff4 + channel_of(p, e + 1)), d.y, v.y);
                o.z = bn_dx(gld(p.coeff4 + channel_of(p, e + 2)), d.z, v.z);
                o.w = bn_dx(gld(p.coeff4 + channel_of(p, e + 3)), d.w, v.w);
            }
            gst(reinterpret_cast<float4*>(p.y) + u, o);
        } else {
            gst(p.y + u, bn_dx(gld(p.coeff4 + channel_of(p, u)), gld(p.dy + u), gld(p.x + u)));
        }
    }
}

struct Shape { long long hw, n_elems; Split split; int items, splits; bool warp_pieces; };

// How many blocks share a channel: one per piece for large planes; for small ones enough pieces per block for about
// 4096 elements each, but never fewer blocks in all than fill the machine a few times over.
int choose_splits(int batch, int channels, long long hw, int items)
{
    const long long by_size = ((long long)batch * hw + 4095) / 4096;
    const long long by_grid = (1184 + channels - 1) / channels;
    long long s = by_size > by_grid ? by_size : by_grid;
    if (s > items) s = items;
    if (s < 1) s = 1;
    return (int)s;
}

int check_shape(int batch, int channels, int height, int width, Shape* s, const char* who)
{
    PXE_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0, "%s: non-positive shape", who);
    s->hw = (long long)height * width;
    s->n_elems = s->hw * channels * batch;
    PXE_REQUIRE(s->hw <= 0x7fffffffLL && s->n_elems < (1LL << 32), "%s: tensor too large for one launch", who);
    s->split = plane_split(s->hw);
    const long long items = (long long)batch * s->split.per_plane;
    PXE_REQUIRE(items <= 0x7fffffffLL, "%s: too many pieces", who);
    s->items = (int)items;
    s->splits = choose_splits(batch, channels, s->hw, s->items);
    PXE_REQUIRE(s->splits <= 65535, "%s: %d blocks per channel exceed 65535", who, s->splits);
    s->warp_pieces = s->split.chunk <= 1024;
    return PXE_OK;
}

size_t workspace_for(int channels, int splits)
{
    return (size_t)channels * ((size_t)splits * sizeof(float2) + sizeof(float4));
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" size_t pxe_batchnorm_workspace_bytes(int batch, int channels, int height, int width)
{
    if (batch <= 0 || channels <= 0 || height <= 0 || width <= 0) return 0;
    const long long hw = (long long)height * width;
    const Split sp = plane_split(hw);
    return workspace_for(channels, choose_splits(batch, channels, hw, batch * sp.per_plane));
}

extern "C" int pxe_batchnorm_forward_training(pxe_stream_t stream, const pxe_bn_train_desc* dp)
{
    PXE_REQUIRE(dp != nullptr, "batchnorm_forward_training: null descriptor");
    const pxe_bn_train_desc& d = *dp;
    PXE_REQUIRE(d.x && d.y && d.gamma && d.beta && d.save_mean && d.save_scale, "batchnorm_forward_training: null pointer");
    PXE_REQUIRE(d.eps_mode == PXE_BN_EPS_CUDNN || d.eps_mode == PXE_BN_EPS_CPU, "batchnorm_forward_training: unknown eps_mode %d", d.eps_mode);
    PXE_REQUIRE(!d.y_act || valid_activation(d.act), "batchnorm_forward_training: unknown activation %d", d.act);
    PXE_REQUIRE(!d.y_act || (d.y_act != d.y && d.y_act != d.x), "batchnorm_forward_training: y_act must not alias x or y");
    Shape sh;
    int rc = check_shape(d.batch, d.channels, d.height, d.width, &sh, "batchnorm_forward_training");
    if (rc != PXE_OK) return rc;
    PXE_REQUIRE(d.workspace && d.workspace_bytes >= workspace_for(d.channels, sh.splits),
                "batchnorm_forward_training: workspace of %zu bytes, %zu needed", d.workspace_bytes, workspace_for(d.channels, sh.splits));
    PXE_REQUIRE(aligned16(d.workspace), "batchnorm_forward_training: workspace must be 16-byte aligned");
    DeviceInfo di;
    rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    float4* coeff4 = static_cast<float4*>(d.workspace);
    float2* partial = reinterpret_cast<float2*>(coeff4 + d.channels);
    ReduceParams rp{};
    rp.x = d.x; rp.partial = partial;
    rp.B = d.batch; rp.C = d.channels; rp.HW = (int)sh.hw; rp.per_plane = sh.split.per_plane; rp.chunk = sh.split.chunk; rp.items = sh.items;
    const bool vec_in = sh.hw % 4 == 0 && aligned16(d.x);
    const dim3 rgrid((unsigned)d.channels, (unsigned)sh.splits);
    if (vec_in) {
        if (sh.warp_pieces) bn_reduce_kernel<false, true, true><<<rgrid, kThreads, 0, s>>>(rp);
        else bn_reduce_kernel<false, true, false><<<rgrid, kThreads, 0, s>>>(rp);
    } else {
        if (sh.warp_pieces) bn_reduce_kernel<false, false, true><<<rgrid, kThreads, 0, s>>>(rp);
        else bn_reduce_kernel<false, false, false><<<rgrid, kThreads, 0, s>>>(rp);
    }
    PXE_LAUNCH_OK("bn_reduce_kernel");

    ForwardFinal ff{};
    ff.x = d.x; ff.partial = partial; ff.gamma = d.gamma; ff.beta = d.beta;
    ff.running_mean = d.running_mean; ff.running_var = d.running_var;
    ff.save_mean = d.save_mean; ff.save_scale = d.save_scale;
    ff.coeff = reinterpret_cast<float2*>(coeff4);
    ff.factor = d.exp_avg_factor; ff.eps = d.eps; ff.eps_mode = d.eps_mode;
    ff.C = d.channels; ff.HW = (int)sh.hw; ff.splits = sh.splits; ff.n = (long long)d.batch * sh.hw;
    bn_forward_final_kernel<<<(d.channels + 3) / 4, 128, 0, s>>>(ff);
    PXE_LAUNCH_OK("bn_forward_final_kernel");

    ApplyParams ap{};
    ap.x = d.x; ap.y = d.y; ap.y_act = d.y_act; ap.act = d.act;
    ap.coeff2 = reinterpret_cast<const float2*>(coeff4);
    const bool vec = sh.n_elems % 4 == 0 && aligned16(d.x) && aligned16(d.y) && (!d.y_act || aligned16(d.y_act));
    ap.units = (uint32_t)(vec ? sh.n_elems / 4 : sh.n_elems);
    ap.HW = (uint32_t)sh.hw;
    ap.div_hw = FastDiv((uint32_t)sh.hw);
    ap.div_c = FastDiv((uint32_t)d.channels);
    const unsigned grid = grid_for(ap.units, kThreads * 4, di.sm_count, 16);
    if (vec) bn_forward_apply_kernel<true><<<grid, kThreads, 0, s>>>(ap);
    else bn_forward_apply_kernel<false><<<grid, kThreads, 0, s>>>(ap);
    PXE_LAUNCH_OK("bn_forward_apply_kernel");
    return PXE_OK;
}

extern "C" int pxe_batchnorm_backward(pxe_stream_t stream, const pxe_bn_backward_desc* dp)
{
    PXE_REQUIRE(dp != nullptr, "batchnorm_backward: null descriptor");
    const pxe_bn_backward_desc& d = *dp;
    PXE_REQUIRE(d.x && d.dy && d.dx && d.gamma && d.save_mean && d.save_scale, "batchnorm_backward: null pointer");
    PXE_REQUIRE(d.dx != d.x, "batchnorm_backward: dx must not alias x");
    PXE_REQUIRE(d.eps_mode == PXE_BN_EPS_CUDNN || d.eps_mode == PXE_BN_EPS_CPU, "batchnorm_backward: unknown eps_mode %d", d.eps_mode);
    Shape sh;
    int rc = check_shape(d.batch, d.channels, d.height, d.width, &sh, "batchnorm_backward");
    if (rc != PXE_OK) return rc;
    PXE_REQUIRE(d.workspace && d.workspace_bytes >= workspace_for(d.channels, sh.splits),
                "batchnorm_backward: workspace of %zu bytes, %zu needed", d.workspace_bytes, workspace_for(d.channels, sh.splits));
    PXE_REQUIRE(aligned16(d.workspace), "batchnorm_backward: workspace must be 16-byte aligned");
    DeviceInfo di;
    rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    float4* coeff4 = static_cast<float4*>(d.workspace);
    float2* partial = reinterpret_cast<float2*>(coeff4 + d.channels);
    ReduceParams rp{};
    rp.x = d.x; rp.dy = d.dy; rp.mean = d.save_mean; rp.partial = partial;
    rp.B = d.batch; rp.C = d.channels; rp.HW = (int)sh.hw; rp.per_plane = sh.split.per_plane; rp.chunk = sh.split.chunk; rp.items = sh.items;
    const bool vec_in = sh.hw % 4 == 0 && aligned16(d.x) && aligned16(d.dy);
    const dim3 rgrid((unsigned)d.channels, (unsigned)sh.splits);
    if (vec_in) {
        if (sh.warp_pieces) bn_reduce_kernel<true, true, true><<<rgrid, kThreads, 0, s>>>(rp);
        else bn_reduce_kernel<true, true, false><<<rgrid, kThreads, 0, s>>>(rp);
    } else {
        if (sh.warp_pieces) bn_reduce_kernel<true, false, true><<<rgrid, kThreads, 0, s>>>(rp);
        else bn_reduce_kernel<true, false, false><<<rgrid, kThreads, 0, s>>>(rp);
    }
    PXE_LAUNCH_OK("bn_reduce_kernel");

    BackwardFinal bf{};
    bf.partial = partial; bf.gamma = d.gamma; bf.save_mean = d.save_mean; bf.save_scale = d.save_scale;
    bf.dgamma = d.dgamma; bf.dbeta = d.dbeta; bf.coeff = coeff4;
    bf.eps = d.eps; bf.eps_mode = d.eps_mode; bf.C = d.channels; bf.splits = sh.splits; bf.n = (long long)d.batch * sh.hw;
    bn_backward_final_kernel<<<(d.channels + 3) / 4, 128, 0, s>>>(bf);
    PXE_LAUNCH_OK("bn_backward_final_kernel");

    ApplyParams ap{};
    ap.x = d.x; ap.dy = d.dy; ap.y = d.dx; ap.coeff4 = coeff4;
    const bool vec = sh.n_elems % 4 == 0 && aligned16(d.x) && aligned16(d.dy) && aligned16(d.dx);
    ap.units = (uint32_t)(vec ? sh.n_elems / 4 : sh.n_elems);
    ap.HW = (uint32_t)sh.hw;
    ap.div_hw = FastDiv((uint32_t)sh.hw);
    ap.div_c = FastDiv((uint32_t)d.channels);
    const unsigned grid = grid_for(ap.units, kThreads * 4, di.sm_count, 16);
    if (vec) bn_backward_apply_kernel<true><<<grid, kThreads, 0, s>>>(ap);
    else bn_backward_apply_kernel<false><<<grid, kThreads, 0, s>>>(ap);
    PXE_LAUNCH_OK("bn_backward_apply_kernel");
    return PXE_OK;
}
