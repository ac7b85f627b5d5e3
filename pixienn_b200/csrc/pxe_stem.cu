// First-layer convolution with its epilogue in one launch.
//
// The reference runs every convolution through cuDNN and then re-reads the result for batch norm / bias and the
// activation (include/cuda/ConvLayer.h:278-307).  For the network's first layer that is the worst case: 3 input
// channels make a GEMM with K = 27, no tensor-core kernel applies (cuDNN falls back to a SIMT kernel: 2.75 ms of a
// 38 ms YOLOv3-608 forward at 64 images), and the layer's output is the largest tensor of the whole network
// (64 x 32 x 608 x 608 = 3 GB), which the separate epilogue then reads and writes once more.  The layer is
// bound by that output traffic, not by arithmetic, so it is done here as a direct convolution: a block stages an
// input patch and the filters in shared memory, a thread accumulates 4 adjacent pixels x 8 output channels in
// registers (27 x 32 fused multiply-adds per pixel), applies y = act(a[k] * acc + b[k]) with the folded
// coefficients of pxe_fold_bn and stores the result once, in NCHW or channels-last.
//
// Supported: 3x3, stride 1, padding 1, dilation 1, one group, 1..4 input channels, 8..64 output channels in
// multiples of 8, NCHW input.  Anything else stays on the cuDNN call.
#include "pxe_common.cuh"

namespace pxe {
namespace {

constexpr int kStemThreads = 256;
constexpr int kStemTH = 16, kStemTW = 128;         // output tile: 16 rows x 128 columns, two rows per thread
constexpr int kStemPatchW = kStemTW + 4;           // columns x0-1 .. x0+128, padded to keep rows 16-byte multiples
constexpr int kStemMaxCin = 4, kStemMaxCout = 64;

// two floats in one 64-bit register, for fma.rn.f32x2
__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b, unsigned long long c)
{
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

struct StemParams {
    const float* x; long long xbs;                 // [B, CIN, H, W]
    const float* w;                                // [COUT, CIN, 3, 3]
    const float* a; const float* b;                // folded coefficients [COUT] (a may be null: 1 / 0)
    float* y; long long ybs, yps;                  // NCHW: batch stride; NHWC: pixel stride
    int B, H, W, cout, act;
    int tiles_x, tiles_y;
};

template <int CIN, bool NHWC, int ACT>
__global__ void __launch_bounds__(kStemThreads, 3)
stem_conv_kernel(const StemParams p)
{
    __shared__ __align__(16) float patch[kStemMaxCin][kStemTH + 2][kStemPatchW];
    __shared__ __align__(16) float wsm[kStemMaxCin * 9][kStemMaxCout];     // [ci*9 + ky*3 + kx][k]
    __shared__ float asm_[kStemMaxCout], bsm[kStemMaxCout];

    const int tile = blockIdx.x;
    const int b = tile / (p.tiles_x * p.tiles_y);
    const int t2 = tile - b * p.tiles_x * p.tiles_y;
    const int ty = t2 / p.tiles_x, tx = t2 - ty * p.tiles_x;
    const int y0 = ty * kStemTH, x0 = tx * kStemTW;
    const int H = p.H, W = p.W;

    // filters (transposed so that 4 output channels are one 128-bit shared-memory read) and coefficients
    for (int i = threadIdx.x; i < CIN * 9 * p.cout; i += kStemThreads) {
        const int k = i / (CIN * 9), r = i - k * (CIN * 9);
        wsm[r][k] = gld(p.w + i);
    }
    for (int i = threadIdx.x; i < p.cout; i += kStemThreads) {
        asm_[i] = p.a ? gld(p.a + i) : 1.0f;
        bsm[i] = p.b ? gld(p.b + i) : 0.0f;
    }
    // input patch rows y0-1 .. y0+8, columns x0-1 .. x0+128; zero outside the image
    const float* xin = p.x + (long long)b * p.xbs;
    for (int r = threadIdx.x >> 5; r < CIN * (kStemTH + 2); r += kStemThreads / 32) {       // one warp per patch row
        const int ci = r / (kStemTH + 2), py = r - ci * (kStemTH + 2);
        const int gy = y0 + py - 1;
        const bool row_in = gy >= 0 && gy < H;
        const float* src = xin + ((long long)ci * H + gy) * W + x0 - 1;
        for (int px = threadIdx.x & 31; px < kStemTW + 2; px += 32) {
            const int gx = x0 + px - 1;
            patch[ci][py][px] = (row_in && gx >= 0 && gx < W) ? gld(src + px) : 0.0f;
        }
    }
    __syncthreads();

    const int xg = threadIdx.x & 31;                              // 32 groups of 4 pixels; a warp takes rows w and w + 8
    const int gx = x0 + 4 * xg;
    if (gx >= W) return;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
    const int row = (threadIdx.x >> 5) + 8 * half;
    const int gy = y0 + row;
    if (gy >= H) break;
    for (int k0 = 0; k0 < p.cout; k0 += 8) {
        // Accumulators as pairs of output channels: fma.rn.f32x2 performs two independent IEEE fused
        // multiply-adds per instruction (same results as two scalar ones), which halves the issue slots the
        // 27 x 32 multiply-adds of a pixel take.
        unsigned long long acc2[4][4];
#pragma unroll
        for (int px = 0; px < 4; ++px)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc2[px][q] = 0ULL;
#pragma unroll 1
        for (int ci = 0; ci < CIN; ++ci)
#pragma unroll 1
            for (int ky = 0; ky < 3; ++ky) {
                // six input columns of this row: one 128-bit and one 64-bit shared-memory read
                const float4 i0 = *reinterpret_cast<const float4*>(&patch[ci][row + ky][4 * xg]);
                const float2 i1 = *reinterpret_cast<const float2*>(&patch[ci][row + ky][4 * xg + 4]);
                const unsigned long long in2[6] = {pack2(i0.x, i0.x), pack2(i0.y, i0.y), pack2(i0.z, i0.z),
                                                   pack2(i0.w, i0.w), pack2(i1.x, i1.x), pack2(i1.y, i1.y)};
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    const ulonglong2 w0 = *reinterpret_cast<const ulonglong2*>(&wsm[ci * 9 + ky * 3 + kx][k0]);
                    const ulonglong2 w1 = *reinterpret_cast<const ulonglong2*>(&wsm[ci * 9 + ky * 3 + kx][k0 + 4]);
                    const unsigned long long wq[4] = {w0.x, w0.y, w1.x, w1.y};
#pragma unroll
                    for (int px = 0; px < 4; ++px)
#pragma unroll
                        for (int q = 0; q < 4; ++q) acc2[px][q] = ffma2(in2[px + kx], wq[q], acc2[px][q]);
                }
            }
        float acc[4][8];
#pragma unroll
        for (int px = 0; px < 4; ++px)
#pragma unroll
            for (int q = 0; q < 4; ++q) unpack2(acc2[px][q], acc[px][2 * q], acc[px][2 * q + 1]);
        // epilogue and store
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float ca = asm_[k0 + k], cb = bsm[k0 + k];
#pragma unroll
            for (int px = 0; px < 4; ++px) {
                const float v = fmaf(ca, acc[px][k], cb);
                acc[px][k] = ACT < 0 ? activate_dyn(p.act, v) : activate<ACT, true>(v);
            }
        }
        if (NHWC) {
#pragma unroll
            for (int px = 0; px < 4; ++px) {
                if (gx + px >= W) break;
                float* dst = p.y + (((long long)b * H + gy) * W + gx + px) * p.yps + k0;
                if ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
                    // one 256-bit store: the pixel's 8 channels are exactly one 32-byte sector
                    if (gcheck(dst) && gcheck(dst + 7))
                    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                 :: "l"(dst), "f"(acc[px][0]), "f"(acc[px][1]), "f"(acc[px][2]), "f"(acc[px][3]),
                                    "f"(acc[px][4]), "f"(acc[px][5]), "f"(acc[px][6]), "f"(acc[px][7]) : "memory");
                } else {
                    gstv(dst, make_float4(acc[px][0], acc[px][1], acc[px][2], acc[px][3]));
                    gstv(dst + 4, make_float4(acc[px][4], acc[px][5], acc[px][6], acc[px][7]));
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float* dst = p.y + (long long)b * p.ybs + ((long long)(k0 + k) * H + gy) * W + gx;
                if (gx + 3 < W && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                    gstv(dst, make_float4(acc[0][k], acc[1][k], acc[2][k], acc[3][k]));
                } else {
#pragma unroll
                    for (int px = 0; px < 4; ++px)
                        if (gx + px < W) gst(dst + px, acc[px][k]);
                }
            }
        }
    }
    }
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" int pxe_conv_stem(pxe_stream_t stream, const pxe_stem_desc* dp)
{
    PXE_REQUIRE(dp != nullptr, "conv_stem: null descriptor");
    const pxe_stem_desc& d = *dp;
    PXE_REQUIRE(d.x && d.weights && d.y, "conv_stem: null pointer");
    PXE_REQUIRE(d.batch > 0 && d.height > 0 && d.width > 0, "conv_stem: non-positive shape");
    PXE_REQUIRE((d.a == nullptr) == (d.b == nullptr), "conv_stem: a and b go together");
    PXE_REQUIRE(valid_activation(d.act), "conv_stem: unknown activation %d", d.act);
    if (d.in_channels < 1 || d.in_channels > kStemMaxCin || d.out_channels < 8 || d.out_channels > kStemMaxCout
        || d.out_channels % 8 != 0)
        return set_error(PXE_ERR_UNSUPPORTED, "conv_stem: %d -> %d channels (supported: 1..%d input, 8..%d output in multiples of 8)",
                         d.in_channels, d.out_channels, kStemMaxCin, kStemMaxCout);
    const long long hw = (long long)d.height * d.width;
    PXE_REQUIRE(d.x_batch_stride == 0 || d.x_batch_stride >= hw * d.in_channels, "conv_stem: x_batch_stride too small");
    StemParams p{};
    p.x = d.x; p.xbs = d.x_batch_stride ? d.x_batch_stride : hw * d.in_channels;
    p.w = d.weights; p.a = d.a; p.b = d.b; p.y = d.y;
    p.B = d.batch; p.H = d.height; p.W = d.width; p.cout = d.out_channels; p.act = d.act;
    p.tiles_x = (d.width + kStemTW - 1) / kStemTW;
    p.tiles_y = (d.height + kStemTH - 1) / kStemTH;
    const long long tiles = (long long)p.tiles_x * p.tiles_y * d.batch;
    PXE_REQUIRE(tiles <= 0x7fffffffLL, "conv_stem: too many tiles");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d.y_is_nhwc) {
        p.yps = d.y_stride ? d.y_stride : d.out_channels;
        PXE_REQUIRE(p.yps >= d.out_channels, "conv_stem: y pixel stride smaller than the channel count");
        PXE_REQUIRE(aligned16(d.y) && p.yps % 4 == 0, "conv_stem: channels-last output must keep 16-byte alignment");
    } else {
        p.ybs = d.y_stride ? d.y_stride : hw * d.out_channels;
        PXE_REQUIRE(p.ybs >= hw * d.out_channels, "conv_stem: y_batch_stride too small");
    }
#define PXE_STEM_LAUNCH2(CIN, ACT)                                                                      \
    do {                                                                                               \
        if (d.y_is_nhwc) stem_conv_kernel<CIN, true, ACT><<<(unsigned)tiles, kStemThreads, 0, s>>>(p); \
        else stem_conv_kernel<CIN, false, ACT><<<(unsigned)tiles, kStemThreads, 0, s>>>(p);            \
    } while (0)
    // the activations the presets use are compiled in; the rest go through the run-time switch
#define PXE_STEM_LAUNCH(CIN)                                                                           \
    do {                                                                                               \
        switch (d.act) {                                                                               \
        case PXE_ACT_LEAKY: PXE_STEM_LAUNCH2(CIN, PXE_ACT_LEAKY); break;                               \
        case PXE_ACT_MISH: PXE_STEM_LAUNCH2(CIN, PXE_ACT_MISH); break;                                 \
        case PXE_ACT_SWISH: PXE_STEM_LAUNCH2(CIN, PXE_ACT_SWISH); break;                               \
        default: PXE_STEM_LAUNCH2(CIN, -1); break;                                                     \
        }                                                                                              \
    } while (0)
    switch (d.in_channels) {
    case 1: PXE_STEM_LAUNCH(1); break;
    case 2: PXE_STEM_LAUNCH(2); break;
    case 3: PXE_STEM_LAUNCH(3); break;
    default: PXE_STEM_LAUNCH(4); break;
    }
#undef PXE_STEM_LAUNCH2
#undef PXE_STEM_LAUNCH
    PXE_LAUNCH_OK("stem_conv_kernel");
    return PXE_OK;
}
