// Max pooling (px::maxPoolForwardGpu, src/MaxPoolKernels.cu:10-59) and the SPP block
// (stride-1 pools of one input with several kernel sizes) as single-read kernels.
//
// Semantics kept bit for bit: output extent (in + padding - kernel)/stride + 1, window origin
// -padding/2 (C truncation), taps outside the input are skipped, the first tap is always taken
// and later taps replace it only when strictly greater (so the first maximum wins and a NaN in
// the first tap sticks), the index is the flat position in a dense [B,C,H,W] input.
#include <algorithm>
#include <type_traits>

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
                const float v = gld(plane + (iy * p.W + ix));
                if (best_idx < 0 || v > best) {
                    best = v;
                    best_idx = ix + p.W * (iy + p.H * ((int)c + p.C * (int)b));
                }
            }
        }
        gst(p.y + ((long long)b * p.ybs + ((long long)c * p.OH + oh) * p.OW + ow), best);
        if (WITH_INDEX) gst(p.idx + (((long long)b * p.C + c) * p.OH * p.OW + (long long)oh * p.OW + ow), best_idx);
    }
}

// Kernel 2, stride 1 (YOLOv3-tiny's last pool, 13x13 or 19x19 planes): a warp per plane walks the outputs in
// flat order, so loads and stores are coalesced, the four taps of neighbouring outputs come out of L1, and the
// row / column of an output advance by constants instead of three divisions per output.  A tap outside the plane
// repeats the window's first tap, which the scan's "strictly greater" never picks.
template <bool WITH_INDEX>
__global__ void __launch_bounds__(kThreads)
maxpool_k2s1_kernel(const PoolParams p, uint32_t planes)
{
    const uint32_t lane = threadIdx.x & 31;
    const int W = p.W, H = p.H, OW = p.OW, n_out = p.OH * p.OW;
    const int step_y = 32 / OW, step_x = 32 - step_y * OW;
    for (uint32_t plane = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); plane < planes; plane += gridDim.x * (kThreads / 32)) {
        uint32_t b, c;
        p.div_c.divmod(plane, b, c);
        const float* src = p.x + (long long)b * p.xbs + (long long)c * H * W;
        float* dst = p.y + (long long)b * p.ybs + (long long)c * n_out;
        int* idx = WITH_INDEX ? p.idx + (long long)plane * n_out : nullptr;
        const int plane_base = (int)plane * H * W;
        int y = (int)lane / OW, x = (int)lane - y * OW;
        for (int i = (int)lane; i < n_out; i += 32) {
            const int at = y * W + x;
            const int dx = x + 1 < W ? 1 : 0, dy = y + 1 < H ? W : 0;
            const float v00 = gld(src + at), v01 = gld(src + (at + dx)), v10 = gld(src + (at + dy)), v11 = gld(src + (at + dy + dx));
            float best = v00;
            int where = at;
            if (v01 > best) { best = v01; where = at + dx; }
            if (v10 > best) { best = v10; where = at + dy; }
            if (v11 > best) { best = v11; where = at + dy + dx; }
            gst(dst + i, best);
            if (WITH_INDEX) gst(idx + i, plane_base + where);
            y += step_y; x += step_x;
            if (x >= OW) { x -= OW; ++y; }
        }
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
        const float ca = p.a ? gld(p.a + c) : 1.0f, cb = p.a ? gld(p.b + c) : 0.0f;
        float* yid = p.yid ? p.yid + (long long)b * p.yidbs + (long long)c * HW : nullptr;
        for (int i = threadIdx.x; i < HW; i += kThreads) {
            float v = gld(src + i);
            if (p.a) v = fmaf(ca, v, cb);
            v = activate_fast_dyn(p.act, v);
            tile[i] = v;
            if (yid) gst(yid + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < HW; i += kThreads) tile[i] = gld(src + i);
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
            gst(p.y[k] + ((long long)b * p.ybs[k] + (long long)c * HW + i), m);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// The 5 / 9 / 13 block on planes small enough for three copies per warp in shared memory (13x13, 19x19,
// 20x20 ...): a warp per plane, several planes per block, no block-wide barrier.
//
// Rows first: a 9-wide row maximum is a 5-wide one over 5-wide ones, a 13-wide one three of them, with taps
// outside the plane skipped at every level, so the row maxima for 5, 9 and 13 are a chain of three 5-wide passes
// (four neighbouring outputs per lane from eight inputs with nine comparisons, 128-bit reads and writes).  Then,
// for each pool, one column pass over its row maxima: a lane reads the 2R + 4 rows that four output rows need
// and takes the four windows of 2R + 1 from them with 2R + 7 comparisons (shared partial maxima) -- 8 / 12 / 16
// vector reads and no intermediate plane, where a chain of 5-high passes would go through shared memory one to
// three times.  That matters: the kernel is bound by shared-memory bandwidth, not by comparisons.  No pass needs
// edge tests on rows: the planes sit between rows of -infinity, which no comparison "v > best" picks; the ends of
// a row are two selects in the row pass.
//
// What the reference's scan returns (src/MaxPoolKernels.cu:26-40) is the FIRST maximum in row-major order (it
// matters for -0 / +0) unless the window's first tap is a NaN.  Every combination here keeps the left (upper)
// operand on ties and takes its operands in scan order, a chain of windows picks the first position that any
// of them would, and rows come before columns, so the value is the one the scan finds.  A plane that holds a NaN
// is not cascaded at all: its warp evaluates the scan itself for every output.
// ---------------------------------------------------------------------------------------------
constexpr int kCascadeWarps = 4;

struct CascadeParams {
    SppParams s;
    FastDiv div_c;
    uint32_t planes;
    int levels;              // 1, 2, 3: the chain runs up to the window 4*levels + 1
    int pool_of_level[3];    // which of the requested pools has the window 5, 9, 13; -1 = not asked for
};

__device__ __forceinline__ float keep_first(float m, float v) { return v > m ? v : m; }

// EXACT: the left operand stays on ties (first of -0 / +0 wins); otherwise one max instruction, which is the same
// value whenever equal operands are the same bits (a plane without a negative zero) and no operand is a NaN
template <bool EXACT>
__device__ __forceinline__ float comb(float m, float v) { return EXACT ? keep_first(m, v) : fmaxf(m, v); }

// four windows of five over v0..v7: outputs for the positions of v2..v5
template <bool EXACT>
__device__ __forceinline__ void window5x4(float v0, float v1, float v2, float v3, float v4, float v5, float v6, float v7,
                                          float& o0, float& o1, float& o2, float& o3)
{
    const float c12 = comb<EXACT>(v1, v2), c34 = comb<EXACT>(v3, v4), c56 = comb<EXACT>(v5, v6);
    const float p = comb<EXACT>(c12, c34), q = comb<EXACT>(c34, c56);
    o0 = comb<EXACT>(v0, p);
    o1 = comb<EXACT>(p, v5);
    o2 = comb<EXACT>(v2, q);
    o3 = comb<EXACT>(q, v7);
}

// D = 5-wide row maxima of S, rows 0..H-1.  Rows are 4*nxg floats apart with nothing between them, so unit u (four
// columns of one row) is the u-th 128-bit vector of the plane: consecutive lanes read and write consecutive
// vectors (no bank conflicts), and the two values to the left and right of a unit are its neighbouring lanes'
// (a shuffle); the first and last lane fetch theirs, and at the ends of a row they are -infinity.
template <bool EXACT>
__device__ __forceinline__ void cascade_rows(const float* S, float* D, int H, int nxg, uint32_t lane)
{
    const int units = H * nxg;
    const float4* S4 = reinterpret_cast<const float4*>(S);
    float4* D4 = reinterpret_cast<float4*>(D);
    const int step_x = 32 % nxg;
    int xg = (int)lane % nxg;
    for (int base = 0; base < units; base += 32) {
        const int u = base + (int)lane;
        const bool active = u < units;
        const float4 m = active ? S4[u] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        float2 l = make_float2(__shfl_up_sync(0xffffffffu, m.z, 1), __shfl_up_sync(0xffffffffu, m.w, 1));
        float2 r = make_float2(__shfl_down_sync(0xffffffffu, m.x, 1), __shfl_down_sync(0xffffffffu, m.y, 1));
        if (lane == 0 && active && xg > 0) l = *reinterpret_cast<const float2*>(S + 4 * u - 2);
        if (lane == 31 && active && xg < nxg - 1) r = *reinterpret_cast<const float2*>(S + 4 * u + 4);
        if (xg == 0) l = make_float2(-INFINITY, -INFINITY);
        if (xg == nxg - 1) r = make_float2(-INFINITY, -INFINITY);
        float4 o;
        window5x4<EXACT>(l.x, l.y, m.x, m.y, m.z, m.w, r.x, r.y, o.x, o.y, o.z, o.w);
        if (active) D4[u] = o;
        xg += step_x;
        if (xg >= nxg) xg -= nxg;
    }
}

// four windows of 2*R + 1 over v[0 .. 2*R + 3], taken in order: o[j] = window v[j .. j + 2*R]
template <bool EXACT, int R>
__device__ __forceinline__ void window_x4(const float (&v)[2 * R + 4], float (&o)[4])
{
    float core = v[3];
#pragma unroll
    for (int i = 4; i <= 2 * R; ++i) core = comb<EXACT>(core, v[i]);
    const float l12 = comb<EXACT>(v[1], v[2]), r12 = comb<EXACT>(v[2 * R + 1], v[2 * R + 2]);
    o[0] = comb<EXACT>(comb<EXACT>(v[0], l12), core);
    o[1] = comb<EXACT>(comb<EXACT>(l12, core), v[2 * R + 1]);
    o[2] = comb<EXACT>(comb<EXACT>(v[2], core), r12);
    o[3] = comb<EXACT>(core, comb<EXACT>(r12, v[2 * R + 3]));
}

// Column maxima over 2*R + 1 rows of S for rows 0..H-1, columns 0..4*nxg-1, straight from the 2*R + 4 rows a strip
// of four output rows needs (no intermediate planes): into the buffer D (rows past H-1 are left alone) or, with
// TO_GLOBAL, as vector stores into a dense W-wide plane (W % 4 == 0).  NC columns per lane.
template <bool EXACT, int R, int NC, bool TO_GLOBAL, bool SCALAR = false>
__device__ __forceinline__ void cascade_cols(const float* S, float* D, int H, int nys, int nxg, int SW, int dw, uint32_t lane,
                                             int W = 0)
{
    using Vec = typename std::conditional<NC == 4, float4, float2>::type;
    const int ncg = 4 * nxg / NC;
    const int units = nys * ncg;
    const int step_y = 32 / ncg, step_x = 32 - step_y * ncg;
    int ys = (int)lane / ncg, cg = (int)lane - ys * ncg;
    for (int u = (int)lane; u < units; u += 32) {
        const float* s = S + (4 * ys - R) * SW + NC * cg;
        float v[NC][2 * R + 4];
#pragma unroll
        for (int j = 0; j < 2 * R + 4; ++j) {
            const Vec t = *reinterpret_cast<const Vec*>(s + j * SW);
            v[0][j] = t.x; v[1][j] = t.y;
            if constexpr (NC == 4) { v[2][j] = t.z; v[3][j] = t.w; }
        }
        float o[NC][4];
#pragma unroll
        for (int c = 0; c < NC; ++c) window_x4<EXACT, R>(v[c], o[c]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (4 * ys + j >= H) continue;
            if constexpr (SCALAR) {
                // a dense plane whose rows are not vector-aligned: element stores, columns past W - 1 dropped
                float* row = D + (4 * ys + j) * dw + NC * cg;
#pragma unroll
                for (int c = 0; c < NC; ++c)
                    if (NC * cg + c < W) gst(row + c, o[c][j]);
            } else {
                Vec t;
                t.x = o[0][j]; t.y = o[1][j];
                if constexpr (NC == 4) { t.z = o[2][j]; t.w = o[3][j]; }
                gstv(D + (4 * ys + j) * dw + NC * cg, t);        // D: an output plane, or shared memory
            }
        }
        ys += step_y; cg += step_x;
        if (cg >= ncg) { cg -= ncg; ++ys; }
    }
}

// the pools of one plane held in X: out[l] receives the pool of size 4*l + 5 (nullptr: not asked for)
template <bool VEC, bool EXACT>
__device__ __forceinline__ void cascade_plane(float* X, float* A, float* B, float* const* out, int levels, int H, int W,
                                              int nxg, int nys, int SW, uint32_t lane)
{
    // 5: rows X -> A; 9: rows A -> B; 13: rows B -> A.  Columns go straight out: as vectors, or element by element where
    // the planes are not aligned for them.
    cascade_rows<EXACT>(X, A, H, nxg, lane);
    __syncwarp();
    if (out[0]) {
        if (VEC) cascade_cols<EXACT, 2, 4, true>(A, out[0], H, nys, nxg, SW, W, lane);
        else {
            cascade_cols<EXACT, 2, 4, true, true>(A, out[0], H, nys, nxg, SW, W, lane, W);
            __syncwarp();
        }
    }
    if (levels > 1) {
        cascade_rows<EXACT>(A, B, H, nxg, lane);
        __syncwarp();
        if (out[1]) {
            if (VEC) cascade_cols<EXACT, 4, 2, true>(B, out[1], H, nys, nxg, SW, W, lane);
            else {
                cascade_cols<EXACT, 4, 2, true, true>(B, out[1], H, nys, nxg, SW, W, lane, W);
                __syncwarp();
            }
        }
    }
    if (levels > 2) {
        cascade_rows<EXACT>(B, A, H, nxg, lane);
        __syncwarp();
        if (VEC) cascade_cols<EXACT, 6, 2, true>(A, out[2], H, nys, nxg, SW, W, lane);
        else {
            cascade_cols<EXACT, 6, 2, true, true>(A, out[2], H, nys, nxg, SW, W, lane, W);
        }
    }
}

// VEC: W % 4 == 0 and every plane of x, of the outputs and of the identity output starts on a 16-byte boundary
template <bool VEC>
__global__ void __launch_bounds__(kCascadeWarps * 32, 8)
spp_cascade_kernel(const CascadeParams cp)
{
    extern __shared__ float4 cascade_smem[];
    const SppParams& p = cp.s;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int H = p.H, W = p.W, HW = H * W;
    const int nxg = (W + 3) >> 2, nys = (H + 3) >> 2;
    const int SW = 4 * nxg;                           // floats from one row to the next: no gap
    // per warp: X, rows 0 .. 4*nys - 1 (never a column source) | A, rows -6 .. 4*nys + 5 (source of the 5- and 13-high
    // windows) | B, rows -4 .. 4*nys + 3 (source of the 9-high ones); the rows outside the plane stay -infinity
    const int rows_all = 12 * nys + 20;
    float* base = reinterpret_cast<float*>(cascade_smem) + (size_t)warp * rows_all * SW;
    float* X = base;
    float* A = X + (4 * nys + 6) * SW;
    float* B = A + (4 * nys + 6 + 4) * SW;
    for (int i = (int)lane; i < rows_all * nxg; i += 32)
        reinterpret_cast<float4*>(base)[i] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    __syncwarp();
    const bool epilogue = p.a != nullptr || p.act != PXE_ACT_LINEAR;

    for (uint32_t plane = blockIdx.x * kCascadeWarps + warp; plane < cp.planes; plane += gridDim.x * kCascadeWarps) {
        uint32_t b, c;
        cp.div_c.divmod(plane, b, c);
        const float* src = p.x + (long long)b * p.xbs + (long long)c * HW;
        float* yid = p.yid ? p.yid + (long long)b * p.yidbs + (long long)c * HW : nullptr;
        const float ca = p.a ? gld(p.a + c) : 1.0f, cb = p.a ? gld(p.b + c) : 0.0f;
        bool nan = false, negzero = false;
        if (VEC) {
            for (int u = (int)lane; u < HW / 4; u += 32) {
                float4 v = gldv<float4>(src + 4 * u);
                if (epilogue) {
                    if (p.a) { v.x = fmaf(ca, v.x, cb); v.y = fmaf(ca, v.y, cb); v.z = fmaf(ca, v.z, cb); v.w = fmaf(ca, v.w, cb); }
                    v.x = activate_fast_dyn(p.act, v.x); v.y = activate_fast_dyn(p.act, v.y);
                    v.z = activate_fast_dyn(p.act, v.z); v.w = activate_fast_dyn(p.act, v.w);
                }
                nan |= (v.x != v.x) | (v.y != v.y) | (v.z != v.z) | (v.w != v.w);
                negzero |= (__float_as_uint(v.x) == 0x80000000u) | (__float_as_uint(v.y) == 0x80000000u)
                           | (__float_as_uint(v.z) == 0x80000000u) | (__float_as_uint(v.w) == 0x80000000u);
                reinterpret_cast<float4*>(X)[u] = v;             // W == 4*nxg: the plane as it lies in memory
                if (yid) gstv(yid + 4 * u, v);
            }
        } else {
            // (columns W .. 4*nxg - 1 of X are never written: they keep the -infinity of the start)
            const int step_y = 32 / W, step_x = 32 - step_y * W;
            int y = (int)lane / W, x = (int)lane - y * W;
            for (int i = (int)lane; i < HW; i += 32) {
                float v = gld(src + i);
                if (epilogue) {
                    if (p.a) v = fmaf(ca, v, cb);
                    v = activate_fast_dyn(p.act, v);
                }
                nan |= v != v;
                negzero |= __float_as_uint(v) == 0x80000000u;
                X[y * SW + x] = v;
                if (yid) gst(yid + i, v);
                y += step_y; x += step_x;
                if (x >= W) { x -= W; ++y; }
            }
        }
        nan = __any_sync(0xffffffffu, nan);
        negzero = __any_sync(0xffffffffu, negzero);
        __syncwarp();
        float* out[3];
#pragma unroll
        for (int l = 0; l < 3; ++l) {
            const int k = cp.pool_of_level[l];
            out[l] = k >= 0 ? p.y[k] + (long long)b * p.ybs[k] + (long long)c * HW : nullptr;
        }

        if (nan) {
            // the scan itself (first tap taken as it is, a later one only when strictly greater), from X
#pragma unroll
            for (int l = 0; l < 3; ++l) {
                if (!out[l]) continue;
                const int K = 5 + 4 * l, off = -(K - 1) / 2;
                for (int i = (int)lane; i < HW; i += 32) {
                    const int oy = i / W, ox = i - oy * W;
                    const int ya = max(oy + off, 0), yb = min(oy + off + K, H);
                    const int xa = max(ox + off, 0), xb = min(ox + off + K, W);
                    float best = X[ya * SW + xa];
                    for (int iy = ya; iy < yb; ++iy)
                        for (int ix = xa; ix < xb; ++ix) best = keep_first(best, X[iy * SW + ix]);
                    gst(out[l] + i, best);
                }
            }
            __syncwarp();
            continue;
        }

        if (negzero) cascade_plane<VEC, true>(X, A, B, out, cp.levels, H, W, nxg, nys, SW, lane);
        else cascade_plane<VEC, false>(X, A, B, out, cp.levels, H, W, nxg, nys, SW, lane);
        __syncwarp();
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
    for (int i = lane; i < area; i += 32) sum += gld(src + i);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) gst(y + ((long long)b * ybs + c), sum / (float)(area > 1 ? area : 1));
}

}  // namespace
}  // namespace pxe

using namespace pxe;

namespace {
// shared memory of the 5 / 9 / 13 chain for planes of this size; 0 = does not fit
size_t cascade_bytes(const DeviceInfo& di, int height, int width)
{
    const int nxg = (width + 3) / 4, nys = (height + 3) / 4;
    const size_t bytes = (size_t)kCascadeWarps * (12 * nys + 20) * (4 * nxg) * sizeof(float);
    return bytes <= 96 * 1024 && bytes <= (size_t)di.max_smem_optin ? bytes : 0;
}

int spp_launch(pxe_stream_t stream, const float* x, long long x_batch_stride, int batch, int channels,
               int height, int width, int n_pools, const int* kernels, float* const* ys,
               const long long* y_batch_strides, const float* a, const float* b, int act, float* y_identity,
               long long y_identity_batch_stride, bool fused);
}  // namespace

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
    // one of the SPP block's windows on its own: the chain of 5-wide windows, where the plane fits it
    if (stride == 1 && !indexes && padding == kernel - 1 && (kernel == 5 || kernel == 9 || kernel == 13)
        && cascade_bytes(di, height, width) != 0)
        return spp_launch(stream, x, x_batch_stride, batch, channels, height, width, 1, &kernel, &y, &y_batch_stride,
                          nullptr, nullptr, PXE_ACT_LINEAR, nullptr, 0, false);
    PoolParams p{};
    p.x = x; p.y = y; p.idx = indexes;
    p.xbs = x_batch_stride ? x_batch_stride : chw;
    p.ybs = y_batch_stride ? y_batch_stride : ochw;
    p.C = channels; p.H = height; p.W = width; p.OH = oh; p.OW = ow;
    p.kernel = kernel; p.stride = stride; p.offset = -padding / 2;
    PXE_REQUIRE((long long)batch * ochw < (1LL << 32), "maxpool: too many outputs for one launch");
    p.total = (uint32_t)((long long)batch * ochw);
    p.div_ow = FastDiv((uint32_t)ow); p.div_oh = FastDiv((uint32_t)oh); p.div_c = FastDiv((uint32_t)channels);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (kernel == 2 && stride == 1 && padding <= 1 && (long long)batch * channels <= 0x7fffffffLL) {
        const uint32_t planes = (uint32_t)(batch * channels);
        const unsigned blocks = std::min((planes + kThreads / 32 - 1) / (kThreads / 32), (uint32_t)di.sm_count * 8u);
        if (indexes) maxpool_k2s1_kernel<true><<<blocks, kThreads, 0, s>>>(p, planes);
        else maxpool_k2s1_kernel<false><<<blocks, kThreads, 0, s>>>(p, planes);
        PXE_LAUNCH_OK("maxpool_k2s1_kernel");
        return PXE_OK;
    }
    unsigned grid = grid_for(p.total, kThreads, di.sm_count, 16);
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
    // the 5 / 9 / 13 block (or its first one or two pools) on planes whose three copies per warp fit
    {
        bool chain = n_pools <= 3;
        int pool_of_level[3] = {-1, -1, -1}, levels = 0;
        for (int k = 0; k < n_pools && chain; ++k) {
            const int l = (kernels[k] - 5) / 4;
            chain = kernels[k] >= 5 && kernels[k] <= 13 && kernels[k] == 5 + 4 * l && pool_of_level[l] < 0;
            if (chain) { pool_of_level[l] = k; levels = std::max(levels, l + 1); }
        }
        const size_t bytes = cascade_bytes(di, height, width);
        if (chain && bytes != 0 && (long long)batch * channels <= 0x7fffffffLL) {
            CascadeParams cp{};
            cp.s = p;
            cp.div_c = FastDiv((uint32_t)channels);
            cp.planes = (uint32_t)(batch * channels);
            cp.levels = levels;
            for (int l = 0; l < 3; ++l) cp.pool_of_level[l] = pool_of_level[l];
            auto a16 = [](const void* ptr, long long bs) { return ((uintptr_t)ptr & 15) == 0 && bs % 4 == 0; };
            bool vec = width % 4 == 0 && a16(x, p.xbs) && (!y_identity || a16(y_identity, p.yidbs));
            for (int k = 0; k < n_pools; ++k) vec = vec && a16(ys[k], p.ybs[k]);
            auto kern = vec ? spp_cascade_kernel<true> : spp_cascade_kernel<false>;
            if (bytes > 48 * 1024)
                PXE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
            int resident = 0;
            PXE_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, kCascadeWarps * 32, bytes));
            if (resident < 1) resident = 1;
            const unsigned want = (cp.planes + kCascadeWarps - 1) / kCascadeWarps;
            const unsigned grid = std::min(want, (unsigned)(di.sm_count * resident));
            kern<<<grid, kCascadeWarps * 32, bytes, static_cast<cudaStream_t>(stream)>>>(cp);
            PXE_LAUNCH_OK("spp_cascade_kernel");
            return PXE_OK;
        }
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
