// Fused convolution epilogue: batch-norm inference (folded to one multiply-add per element),
// bias, activation, and optionally the residual add of a following shortcut layer, the 2x2
// stride-2 max pool of a following maxpool layer, and a store into a concat slot -- one pass
// over the conv output instead of the reference's separate full-tensor passes
// (include/cuda/ConvLayer.h:284-307, include/cuda/ShortcutLayer.h:23-34,
// include/cuda/MaxPoolLayer.h:36-42, include/cuda/RouteLayer.h:21-44).
//
// Memory-bound by design: 4 bytes read + 4 bytes written per element (12 with a residual,
// 4 + 1 with pooled-only output).  No tensor cores: nothing here is a contraction.
//
// Work split.  The element space [batch*channels planes][H*W] is cut into contiguous chunks,
// one per thread block.  A block first writes, for every plane its chunk touches, the folded
// batch-norm coefficients and the plane's image / channel numbers into shared memory; the
// streaming loop then needs one shared-memory read and one exact division per 128-bit vector.
#include "pxe_common.cuh"

namespace pxe {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kMaxPlanesPerBlock = 3000;   // 16 B each -> 48 KB of shared memory at most

struct PlaneEntry {
    float a, b;          // y = a*x + b
    int image;           // batch index of the plane
    int chan;            // channel; bit 30 set = "identity entry" for PXE_ACT_YOLO_HEAD
};

// image / channel numbers of a plane without the table (used to issue the first loads of a block
// before its table exists)
struct PlaneId { uint32_t image, chan; };

struct EpiParams {
    const float* x; float* y; float* y2; const float* res; float* ypool;
    long long xbs, ybs, y2bs, rbs, pbs;
    const float *gamma, *beta, *mean, *var, *bias;
    const float *fa, *fb;      // coefficients folded once by the caller (pxe_fold_bn): no per-block table, no barrier
    float eps; int eps_mode;
    int C, H, W, HW;
    int yolo_entries;
    float ralpha, rbeta; int res_act;
    // streaming kernels: `units` of work (vectors or elements), `chunk` per block
    uint32_t units, chunk;
    FastDiv div_plane;   // units per plane (vector path) or HW (scalar / straddle path)
    FastDiv div_c;
    // pool kernels
    int OH, OW, OWV;
    FastDiv div_owv, div_ohowv;
    // even pool kernel: row pairs per plane (OH), units per image, dense-output flags
    FastDiv div_oh;
    uint32_t units_per_image;
    int y_dense, pool_dense;
    int pool_general;          // host side only: skip the specialised pooled kernels
    int flat_ok;               // host side only: groups of four planes are whole aligned vectors (flat pooled kernel)
};

// Folded coefficients and image / channel numbers of plane `pl` (= image*C + channel).
__device__ __forceinline__ PlaneEntry make_entry(const EpiParams& p, uint32_t pl)
{
    const uint32_t img = p.div_c.div(pl);
    const uint32_t c = pl - img * (uint32_t)p.C;
    float a = 1.0f, b = 0.0f;
    if (p.fa) {
        a = gld(p.fa + c); b = gld(p.fb + c);
    } else {
        if (p.gamma) {
            const float v = gld(p.var + c);
            const float denom = p.eps_mode == PXE_BN_EPS_CPU ? (sqrtf(v) + p.eps) : sqrtf(v + p.eps);
            a = gld(p.gamma + c) / denom;
            b = gld(p.beta + c) - gld(p.mean + c) * a;
        }
        if (p.bias) b += gld(p.bias + c);
    }
    int chan = (int)c;
    if (p.yolo_entries > 0) {
        const uint32_t e = c % (uint32_t)p.yolo_entries;
        if (e == 2 || e == 3) chan |= (1 << 30);
    }
    PlaneEntry t;
    t.a = a; t.b = b; t.image = (int)img; t.chan = chan;
    return t;
}

__device__ __forceinline__ void build_table(const EpiParams& p, PlaneEntry* tab, uint32_t plane_lo,
                                            uint32_t plane_hi)
{
    for (uint32_t pl = plane_lo + threadIdx.x; pl <= plane_hi; pl += blockDim.x)
        tab[pl - plane_lo] = make_entry(p, pl);
}

// The entry of plane `plane_lo + pl`: from the block's table, or, with coefficients the caller folded once per layer,
// straight from their two arrays (a warp's lanes mostly share a channel: one broadcast load each from L1).  In that
// form a block builds no table and meets no barrier.
__device__ __forceinline__ PlaneEntry entry_of(const EpiParams& p, const PlaneEntry* tab, uint32_t plane_lo, uint32_t pl)
{
    if (p.fa == nullptr) return tab[pl];
    const uint32_t q = plane_lo + pl;
    const uint32_t img = p.div_c.div(q);
    const uint32_t c = q - img * (uint32_t)p.C;
    int chan = (int)c;
    if (p.yolo_entries > 0) {
        const uint32_t e = c % (uint32_t)p.yolo_entries;
        if (e == 2 || e == 3) chan |= (1 << 30);
    }
    PlaneEntry t;
    t.a = gld(p.fa + c); t.b = gld(p.fb + c); t.image = (int)img; t.chan = chan;
    return t;
}

template <int ACT, bool AFFINE>
__device__ __forceinline__ float apply_one(float v, const PlaneEntry& t)
{
    if (AFFINE) v = fmaf(t.a, v, t.b);
    if (ACT == PXE_ACT_YOLO_HEAD) return (t.chan & (1 << 30)) ? v : act_logistic(v);
    return activate<ACT, true>(v);
}

__device__ __forceinline__ float residual_one(float v, float r, const EpiParams& p)
{
    // alpha*v + beta*r as the reference's CUDA kernel evaluates it (src/ShortcutKernel.cu:41,
    // contracted to one fused multiply-add by nvcc's default -fmad=true)
    return activate_dyn(p.res_act, fmaf(p.ralpha, v, p.rbeta * r));
}

// ---------------------------------------------------------------------------------------------
// MODE 0: plane-aligned vectors.  HW % 4 == 0 and every base pointer / batch stride keeps
//         16-byte alignment, so a float4 never crosses a plane.
// MODE 1: dense straddling vectors.  x, y (y2, res) are densely packed and 16-byte aligned but
//         HW % 4 != 0 (13x13, 19x19 ...): a float4 may span two planes; HW >= 4.
// MODE 2: scalar, anything goes.
// ---------------------------------------------------------------------------------------------
template <int ACT, bool AFFINE, bool RES, int MODE>
__global__ void __launch_bounds__(kThreads, 5)
epilogue_kernel(const EpiParams p)
{
    extern __shared__ PlaneEntry tab[];
    const uint32_t lo = blockIdx.x * p.chunk;
    if (lo >= p.units) return;
    uint32_t hi = lo + p.chunk;
    if (hi > p.units) hi = p.units;

    constexpr int VW = (MODE == 2) ? 1 : 4;
    // element index of a unit = unit * VW; plane of an element = elem / HW
    uint32_t plane_lo, plane_hi;
    if (MODE == 0) {
        plane_lo = p.div_plane.div(lo);
        plane_hi = p.div_plane.div(hi - 1);
    } else {
        plane_lo = p.div_plane.div(lo * VW);
        plane_hi = p.div_plane.div((hi - 1) * VW + (VW - 1));
    }

    // Every thread runs the same number of rounds (the barrier below sits inside the loop).  The
    // first round issues its global loads BEFORE the coefficient table is built, so the table's own
    // parameter loads and the square roots overlap the first wave of data instead of preceding it.
    // With a residual every vector has two loads in flight: half the unroll keeps the bytes in flight per
    // thread (64) and the registers of the plain form, so that five blocks stay resident per SM.
    constexpr int UN = RES ? kUnroll / 2 : kUnroll;
    const uint32_t step = kThreads * UN;
    const uint32_t rounds = (hi - lo + step - 1) / step;
    for (uint32_t rd = 0; rd < rounds; ++rd) {
        const uint32_t base = lo + rd * step + threadIdx.x;
        if (MODE == 0) {
            float4 v[UN];
            float4 r[UN];
            uint32_t off[UN];          // offset inside one image: C*H*W < 2^31
            uint32_t pl[UN], img[UN];
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = base + k * kThreads;
                if (u < hi) {
                    uint32_t q, rem, c;
                    p.div_plane.divmod(u, q, rem);
                    p.div_c.divmod(q, img[k], c);
                    pl[k] = q - plane_lo;
                    off[k] = c * (uint32_t)p.HW + rem * 4;
                    v[k] = gldv<float4>(p.x + (long long)img[k] * p.xbs + off[k]);
                    if (RES) r[k] = gldv<float4>(p.res + (long long)img[k] * p.rbs + off[k]);
                }
            }
            if (rd == 0 && p.fa == nullptr) {
                build_table(p, tab, plane_lo, plane_hi);
                __syncthreads();
            }
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = base + k * kThreads;
                if (u < hi) {
                    const PlaneEntry t = entry_of(p, tab, plane_lo, pl[k]);
                    float4 o;
                    o.x = apply_one<ACT, AFFINE>(v[k].x, t);
                    o.y = apply_one<ACT, AFFINE>(v[k].y, t);
                    o.z = apply_one<ACT, AFFINE>(v[k].z, t);
                    o.w = apply_one<ACT, AFFINE>(v[k].w, t);
                    if (RES) {
                        o.x = residual_one(o.x, r[k].x, p);
                        o.y = residual_one(o.y, r[k].y, p);
                        o.z = residual_one(o.z, r[k].z, p);
                        o.w = residual_one(o.w, r[k].w, p);
                    }
                    if (p.y) gstv(p.y + (long long)img[k] * p.ybs + off[k], o);
                    if (p.y2) gstv(p.y2 + (long long)img[k] * p.y2bs + off[k], o);
                }
            }
        } else if (MODE == 1) {
            // dense tensors: offset == element index
            float4 v[UN];
            float4 r[UN];
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = base + k * kThreads;
                if (u < hi) {
                    v[k] = gldv<float4>(p.x + (size_t)u * 4);
                    if (RES) r[k] = gldv<float4>(p.res + (size_t)u * 4);
                }
            }
            if (rd == 0 && p.fa == nullptr) {
                build_table(p, tab, plane_lo, plane_hi);
                __syncthreads();
            }
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = base + k * kThreads;
                if (u < hi) {
                    uint32_t q, rem;
                    p.div_plane.divmod(u * 4, q, rem);
                    const uint32_t room = (uint32_t)p.HW - rem;      // elements left in plane q
                    const PlaneEntry t0 = entry_of(p, tab, plane_lo, q - plane_lo);
                    const PlaneEntry t1 = (room < 4) ? entry_of(p, tab, plane_lo, q - plane_lo + 1) : t0;
                    float4 o;
                    o.x = apply_one<ACT, AFFINE>(v[k].x, t0);
                    o.y = apply_one<ACT, AFFINE>(v[k].y, room > 1 ? t0 : t1);
                    o.z = apply_one<ACT, AFFINE>(v[k].z, room > 2 ? t0 : t1);
                    o.w = apply_one<ACT, AFFINE>(v[k].w, room > 3 ? t0 : t1);
                    if (RES) {
                        o.x = residual_one(o.x, r[k].x, p);
                        o.y = residual_one(o.y, r[k].y, p);
                        o.z = residual_one(o.z, r[k].z, p);
                        o.w = residual_one(o.w, r[k].w, p);
                    }
                    if (p.y) gstv(p.y + (size_t)u * 4, o);
                    if (p.y2) gstv(p.y2 + (size_t)u * 4, o);
                }
            }
        } else {
            float v[UN], r[UN];
            uint32_t off[UN];
            uint32_t pl[UN], img[UN];
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = base + k * kThreads;
                if (u < hi) {
                    uint32_t q, rem, c;
                    p.div_plane.divmod(u, q, rem);
                    p.div_c.divmod(q, img[k], c);
                    pl[k] = q - plane_lo;
                    off[k] = c * (uint32_t)p.HW + rem;
                    v[k] = gld(p.x + ((long long)img[k] * p.xbs + off[k]));
                    if (RES) r[k] = gld(p.res + ((long long)img[k] * p.rbs + off[k]));
                }
            }
            if (rd == 0 && p.fa == nullptr) {
                build_table(p, tab, plane_lo, plane_hi);
                __syncthreads();
            }
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const uint32_t u = base + k * kThreads;
                if (u < hi) {
                    float o = apply_one<ACT, AFFINE>(v[k], entry_of(p, tab, plane_lo, pl[k]));
                    if (RES) o = residual_one(o, r[k], p);
                    if (p.y) gst(p.y + ((long long)img[k] * p.ybs + off[k]), o);
                    if (p.y2) gst(p.y2 + ((long long)img[k] * p.y2bs + off[k]), o);
                }
            }
        }
    }
}

// Tail of MODE 1: the last (n % 4) elements of a dense tensor, one thread each.
template <int ACT, bool AFFINE, bool RES>
__global__ void epilogue_tail_kernel(const EpiParams p, uint32_t first, uint32_t count)
{
    if (threadIdx.x >= count) return;
    const uint32_t e = first + threadIdx.x;
    const PlaneEntry t = make_entry(p, p.div_plane.div(e));
    float o = apply_one<ACT, AFFINE>(gld(p.x + e), t);
    if (RES) o = residual_one(o, gld(p.res + e), p);
    if (p.y) gst(p.y + e, o);
    if (p.y2) gst(p.y2 + e, o);
}

// ---------------------------------------------------------------------------------------------
// Epilogue + 2x2 stride-2 max pool.  One thread produces VO pooled outputs from a 2 x (2*VO)
// input patch (VO = 4, 2, 1 by row alignment); VO = 0 is the scalar form for odd widths, one
// pooled output per thread with bounds-checked taps.  Window origin is (2*oh, 2*ow); taps past
// the edge are skipped; the first maximum in (ky, kx) scan order wins, as in
// src/MaxPoolKernels.cu:26-40.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float pick(float m, float v) { return v > m ? v : m; }

template <int ACT, bool AFFINE, int VO>
__global__ void __launch_bounds__(kThreads, VO == 4 ? 6 : 4)
epilogue_pool_kernel(const EpiParams p)
{
    extern __shared__ PlaneEntry tab[];
    const uint32_t lo = blockIdx.x * p.chunk;
    if (lo >= p.units) return;
    uint32_t hi = lo + p.chunk;
    if (hi > p.units) hi = p.units;
    const uint32_t plane_lo = p.div_ohowv.div(lo);
    const uint32_t plane_hi = p.div_ohowv.div(hi - 1);

    constexpr int NV = VO == 0 ? 1 : VO;       // pooled outputs per patch
    constexpr int NI = 2 * NV;                 // input columns per patch row
    constexpr int U = 16 / (2 * NI);           // patches per thread per round: 16 input floats in flight
    const uint32_t step = kThreads * U;
    const uint32_t rounds = (hi - lo + step - 1) / step;
    for (uint32_t rd = 0; rd < rounds; ++rd) {
        const uint32_t base = lo + rd * step + threadIdx.x;
        float r0[U][NI], r1[U][NI];
        uint32_t pl[U], img[U], in0[U], oh_[U], owv_[U];
        bool row1[U], col1[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const uint32_t u = base + k * kThreads;
            if (u < hi) {
                uint32_t q, rem, oh, owv, c;
                p.div_ohowv.divmod(u, q, rem);
                p.div_owv.divmod(rem, oh, owv);
                p.div_c.divmod(q, img[k], c);
                pl[k] = q - plane_lo; oh_[k] = oh; owv_[k] = owv;
                const int ih = 2 * (int)oh, iw = NI * (int)owv;
                row1[k] = ih + 1 < p.H;
                col1[k] = (VO != 0) || (iw + 1 < p.W);
                in0[k] = c * (uint32_t)p.HW + (uint32_t)ih * (uint32_t)p.W + (uint32_t)iw;
                const float* x0 = p.x + (long long)img[k] * p.xbs + in0[k];
                if (VO == 4) {
                    const float4 a0 = gldv<float4>(x0);
                    const float4 a1 = gldv<float4>(x0 + 4);
                    r0[k][0] = a0.x; r0[k][1] = a0.y; r0[k][2] = a0.z; r0[k][3] = a0.w;
                    r0[k][4] = a1.x; r0[k][5] = a1.y; r0[k][6] = a1.z; r0[k][7] = a1.w;
                    if (row1[k]) {
                        const float4 b0 = gldv<float4>(x0 + p.W);
                        const float4 b1 = gldv<float4>(x0 + p.W + 4);
                        r1[k][0] = b0.x; r1[k][1] = b0.y; r1[k][2] = b0.z; r1[k][3] = b0.w;
                        r1[k][4] = b1.x; r1[k][5] = b1.y; r1[k][6] = b1.z; r1[k][7] = b1.w;
                    }
                } else if (VO == 2) {
                    const float4 a0 = gldv<float4>(x0);
                    r0[k][0] = a0.x; r0[k][1] = a0.y; r0[k][2] = a0.z; r0[k][3] = a0.w;
                    if (row1[k]) {
                        const float4 b0 = gldv<float4>(x0 + p.W);
                        r1[k][0] = b0.x; r1[k][1] = b0.y; r1[k][2] = b0.z; r1[k][3] = b0.w;
                    }
                } else if (VO == 1) {
                    const float2 a0 = gldv<float2>(x0);
                    r0[k][0] = a0.x; r0[k][1] = a0.y;
                    if (row1[k]) {
                        const float2 b0 = gldv<float2>(x0 + p.W);
                        r1[k][0] = b0.x; r1[k][1] = b0.y;
                    }
                } else {
                    r0[k][0] = gld(x0);
                    r0[k][1] = col1[k] ? gld(x0 + 1) : 0.0f;
                    if (row1[k]) {
                        r1[k][0] = gld(x0 + p.W);
                        r1[k][1] = col1[k] ? gld(x0 + (p.W + 1)) : 0.0f;
                    }
                }
            }
        }
        if (rd == 0 && p.fa == nullptr) {
            build_table(p, tab, plane_lo, plane_hi);
            __syncthreads();
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const uint32_t u = base + k * kThreads;
            if (u >= hi) continue;
            const PlaneEntry t = entry_of(p, tab, plane_lo, pl[k]);
            const uint32_t c = (uint32_t)(t.chan & 0xFFFFFF);
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                r0[k][j] = apply_one<ACT, AFFINE>(r0[k][j], t);
                r1[k][j] = row1[k] ? apply_one<ACT, AFFINE>(r1[k][j], t) : 0.0f;
            }
            float m[NV];
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float best = r0[k][2 * j];
                if (col1[k]) best = pick(best, r0[k][2 * j + 1]);
                if (row1[k]) {
                    best = pick(best, r1[k][2 * j]);
                    if (col1[k]) best = pick(best, r1[k][2 * j + 1]);
                }
                m[j] = best;
            }
            float* yp = p.ypool + (long long)img[k] * p.pbs + (long long)c * p.OH * p.OW
                        + (long long)oh_[k] * p.OW + (long long)NV * owv_[k];
            if (VO == 4) gstv(yp, make_float4(m[0], m[1], m[2], m[3]));
            else if (VO == 2) gstv(yp, make_float2(m[0], m[1]));
            else gst(yp, m[0]);

            if (p.y) {
                float* y0 = p.y + (long long)img[k] * p.ybs + in0[k];
                if (VO == 4) {
                    gstv(y0, make_float4(r0[k][0], r0[k][1], r0[k][2], r0[k][3]));
                    gstv(y0 + 4, make_float4(r0[k][4], r0[k][5], r0[k][6], r0[k][7]));
                    if (row1[k]) {
                        gstv(y0 + p.W, make_float4(r1[k][0], r1[k][1], r1[k][2], r1[k][3]));
                        gstv(y0 + p.W + 4, make_float4(r1[k][4], r1[k][5], r1[k][6], r1[k][7]));
                    }
                } else if (VO == 2) {
                    gstv(y0, make_float4(r0[k][0], r0[k][1], r0[k][2], r0[k][3]));
                    if (row1[k]) gstv(y0 + p.W, make_float4(r1[k][0], r1[k][1], r1[k][2], r1[k][3]));
                } else if (VO == 1) {
                    gstv(y0, make_float2(r0[k][0], r0[k][1]));
                    if (row1[k]) gstv(y0 + p.W, make_float2(r1[k][0], r1[k][1]));
                } else {
                    gst(y0, r0[k][0]);
                    if (col1[k]) gst(y0 + 1, r0[k][1]);
                    if (row1[k]) {
                        gst(y0 + p.W, r1[k][0]);
                        if (col1[k]) gst(y0 + (p.W + 1), r1[k][1]);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The common case of the kernel above with the index arithmetic stripped: H even, W a multiple
// of the patch width, x densely packed.  Row pairs then tile the whole tensor without gaps, so
// the input offset of patch u is (u / OWV) * 2W + (u % OWV) * NI -- one division -- and no tap is
// ever out of range.  The image number (needed only for strided destinations) comes from the
// coefficient table.  The pooled kernels are issue-bound rather than HBM-bound once a row is
// short, so instructions per patch are what this form saves.
// ---------------------------------------------------------------------------------------------
template <int ACT, bool AFFINE, int VO>
__global__ void __launch_bounds__(kThreads, VO == 4 ? 6 : 5)
epilogue_pool_even_kernel(const EpiParams p)
{
    extern __shared__ PlaneEntry tab[];
    const uint32_t lo = blockIdx.x * p.chunk;
    if (lo >= p.units) return;
    uint32_t hi = lo + p.chunk;
    if (hi > p.units) hi = p.units;
    const uint32_t plane_lo = p.div_ohowv.div(lo);
    const uint32_t plane_hi = p.div_ohowv.div(hi - 1);

    constexpr int NV = VO;                     // pooled outputs per patch
    constexpr int NI = 2 * NV;                 // input columns per patch row
    constexpr int U = 16 / (2 * NI);           // patches per thread per round: 16 input floats in flight
    const uint32_t W = (uint32_t)p.W;
    const uint32_t step = kThreads * U;
    const uint32_t rounds = (hi - lo + step - 1) / step;
    for (uint32_t rd = 0; rd < rounds; ++rd) {
        const uint32_t base = lo + rd * step + threadIdx.x;
        float r0[U][NI], r1[U][NI];
        uint32_t off[U], pl[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const uint32_t u = base + k * kThreads;
            if (u < hi) {
                uint32_t rp, owv;
                p.div_owv.divmod(u, rp, owv);
                off[k] = rp * (2 * W) + owv * NI;
                pl[k] = p.div_oh.div(rp) - plane_lo;
                const float* x0 = p.x + off[k];
                if (VO == 4) {
                    const float4 a0 = gldv<float4>(x0);
                    const float4 a1 = gldv<float4>(x0 + 4);
                    const float4 b0 = gldv<float4>(x0 + W);
                    const float4 b1 = gldv<float4>(x0 + W + 4);
                    r0[k][0] = a0.x; r0[k][1] = a0.y; r0[k][2] = a0.z; r0[k][3] = a0.w;
                    r0[k][4] = a1.x; r0[k][5] = a1.y; r0[k][6] = a1.z; r0[k][7] = a1.w;
                    r1[k][0] = b0.x; r1[k][1] = b0.y; r1[k][2] = b0.z; r1[k][3] = b0.w;
                    r1[k][4] = b1.x; r1[k][5] = b1.y; r1[k][6] = b1.z; r1[k][7] = b1.w;
                } else if (VO == 2) {
                    const float4 a0 = gldv<float4>(x0);
                    const float4 b0 = gldv<float4>(x0 + W);
                    r0[k][0] = a0.x; r0[k][1] = a0.y; r0[k][2] = a0.z; r0[k][3] = a0.w;
                    r1[k][0] = b0.x; r1[k][1] = b0.y; r1[k][2] = b0.z; r1[k][3] = b0.w;
                } else {
                    const float2 a0 = gldv<float2>(x0);
                    const float2 b0 = gldv<float2>(x0 + W);
                    r0[k][0] = a0.x; r0[k][1] = a0.y;
                    r1[k][0] = b0.x; r1[k][1] = b0.y;
                }
            }
        }
        if (rd == 0 && p.fa == nullptr) {
            build_table(p, tab, plane_lo, plane_hi);
            __syncthreads();
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const uint32_t u = base + k * kThreads;
            if (u >= hi) continue;
            const PlaneEntry t = entry_of(p, tab, plane_lo, pl[k]);
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                r0[k][j] = apply_one<ACT, AFFINE>(r0[k][j], t);
                r1[k][j] = apply_one<ACT, AFFINE>(r1[k][j], t);
            }
            float m[NV];
#pragma unroll
            for (int j = 0; j < NV; ++j)
                m[j] = pick(pick(pick(r0[k][2 * j], r0[k][2 * j + 1]), r1[k][2 * j]), r1[k][2 * j + 1]);
            float* yp = p.ypool + (size_t)u * NV;
            if (!p.pool_dense) {
                const uint32_t img = (uint32_t)t.image;
                yp = p.ypool + (long long)img * p.pbs + (size_t)(u - img * p.units_per_image) * NV;
            }
            if (VO == 4) gstv(yp, make_float4(m[0], m[1], m[2], m[3]));
            else if (VO == 2) gstv(yp, make_float2(m[0], m[1]));
            else gst(yp, m[0]);

            if (p.y) {
                float* y0 = p.y + off[k];
                if (!p.y_dense) {
                    const uint32_t img = (uint32_t)t.image;
                    y0 = p.y + (long long)img * p.ybs + (off[k] - img * (uint32_t)(p.C * p.HW));
                }
                if (VO == 4) {
                    gstv(y0, make_float4(r0[k][0], r0[k][1], r0[k][2], r0[k][3]));
                    gstv(y0 + 4, make_float4(r0[k][4], r0[k][5], r0[k][6], r0[k][7]));
                    gstv(y0 + W, make_float4(r1[k][0], r1[k][1], r1[k][2], r1[k][3]));
                    gstv(y0 + W + 4, make_float4(r1[k][4], r1[k][5], r1[k][6], r1[k][7]));
                } else if (VO == 2) {
                    gstv(y0, make_float4(r0[k][0], r0[k][1], r0[k][2], r0[k][3]));
                    gstv(y0 + W, make_float4(r1[k][0], r1[k][1], r1[k][2], r1[k][3]));
                } else {
                    gstv(y0, make_float2(r0[k][0], r0[k][1]));
                    gstv(y0 + W, make_float2(r1[k][0], r1[k][1]));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Odd widths with small planes (13x13 -> 7x7, 19x19 -> 10x10, where no row pair is aligned and the
// scalar form above spends ~150 instructions of index arithmetic per pooled output).  A warp takes
// whole planes: lane l owns pooled outputs l, l+32, ... of EVERY plane the warp visits, so its
// window offsets, edge predicates and output offset are computed once per thread and the loop over
// planes is loads, the epilogue, three comparisons and a store.  PU planes are in flight per warp.
// Four resident blocks where the activation is cheap enough to fit 64 registers (measured: 11.1 against
// 13.1 us with three at [64,512,13,13] leaky), three for the transcendental ones (which spill at 64).
// ---------------------------------------------------------------------------------------------
template <int ACT, bool AFFINE, int SLOTS>
__global__ void __launch_bounds__(kThreads, (ACT == PXE_ACT_LEAKY || ACT == PXE_ACT_LINEAR || ACT == PXE_ACT_RELU) ? 4 : 3)
epilogue_pool_smallplane_kernel(const EpiParams p, uint32_t planes, uint32_t planes_per_block)
{
    extern __shared__ PlaneEntry tab[];
    constexpr int PU = SLOTS >= 8 ? 1 : 8 / SLOTS;          // planes in flight per warp: 32 loads per lane
    const uint32_t plane_lo = blockIdx.x * planes_per_block;
    if (plane_lo >= planes) return;
    uint32_t plane_end = plane_lo + planes_per_block;
    if (plane_end > planes) plane_end = planes;
    build_table(p, tab, plane_lo, plane_end - 1);

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr uint32_t kWarps = kThreads / 32;
    const uint32_t ohow = (uint32_t)(p.OH * p.OW);
    uint32_t in_off[SLOTS];
    bool valid[SLOTS], row1[SLOTS], col1[SLOTS];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const uint32_t idx = lane + 32u * s;
        valid[s] = idx < ohow;
        uint32_t oh, ow;
        p.div_owv.divmod(valid[s] ? idx : 0u, oh, ow);       // OWV == OW in this form
        in_off[s] = 2u * oh * (uint32_t)p.W + 2u * ow;
        row1[s] = 2 * (int)oh + 1 < p.H;
        col1[s] = 2 * (int)ow + 1 < p.W;
    }
    __syncthreads();

    for (uint32_t q0 = plane_lo + warp * PU; q0 < plane_end; q0 += kWarps * PU) {
        float t00[PU][SLOTS], t01[PU][SLOTS], t10[PU][SLOTS], t11[PU][SLOTS];
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            const uint32_t q = q0 + u;
            if (q < plane_end) {
                const PlaneEntry t = tab[q - plane_lo];
                const float* xb = p.x + (long long)t.image * p.xbs + (long long)(t.chan & 0xFFFFFF) * p.HW;
#pragma unroll
                for (int s = 0; s < SLOTS; ++s) {
                    if (valid[s]) {
                        const float* x0 = xb + in_off[s];
                        t00[u][s] = gld(x0);
                        t01[u][s] = col1[s] ? gld(x0 + 1) : 0.0f;
                        t10[u][s] = row1[s] ? gld(x0 + p.W) : 0.0f;
                        t11[u][s] = (row1[s] && col1[s]) ? gld(x0 + (p.W + 1)) : 0.0f;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            const uint32_t q = q0 + u;
            if (q >= plane_end) continue;
            const PlaneEntry t = tab[q - plane_lo];
            const uint32_t c = (uint32_t)(t.chan & 0xFFFFFF);
            float* yp = p.ypool + (long long)t.image * p.pbs + (long long)c * ohow;
            float* yb = p.y ? p.y + (long long)t.image * p.ybs + (long long)c * p.HW : nullptr;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                if (!valid[s]) continue;
                const float a00 = apply_one<ACT, AFFINE>(t00[u][s], t);
                float best = a00, a01 = 0.0f, a10 = 0.0f, a11 = 0.0f;
                if (col1[s]) { a01 = apply_one<ACT, AFFINE>(t01[u][s], t); best = pick(best, a01); }
                if (row1[s]) {
                    a10 = apply_one<ACT, AFFINE>(t10[u][s], t); best = pick(best, a10);
                    if (col1[s]) { a11 = apply_one<ACT, AFFINE>(t11[u][s], t); best = pick(best, a11); }
                }
                gst(yp + (lane + 32u * s), best);
                if (yb) {
                    float* y0 = yb + in_off[s];
                    gst(y0, a00);
                    if (col1[s]) gst(y0 + 1, a01);
                    if (row1[s]) {
                        gst(y0 + p.W, a10);
                        if (col1[s]) gst(y0 + (p.W + 1), a11);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Odd small planes of a tensor whose images are dense and 16-byte aligned, channels a multiple of four: four
// consecutive planes are 4*HW floats = HW whole 128-bit vectors starting on a 16-byte boundary.  A warp loads such
// a group as flat coalesced vectors (one sector per 32 bytes, where the scalar stride-2 taps of the form above
// touch eight sectors per request), applies the epilogue once per element on the vector, leaves the result in
// the warp's own staging area and takes the 2x2 taps of its pooled outputs from there.
//
// The kernel is bound by instruction issue and latency, not by memory, so everything that does not depend on the
// data is tabulated once per block: for each pooled output of a group the four staging offsets of its taps (a tap
// outside the plane repeats the window's first tap, which never changes "first maximum wins"), for each vector the
// table offsets of the planes its components lie in (a vector may straddle two planes; which of a lane's vectors
// can is the same for the whole warp).  The loop over groups is then loads, the epilogue, four shared-memory reads
// and three comparisons per pooled output, and stores.  Each warp folds the coefficients of its own planes after
// the block's one barrier, so no warp waits there for another one's loads; the loads of a warp's next group go
// out as soon as the registers of the current one are free (its values sit in the staging by then).
//
// Measured on B200 at [64,512,13,13] -> 7x7 (leaky / mish, us): the warp-per-plane form above 11.1 / 13.7; this
// kernel with geometry in registers instead of tables 12.8 / 15.2; tables, 8 warps x 2 groups 10.0 / 11.6; the
// same with all groups requested up front by asynchronous copies into a two-group staging 11.0 / 11.7; 4 warps x 2
// groups (1024 blocks, seven resident per SM: 56 groups on every SM) 9.5 / 10.9; 1, 3, 4 groups per warp and 2- or
// 8-warp blocks are all behind.  A launch that only reads the tensor takes 5.1, an empty one 1.2.
// ---------------------------------------------------------------------------------------------
constexpr int kFlatWarps = 4;             // warps per block
constexpr int kFlatGroups = 2;            // groups per warp
constexpr int kFlatVectors = 6;           // vectors per lane and group: planes of up to 192 elements
constexpr int kFlatSlots = 7;             // pooled outputs per lane and group: up to 56 per plane

// G: planes per group (4 for planes of odd size: 4 * HW floats are whole vectors)
template <int ACT, bool AFFINE, int G, int NV, int SLOTS, int WARPS, int GPW>
__global__ void __launch_bounds__(WARPS * 32, 7)
epilogue_pool_flat_kernel(const EpiParams p, uint32_t groups)
{
    extern __shared__ float4 flat_smem[];
    constexpr uint32_t kBlock = WARPS * 32;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t HW = (uint32_t)p.HW, W = (uint32_t)p.W;
    const uint32_t ohow = (uint32_t)(p.OH * p.OW);
    // shared memory: staging, HW vectors per warp | the warps' plane entries | tap offsets | component planes
    const uint32_t V = (uint32_t)G * HW / 4;               // vectors per group
    float4* stage4 = flat_smem + (size_t)warp * V;
    PlaneEntry* tab = reinterpret_cast<PlaneEntry*>(flat_smem + (size_t)WARPS * V) + warp * GPW * G;
    uint2* tap_tab = reinterpret_cast<uint2*>(flat_smem + (size_t)WARPS * V + WARPS * GPW * G);
    uint32_t* comp_tab = reinterpret_cast<uint32_t*>(tap_tab + 32 * SLOTS);

    const uint32_t w0 = (blockIdx.x * WARPS + warp) * GPW;                   // the warp's first group
    float4 d[NV];
    auto load_group = [&](uint32_t g) {
        if (g >= groups) return;
        const uint32_t q0 = g * G;
        const uint32_t img = p.div_c.div(q0);
        const float4* x4 = reinterpret_cast<const float4*>(p.x + (long long)img * p.xbs + (long long)(q0 - img * (uint32_t)p.C) * HW);
#pragma unroll
        for (int r = 0; r < NV; ++r)
            if (lane + 32u * r < V) d[r] = gld(x4 + (lane + 32u * r));
    };
    load_group(w0);                                        // before anything else
    for (uint32_t o = threadIdx.x; o < 32u * SLOTS; o += kBlock) {
        // pooled output o of a group: byte offsets of its four taps in the group's staging, two per word
        const uint32_t oo = o < G * ohow ? o : 0u;
        const uint32_t pl = (oo >= ohow) + (oo >= 2 * ohow) + (oo >= 3 * ohow);
        uint32_t oh, ow;
        p.div_owv.divmod(oo - pl * ohow, oh, ow);                       // OWV == OW in this form
        const uint32_t t00 = 4u * (pl * HW + 2u * oh * W + 2u * ow);
        const uint32_t dx = 2 * ow + 1 < W ? 4u : 0u, dy = 2 * oh + 1 < (uint32_t)p.H ? 4u * W : 0u;
        tap_tab[o] = make_uint2(t00 | ((t00 + dx) << 16), (t00 + dy) | ((t00 + dy + dx) << 16));
    }
    for (uint32_t i = threadIdx.x; i < 32u * NV; i += kBlock) {
        // vector i of a group: 16 * (plane of component j) in byte j; HW > 3, so a vector meets one boundary at most
        const uint32_t e = 4u * i;
        const uint32_t lo = e < G * HW ? (e >= HW) + (e >= 2 * HW) + (e >= 3 * HW) : 0u;
        const uint32_t hi = e + 3 < G * HW ? (e + 3 >= HW) + (e + 3 >= 2 * HW) + (e + 3 >= 3 * HW) : lo;
        const uint32_t edge = hi * HW;
        const uint32_t p1 = e + 1 >= edge ? hi : lo, p2 = e + 2 >= edge ? hi : lo;
        comp_tab[i] = (lo | (p1 << 8) | (p2 << 16) | (hi << 24)) * (uint32_t)sizeof(PlaneEntry);
    }
    __syncthreads();
    if (lane < GPW * G && w0 * G + lane < groups * G)
        tab[lane] = make_entry(p, w0 * G + lane);
    __syncwarp();

    uint32_t straddles = 0;          // bit r: some lane's vector r crosses a plane boundary (the same for every lane)
#pragma unroll
    for (int r = 0; r < NV; ++r) {
        const uint32_t w = comp_tab[lane + 32 * r];
        if (__any_sync(0xffffffffu, (w >> 24) != (w & 0xFFu))) straddles |= 1u << r;
    }
    const uint32_t n_out = G * ohow;
    const char* stage_bytes = reinterpret_cast<const char*>(stage4);

#pragma unroll 1
    for (int k = 0; k < GPW; ++k) {
        const uint32_t g = w0 + k;
        if (g >= groups) break;
        const uint32_t q0 = g * G;
        const uint32_t img = p.div_c.div(q0);
        const uint32_t c0 = q0 - img * (uint32_t)p.C;
        const char* tab_bytes = reinterpret_cast<const char*>(tab + k * G);
        auto entry = [&](uint32_t off) { return *reinterpret_cast<const PlaneEntry*>(tab_bytes + off); };
        float4* y4 = p.y ? reinterpret_cast<float4*>(p.y + (long long)img * p.ybs + (long long)c0 * HW) : nullptr;
#pragma unroll
        for (int r = 0; r < NV; ++r) {
            const uint32_t v = lane + 32u * r;
            if (v >= V) continue;
            const uint32_t w = comp_tab[v];
            const PlaneEntry t0 = entry(w & 0xFFu);
            float4 o;
            o.x = apply_one<ACT, AFFINE>(d[r].x, t0);
            if (!(straddles & (1u << r))) {
                o.y = apply_one<ACT, AFFINE>(d[r].y, t0);
                o.z = apply_one<ACT, AFFINE>(d[r].z, t0);
                o.w = apply_one<ACT, AFFINE>(d[r].w, t0);
            } else {
                o.y = apply_one<ACT, AFFINE>(d[r].y, entry((w >> 8) & 0xFFu));
                o.z = apply_one<ACT, AFFINE>(d[r].z, entry((w >> 16) & 0xFFu));
                o.w = apply_one<ACT, AFFINE>(d[r].w, entry(w >> 24));
            }
            stage4[v] = o;
            if (y4) gst(y4 + v, o);
        }
        if (k + 1 < GPW) load_group(g + 1);
        __syncwarp();
        float* yp = p.ypool + (long long)img * p.pbs + (long long)c0 * ohow + lane;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const uint2 t = tap_tab[lane + 32 * s];
            float best = *reinterpret_cast<const float*>(stage_bytes + (t.x & 0xFFFFu));
            best = pick(best, *reinterpret_cast<const float*>(stage_bytes + (t.x >> 16)));
            best = pick(best, *reinterpret_cast<const float*>(stage_bytes + (t.y & 0xFFFFu)));
            best = pick(best, *reinterpret_cast<const float*>(stage_bytes + (t.y >> 16)));
            if (lane + 32u * s < n_out) gst(yp + 32 * s, best);
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------- launch helpers
// Rounds of the per-thread loop one block runs (a round = one batch of loads per thread).  Measured
// on B200: short blocks (2 rounds, 32 KB of input each for the streaming kernel) in many waves give
// the best HBM throughput at every tensor size.
// Splits `units` into per-block chunks of `rounds` granules, at most `max_chunk`.
void plan_chunks(uint32_t units, uint32_t granule, uint32_t max_chunk, int rounds, uint32_t* chunk, unsigned* grid)
{
    long long c = (long long)granule * rounds;
    if (max_chunk >= granule && c > (long long)(max_chunk / granule) * granule) c = (long long)(max_chunk / granule) * granule;
    if (c < granule) c = granule;
    *chunk = (uint32_t)c;
    *grid = (unsigned)((units + c - 1) / c);
}

template <int ACT, bool AFFINE, bool RES, int MODE>
int launch_stream_kernel(cudaStream_t s, EpiParams& p, const DeviceInfo& di)
{
    const int vw = MODE == 2 ? 1 : 4;
    // planes touched by a chunk of `chunk` units: chunk*vw/HW + 2  <= kMaxPlanesPerBlock
    long long max_chunk_ll = (long long)(kMaxPlanesPerBlock - 2) * p.HW / vw;
    uint32_t max_chunk = max_chunk_ll > 0x7fffffffLL ? 0x7fffffffu : (uint32_t)max_chunk_ll;
    uint32_t granule = kThreads * kUnroll;
    if (max_chunk < granule) { granule = kThreads; }
    if (max_chunk < granule) { max_chunk = granule; }   // tiny HW: checked below
    unsigned grid;
    // with folded coefficients a block has no table to amortise: one round per block measured ahead of two for the plain
    // form at every size below 700 MB (0.95 against 0.91 of peak at 177 MB), level with it for the residual form
    const int rounds = (p.fa && !RES) ? 1 : 2;
    plan_chunks(p.units, granule, max_chunk, rounds, &p.chunk, &grid);
    long long planes = (long long)p.chunk * vw / p.HW + 2;
    size_t smem = (size_t)planes * sizeof(PlaneEntry);
    if (smem > 48 * 1024) {
        if (smem > (size_t)di.max_smem_optin)
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue: plane table of %zu bytes does not fit shared memory", smem);
        PXE_CUDA_OK(cudaFuncSetAttribute(epilogue_kernel<ACT, AFFINE, RES, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    epilogue_kernel<ACT, AFFINE, RES, MODE><<<grid, kThreads, smem, s>>>(p);
    PXE_LAUNCH_OK("epilogue_kernel");
    return PXE_OK;
}

template <int ACT, bool AFFINE, bool RES>
int dispatch_mode(cudaStream_t s, EpiParams& p, const DeviceInfo& di, int mode, long long n_elems)
{
    if (mode == 0) {
        p.units = (uint32_t)(n_elems / 4);
        p.div_plane = FastDiv((uint32_t)(p.HW / 4));
        return launch_stream_kernel<ACT, AFFINE, RES, 0>(s, p, di);
    }
    if (mode == 1) {
        p.units = (uint32_t)(n_elems / 4);
        p.div_plane = FastDiv((uint32_t)p.HW);
        int rc = PXE_OK;
        if (p.units) rc = launch_stream_kernel<ACT, AFFINE, RES, 1>(s, p, di);
        if (rc != PXE_OK) return rc;
        uint32_t tail = (uint32_t)(n_elems % 4);
        if (tail) {
            epilogue_tail_kernel<ACT, AFFINE, RES><<<1, 32, 0, s>>>(p, (uint32_t)(n_elems - tail), tail);
            PXE_LAUNCH_OK("epilogue_tail_kernel");
        }
        return PXE_OK;
    }
    p.units = (uint32_t)n_elems;
    p.div_plane = FastDiv((uint32_t)p.HW);
    return launch_stream_kernel<ACT, AFFINE, RES, 2>(s, p, di);
}

template <int ACT>
int dispatch_flags(cudaStream_t s, EpiParams& p, const DeviceInfo& di, int mode, long long n, bool affine)
{
    const bool res = p.res != nullptr;
    if (affine) {
        return res ? dispatch_mode<ACT, true, true>(s, p, di, mode, n)
                   : dispatch_mode<ACT, true, false>(s, p, di, mode, n);
    }
    return res ? dispatch_mode<ACT, false, true>(s, p, di, mode, n)
               : dispatch_mode<ACT, false, false>(s, p, di, mode, n);
}

template <int ACT, bool AFFINE>
int launch_pool(cudaStream_t s, EpiParams& p, const DeviceInfo& di, int vo)
{
    const bool general_only = p.pool_general != 0;       // the caller asked for the general kernel (pxe_epilogue_desc.pool_variant)
    const int nv = vo == 0 ? 1 : vo;
    p.OWV = p.OW / nv;
    p.div_owv = FastDiv((uint32_t)p.OWV);
    p.div_ohowv = FastDiv((uint32_t)(p.OH * p.OWV));
    const uint32_t per_plane = (uint32_t)(p.OH * p.OWV);
    long long max_chunk_ll = (long long)(kMaxPlanesPerBlock - 2) * per_plane;
    uint32_t max_chunk = max_chunk_ll > 0x7fffffffLL ? 0x7fffffffu : (uint32_t)max_chunk_ll;
    uint32_t granule = kThreads * (vo == 4 ? 1 : (vo == 2 ? 2 : 4));     // patches per thread per round, see the kernel
    if (max_chunk < granule) granule = kThreads;
    if (max_chunk < granule) max_chunk = granule;
    unsigned grid;
    constexpr int rounds = 2;
    plan_chunks(p.units, granule, max_chunk, rounds, &p.chunk, &grid);
    long long planes = (long long)p.chunk / per_plane + 2;
    size_t smem = (size_t)planes * sizeof(PlaneEntry);
    // odd widths, small planes: a warp per plane with per-thread window geometry hoisted out of the loop
    const uint32_t ohow = (uint32_t)(p.OH * p.OW);
    const int slots = ohow <= 64 ? 2 : 4;
    // measured on B200: ahead of the general form with two or four output slots per lane and at least 70 % of the
    // lane slots in use (13x13 -> 7x7, 19x19 -> 10x10); behind it with one slot (tiny planes) or eight (27x27, 31x31)
    // ahead of the warp-per-plane form wherever it applies (9.5 against 11.1 us at [64,512,13,13] leaky, 10.9 against 13.7 mish).
    // Planes that are themselves whole vectors (26x26 = 169 of them) could run it with one plane per group; measured, that
    // is behind the row-pair form there (15.6 against 13.5 us at [64,256,26,26] leaky), so only odd planes come here.
    constexpr int flat_g = 4;
    if (vo == 0 && p.HW % 2 != 0 && p.flat_ok && p.C % flat_g == 0 && !general_only && p.HW > 32
        && p.HW <= 32 * kFlatVectors && (uint32_t)flat_g * ohow <= 32 * kFlatSlots) {
        const uint32_t groups = p.units / per_plane / (uint32_t)flat_g;
        constexpr int per_block = kFlatWarps * kFlatGroups;
        const unsigned blocks = (groups + per_block - 1) / per_block;
        const size_t bytes = (size_t)kFlatWarps * ((size_t)flat_g * p.HW * sizeof(float) + kFlatGroups * flat_g * sizeof(PlaneEntry))
                             + 32 * kFlatSlots * sizeof(uint2) + 32 * kFlatVectors * sizeof(uint32_t);
        epilogue_pool_flat_kernel<ACT, AFFINE, flat_g, kFlatVectors, kFlatSlots, kFlatWarps, kFlatGroups>
            <<<blocks, kFlatWarps * 32, bytes, s>>>(p, groups);
        PXE_LAUNCH_OK("epilogue_pool_flat_kernel");
        return PXE_OK;
    }
    if (vo == 0 && ohow > 32 && ohow <= 128 && 10 * ohow >= 7 * 32 * (uint32_t)slots && !general_only) {
        const uint32_t n_planes = p.units / per_plane;
        const uint32_t pu = 8 / slots;
        const uint32_t planes_per_block = (kThreads / 32) * pu * 2;          // two rounds per warp: short blocks
        const unsigned blocks = (n_planes + planes_per_block - 1) / planes_per_block;
        const size_t tab_bytes = (size_t)planes_per_block * sizeof(PlaneEntry);
        if (slots == 2)
            epilogue_pool_smallplane_kernel<ACT, AFFINE, 2><<<blocks, kThreads, tab_bytes, s>>>(p, n_planes, planes_per_block);
        else
            epilogue_pool_smallplane_kernel<ACT, AFFINE, 4><<<blocks, kThreads, tab_bytes, s>>>(p, n_planes, planes_per_block);
        PXE_LAUNCH_OK("epilogue_pool_smallplane_kernel");
        return PXE_OK;
    }
    // stripped index arithmetic when row pairs tile the tensor: even H, dense x (W already is a multiple of the patch)
    const bool even = !general_only && vo != 0 && p.H % 2 == 0 && p.xbs == (long long)p.C * p.HW;
    void (*kern)(const EpiParams) = nullptr;
    if (even) {
        p.div_oh = FastDiv((uint32_t)p.OH);
        p.units_per_image = per_plane * (uint32_t)p.C;
        p.y_dense = p.ybs == (long long)p.C * p.HW;
        p.pool_dense = p.pbs == (long long)p.C * p.OH * p.OW;
        switch (vo) {
        case 4: kern = epilogue_pool_even_kernel<ACT, AFFINE, 4>; break;
        case 2: kern = epilogue_pool_even_kernel<ACT, AFFINE, 2>; break;
        default: kern = epilogue_pool_even_kernel<ACT, AFFINE, 1>; break;
        }
    } else {
        switch (vo) {
        case 4: kern = epilogue_pool_kernel<ACT, AFFINE, 4>; break;
        case 2: kern = epilogue_pool_kernel<ACT, AFFINE, 2>; break;
        case 1: kern = epilogue_pool_kernel<ACT, AFFINE, 1>; break;
        default: kern = epilogue_pool_kernel<ACT, AFFINE, 0>; break;
        }
    }
    if (smem > 48 * 1024) {
        if (smem > (size_t)di.max_smem_optin)
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue(pool): plane table of %zu bytes does not fit shared memory", smem);
        PXE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    kern<<<grid, kThreads, smem, s>>>(p);
    PXE_LAUNCH_OK("epilogue_pool_kernel");
    return PXE_OK;
}

template <int ACT>
int dispatch_act(cudaStream_t s, EpiParams& p, const DeviceInfo& di, int mode, long long n, bool affine,
                 bool pool, int vo)
{
    if (pool) return affine ? launch_pool<ACT, true>(s, p, di, vo) : launch_pool<ACT, false>(s, p, di, vo);
    return dispatch_flags<ACT>(s, p, di, mode, n, affine);
}

int dispatch(cudaStream_t s, EpiParams& p, const DeviceInfo& di, int act, int mode, long long n, bool affine,
             bool pool, int vo)
{
    switch (act) {
    case PXE_ACT_LEAKY: return dispatch_act<PXE_ACT_LEAKY>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_LINEAR: return dispatch_act<PXE_ACT_LINEAR>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_LOGGY: return dispatch_act<PXE_ACT_LOGGY>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_LOGISTIC: return dispatch_act<PXE_ACT_LOGISTIC>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_MISH: return dispatch_act<PXE_ACT_MISH>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_RELU: return dispatch_act<PXE_ACT_RELU>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_SOFTPLUS: return dispatch_act<PXE_ACT_SOFTPLUS>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_SWISH: return dispatch_act<PXE_ACT_SWISH>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_TANH: return dispatch_act<PXE_ACT_TANH>(s, p, di, mode, n, affine, pool, vo);
    case PXE_ACT_YOLO_HEAD: return dispatch_act<PXE_ACT_YOLO_HEAD>(s, p, di, mode, n, affine, pool, vo);
    default: return set_error(PXE_ERR_BAD_ARG, "conv_epilogue: unknown activation %d", act);
    }
}

long long dense_or(long long stride, long long dense) { return stride == 0 ? dense : stride; }

// One slice of the batch whose element count fits 32-bit unit indices.
int run_slice(cudaStream_t s, const pxe_epilogue_desc& d, int b0, int nb, const DeviceInfo& di)
{
    const long long HW = (long long)d.height * d.width;
    const long long CHW = HW * d.channels;
    EpiParams p{};
    p.xbs = dense_or(d.x_batch_stride, CHW);
    p.ybs = dense_or(d.y_batch_stride, CHW);
    p.y2bs = dense_or(d.y2_batch_stride, CHW);
    p.rbs = dense_or(d.residual_batch_stride, CHW);
    p.x = d.x + (long long)b0 * p.xbs;
    p.y = d.y ? d.y + (long long)b0 * p.ybs : nullptr;
    p.y2 = d.y2 ? d.y2 + (long long)b0 * p.y2bs : nullptr;
    p.res = d.residual ? d.residual + (long long)b0 * p.rbs : nullptr;
    p.gamma = d.gamma; p.beta = d.beta; p.mean = d.mean; p.var = d.var; p.bias = d.bias;
    p.fa = d.folded_a; p.fb = d.folded_b;
    p.eps = d.eps; p.eps_mode = d.eps_mode;
    p.C = d.channels; p.H = d.height; p.W = d.width; p.HW = (int)HW;
    p.yolo_entries = d.act == PXE_ACT_YOLO_HEAD ? d.yolo_classes + 5 : 0;
    p.ralpha = d.res_alpha; p.rbeta = d.res_beta; p.res_act = d.res_act;
    p.div_c = FastDiv((uint32_t)d.channels);
    const long long n = (long long)nb * CHW;
    const bool affine = d.gamma != nullptr || d.bias != nullptr || d.folded_a != nullptr;

    if (d.pool_kernel) {
        PXE_REQUIRE(d.pool_variant == PXE_POOL_AUTO || d.pool_variant == PXE_POOL_GENERAL, "conv_epilogue: unknown pool_variant %d", d.pool_variant);
        p.pool_general = d.pool_variant == PXE_POOL_GENERAL;
        p.OH = pxe_maxpool_out_dim(d.height, 2, 2, d.pool_padding);
        p.OW = pxe_maxpool_out_dim(d.width, 2, 2, d.pool_padding);
        p.pbs = dense_or(d.y_pool_batch_stride, (long long)d.channels * p.OH * p.OW);
        p.ypool = d.y_pool + (long long)b0 * p.pbs;
        int vo = 0;
        const bool a16 = aligned16(p.x) && p.xbs % 4 == 0 && (!p.y || (aligned16(p.y) && p.ybs % 4 == 0));
        const bool a8 = aligned8(p.x) && p.xbs % 2 == 0 && (!p.y || (aligned8(p.y) && p.ybs % 2 == 0));
        if (d.width % 8 == 0 && a16 && aligned16(p.ypool) && p.pbs % 4 == 0) vo = 4;
        else if (d.width % 4 == 0 && a16 && aligned8(p.ypool) && p.pbs % 2 == 0) vo = 2;
        else if (d.width % 2 == 0 && a8) vo = 1;
        p.flat_ok = a16;
        const int nv = vo == 0 ? 1 : vo;
        p.units = (uint32_t)((long long)nb * d.channels * p.OH * (p.OW / nv));
        return dispatch(s, p, di, d.act, 0, n, affine, true, vo);
    }

    int mode = 2;
    auto ok16 = [](const float* ptr, long long bs) { return !ptr || (aligned16(ptr) && bs % 4 == 0); };
    const bool all16 = ok16(p.x, p.xbs) && ok16(p.y, p.ybs) && ok16(p.y2, p.y2bs) && ok16(p.res, p.rbs);
    const bool dense = p.xbs == CHW && (!p.y || p.ybs == CHW) && (!p.y2 || p.y2bs == CHW) && (!p.res || p.rbs == CHW);
    if (HW % 4 == 0 && all16) mode = 0;
    else if (dense && all16 && HW >= 4) mode = 1;
    return dispatch(s, p, di, d.act, mode, n, affine, false, 0);
}

// A tensor argument as the kernels see it: `batch` blocks of `n` floats, `bs` floats apart.
struct Span {
    const float* p;
    long long bs, n;
    int batch;
};

// True when some image block of `a` shares an element with some image block of `b` -- unless they are the same
// tensor (same base, same stride), which the kernels handle: every element is read before it is written by the
// same thread.  Channel slots of one concat buffer interleave without touching and pass.
bool conflict(const Span& a, const Span& b)
{
    if (!a.p || !b.p) return false;
    if (a.p == b.p && (a.bs == b.bs || (a.batch == 1 && b.batch == 1))) return false;
    const long long base_a = (long long)(reinterpret_cast<uintptr_t>(a.p) / sizeof(float));
    const long long base_b = (long long)(reinterpret_cast<uintptr_t>(b.p) / sizeof(float));
    const long long sb = b.bs > 0 ? b.bs : b.n;
    for (int i = 0; i < a.batch; ++i) {
        const long long lo = base_a + i * a.bs, hi = lo + a.n;         // [lo, hi) in float units
        // image j of b is [base_b + j*sb, + b.n): intersects iff base_b + j*sb < hi and base_b + j*sb + b.n > lo
        long long j_lo = lo - base_b - b.n + 1, j_hi = hi - 1 - base_b;
        j_lo = j_lo <= 0 ? 0 : (j_lo + sb - 1) / sb;
        if (j_hi < 0) continue;
        j_hi = j_hi / sb;
        if (j_hi > b.batch - 1) j_hi = b.batch - 1;
        if (j_lo <= j_hi) return true;
    }
    return false;
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" int pxe_conv_epilogue(pxe_stream_t stream, const pxe_epilogue_desc* dp)
{
    PXE_REQUIRE(dp != nullptr, "conv_epilogue: null descriptor");
    const pxe_epilogue_desc& d = *dp;
    PXE_REQUIRE(d.x != nullptr, "conv_epilogue: x is null");
    PXE_REQUIRE(d.batch > 0 && d.channels > 0 && d.height > 0 && d.width > 0,
                "conv_epilogue: non-positive shape [%d,%d,%d,%d]", d.batch, d.channels, d.height, d.width);
    PXE_REQUIRE(d.channels < (1 << 24), "conv_epilogue: too many channels (%d)", d.channels);
    PXE_REQUIRE((long long)d.height * d.width < (1LL << 30), "conv_epilogue: plane too large");
    PXE_REQUIRE(d.act == PXE_ACT_YOLO_HEAD || valid_activation(d.act), "conv_epilogue: unknown activation %d", d.act);
    if (d.act == PXE_ACT_YOLO_HEAD)
        PXE_REQUIRE(d.yolo_classes >= 0 && d.channels % (d.yolo_classes + 5) == 0,
                    "conv_epilogue: channels %d not a multiple of yolo_classes+5 = %d", d.channels, d.yolo_classes + 5);
    if (d.gamma)
        PXE_REQUIRE(d.beta && d.mean && d.var, "conv_epilogue: gamma given but beta/mean/var missing");
    PXE_REQUIRE((d.folded_a == nullptr) == (d.folded_b == nullptr), "conv_epilogue: folded_a and folded_b go together");
    PXE_REQUIRE(d.eps_mode == PXE_BN_EPS_CUDNN || d.eps_mode == PXE_BN_EPS_CPU, "conv_epilogue: bad eps_mode %d", d.eps_mode);
    const long long HW = (long long)d.height * d.width, CHW = HW * d.channels;
    PXE_REQUIRE(d.x_batch_stride == 0 || d.x_batch_stride >= CHW, "conv_epilogue: x_batch_stride too small");
    PXE_REQUIRE(d.y_batch_stride == 0 || d.y_batch_stride >= CHW, "conv_epilogue: y_batch_stride too small");
    PXE_REQUIRE(d.y2_batch_stride == 0 || d.y2_batch_stride >= CHW, "conv_epilogue: y2_batch_stride too small");
    PXE_REQUIRE(d.residual_batch_stride == 0 || d.residual_batch_stride >= CHW, "conv_epilogue: residual_batch_stride too small");
    if (d.residual) PXE_REQUIRE(valid_activation(d.res_act), "conv_epilogue: unknown residual activation %d", d.res_act);
    if (d.pool_kernel) {
        PXE_REQUIRE(d.y_pool != nullptr, "conv_epilogue: pooling requested but y_pool is null");
        if (d.pool_kernel != 2 || d.pool_stride != 2 || d.pool_padding < 0 || d.pool_padding > 1)
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue: fused pooling supports kernel 2 / stride 2 / padding 0|1 only (got %d/%d/%d)",
                             d.pool_kernel, d.pool_stride, d.pool_padding);
        if (d.residual || d.y2)
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue: fused pooling cannot be combined with residual or y2");
        const int oh = pxe_maxpool_out_dim(d.height, 2, 2, d.pool_padding);
        const int ow = pxe_maxpool_out_dim(d.width, 2, 2, d.pool_padding);
        PXE_REQUIRE(oh > 0 && ow > 0, "conv_epilogue: empty pooled output");
        if (d.y && (2 * oh < d.height || 2 * ow < d.width))
            return set_error(PXE_ERR_UNSUPPORTED, "conv_epilogue: padding 0 with an odd extent leaves full-resolution rows uncovered; run pxe_maxpool separately");
        const long long pchw = (long long)d.channels * oh * ow;
        PXE_REQUIRE(d.y_pool_batch_stride == 0 || d.y_pool_batch_stride >= pchw, "conv_epilogue: y_pool_batch_stride too small");
    } else {
        PXE_REQUIRE(d.y != nullptr, "conv_epilogue: y is null");
    }
    {
        // A destination that shares memory with an input (other than being that very tensor), or with another
        // destination, would be read after being written or written twice: refuse it.  Slots of one concat buffer
        // interleave image by image without sharing an element, so the test is per image block.
        const Span x{d.x, d.x_batch_stride ? d.x_batch_stride : CHW, CHW, d.batch};
        const Span y{d.y, d.y_batch_stride ? d.y_batch_stride : CHW, CHW, d.batch};
        const Span y2{d.y2, d.y2_batch_stride ? d.y2_batch_stride : CHW, CHW, d.batch};
        const Span res{d.residual, d.residual_batch_stride ? d.residual_batch_stride : CHW, CHW, d.batch};
        long long pchw = 0;
        if (d.pool_kernel) pchw = (long long)d.channels * pxe_maxpool_out_dim(d.height, 2, 2, d.pool_padding) *
                                  pxe_maxpool_out_dim(d.width, 2, 2, d.pool_padding);
        const Span yp{d.pool_kernel ? d.y_pool : nullptr, d.y_pool_batch_stride ? d.y_pool_batch_stride : pchw, pchw, d.batch};
        PXE_REQUIRE(!conflict(y, x), "conv_epilogue: y partially overlaps x");
        PXE_REQUIRE(!conflict(y2, x), "conv_epilogue: y2 partially overlaps x");
        PXE_REQUIRE(!d.y2 || d.y2 != d.y, "conv_epilogue: y2 is y");
        PXE_REQUIRE(!conflict(y2, y), "conv_epilogue: y2 overlaps y");
        PXE_REQUIRE(!conflict(y, res) && !conflict(y2, res), "conv_epilogue: a destination partially overlaps the residual");
        PXE_REQUIRE(!conflict(yp, x) && !(d.pool_kernel && d.y_pool == d.x), "conv_epilogue: y_pool overlaps x");
        PXE_REQUIRE(!conflict(yp, y) && !conflict(yp, y2) && !conflict(yp, res) &&
                        !(d.pool_kernel && (d.y_pool == d.y || d.y_pool == d.y2 || d.y_pool == d.residual)),
                    "conv_epilogue: y_pool overlaps another tensor of the call");
    }
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // keep unit indices inside 32 bits: at most 2^31 elements per launch
    const long long max_elems = 1LL << 31;
    PXE_REQUIRE(CHW < max_elems, "conv_epilogue: one image has %lld elements, limit is 2^31", CHW);
    int per = (int)(max_elems / CHW);
    if (per < 1) per = 1;
    for (int b0 = 0; b0 < d.batch; b0 += per) {
        int nb = d.batch - b0 < per ? d.batch - b0 : per;
        rc = run_slice(s, d, b0, nb, di);
        if (rc != PXE_OK) return rc;
    }
    return PXE_OK;
}

extern "C" int pxe_activate(pxe_stream_t stream, int act, float* x, size_t n)
{
    PXE_REQUIRE(valid_activation(act), "activate: unknown activation %d", act);
    if (n == 0) return PXE_OK;
    PXE_REQUIRE(x != nullptr, "activate: x is null");
    // a [1, 1, rows, 1<<20]-shaped view of the flat array, sliced so every launch stays in range
    const size_t cols = 1u << 20;
    size_t done = 0;
    while (done < n) {
        size_t left = n - done;
        pxe_epilogue_desc d{};
        d.x = x + done; d.y = x + done;
        d.batch = 1; d.channels = 1; d.act = act;
        size_t take;
        if (left >= cols) {
            size_t rows = left / cols;
            if (rows > 512) rows = 512;
            d.height = (int)rows; d.width = (int)cols;
            take = rows * cols;
        } else {
            d.height = 1; d.width = (int)left;
            take = left;
        }
        int rc = pxe_conv_epilogue(stream, &d);
        if (rc != PXE_OK) return rc;
        done += take;
    }
    return PXE_OK;
}

extern "C" int pxe_add_bias(pxe_stream_t stream, float* out, const float* bias, int batch, int n, int size)
{
    PXE_REQUIRE(out && bias, "add_bias: null pointer");
    PXE_REQUIRE(batch > 0 && n > 0 && size > 0, "add_bias: non-positive shape");
    pxe_epilogue_desc d{};
    d.x = out; d.y = out; d.batch = batch; d.channels = n; d.height = 1; d.width = size;
    d.bias = bias; d.act = PXE_ACT_LINEAR;
    return pxe_conv_epilogue(stream, &d);
}
