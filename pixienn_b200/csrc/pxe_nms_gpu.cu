// Non-maximum suppression on the device with the behaviour of px::nms (src/Box.cpp:56-145), record for
// record the result of pxe_nms_host:
//   1. stable sort by probability, descending                      (src/Box.cpp:63-66);
//   2. per image, in that order: a box is dropped when an earlier box of the same image and a DIFFERENT class
//      that is still alive overlaps it with IoU > 0.9              (src/Box.cpp:68-87);
//   3. per (image, class) group, looking only at the group's first 1024 members in that order: greedy
//      suppression at IoU > threshold against the members kept so far  (src/Box.cpp:89-139);
//   4. the survivors, in the order of step 1.
// Steps 2 and 3 are sequential in the pivot (whether box i suppresses anything depends on whether an earlier
// box suppressed i) and parallel in the boxes behind it: one block per image (step 2) or per group (step 3)
// walks the pivots in order; for a live pivot all threads test the boxes behind it at once.  The three
// orderings come from stable radix sorts (CUB, caller-supplied temporary storage): by (probability, index),
// then by image, then by (image, class) -- a stable sort keeps the probability order inside every segment.
// IoU is evaluated with the same single-rounded operations, in the same order, as the host form
// (cv::Rect2f intersection and area of OpenCV >= 4.5.4); no fused multiply-add.
#include <cub/cub.cuh>

#include "pxe_common.cuh"

namespace pxe {
namespace {

struct Rect { float x, y, w, h; };

__device__ __forceinline__ bool rect_empty(const Rect& r) { return r.w <= 0 || r.h <= 0; }

__device__ __forceinline__ float rect_area(const Rect& r) { return __fmul_rn(r.w, r.h); }

__device__ __forceinline__ Rect rect_intersect(const Rect& a, const Rect& b)
{
    const Rect zero{0, 0, 0, 0};
    if (rect_empty(a) || rect_empty(b)) return zero;
    const Rect& rx_min = (a.x < b.x) ? a : b;
    const Rect& rx_max = (a.x < b.x) ? b : a;
    const Rect& ry_min = (a.y < b.y) ? a : b;
    const Rect& ry_max = (a.y < b.y) ? b : a;
    if ((rx_min.x < 0 && __fadd_rn(rx_min.x, rx_min.w) < rx_max.x) || (ry_min.y < 0 && __fadd_rn(ry_min.y, ry_min.h) < ry_max.y))
        return zero;
    Rect r;
    r.w = fminf(__fsub_rn(rx_min.w, __fsub_rn(rx_max.x, rx_min.x)), rx_max.w);
    r.h = fminf(__fsub_rn(ry_min.h, __fsub_rn(ry_max.y, ry_min.y)), ry_max.h);
    r.x = rx_max.x;
    r.y = ry_max.y;
    if (rect_empty(r)) return zero;
    return r;
}

__device__ __forceinline__ float rect_iou(const Rect& a, const Rect& b)
{
    const float inter = rect_area(rect_intersect(a, b));
    const float uni = fmaxf(0.0f, __fsub_rn(__fadd_rn(rect_area(a), rect_area(b)), inter));
    const float r = __fdiv_rn(inter, uni);
    return (isnan(r) || isinf(r)) ? 0.0f : r;
}

__device__ __forceinline__ uint32_t prob_order(float f)
{
    // larger probability <=> larger integer, any sign; -0 and +0 compare equal in the reference's "a > b"
    if (f == 0.0f) f = 0.0f;
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// keys of the first sort (ascending: probability descending, then input index ascending), the boxes as the
// host form normalises them, and the per-record image / class words
__global__ void nms_prepare_kernel(const pxe_detection* dets, int n, unsigned long long* key, Rect* rect,
                                   unsigned* image, unsigned* cls)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const pxe_detection d = gld(dets + i);
    gst(key + i, ((unsigned long long)(~prob_order(d.prob)) << 32) | (unsigned)i);
    const float x2 = __fadd_rn(d.x, d.w), y2 = __fadd_rn(d.y, d.h);
    const float xa = fminf(d.x, x2), ya = fminf(d.y, y2), xb = fmaxf(d.x, x2), yb = fmaxf(d.y, y2);
    gst(rect + i, Rect{xa, ya, fmaxf(0.0f, __fsub_rn(xb, xa)), fmaxf(0.0f, __fsub_rn(yb, ya))});
    gst(image + i, (unsigned)d.batch_id);
    gst(cls + i, (unsigned)d.class_id);
}

// after the first sort: order[r] = input index of the r-th record; keys for the two segment sorts
__global__ void nms_segment_keys_kernel(const unsigned long long* sorted_key, const unsigned* image, const unsigned* cls,
                                        int n, int* order, unsigned* image_key, unsigned long long* group_key)
{
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    const int i = (int)(unsigned)gld(sorted_key + r);
    gst(order + r, i);
    gst(image_key + r, gld(image + i));
    gst(group_key + r, ((unsigned long long)gld(image + i) << 32) | gld(cls + i));
}

// starts[s] = first position of segment s in a sorted key array; *count = number of segments
template <typename K>
__global__ void nms_segment_starts_kernel(const K* sorted, int n, int* starts, int* count)
{
    // one block; segments are listed in ascending position so that a segment's end is the next start.  A thread takes
    // eight consecutive positions per turn, so a turn's three barriers cover 8192 positions.
    constexpr int U = 8;
    __shared__ int warp_tot[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < n; base += U * blockDim.x) {
        const int i0 = base + U * threadIdx.x;
        K key[U + 1];
        key[0] = (i0 > 0 && i0 - 1 < n) ? gld(sorted + (i0 - 1)) : K(0);
#pragma unroll
        for (int k = 0; k < U; ++k) key[k + 1] = i0 + k < n ? gld(sorted + (i0 + k)) : K(0);
        unsigned flags = 0;
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (i0 + k < n && (i0 + k == 0 || key[k + 1] != key[k])) flags |= 1u << k;
        const int mine = __popc(flags);
        int inc = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        int before = carry;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        int at = before + inc - mine;
#pragma unroll
        for (int k = 0; k < U; ++k)
            if ((flags >> k) & 1u) gst(starts + at++, i0 + k);
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + inc;
        __syncthreads();
    }
    if (threadIdx.x == 0) gst(count, carry);
}

// Step 2.  members[start..end) = input indices of one image's records in probability order.  An image with at
// most kImageStage records is staged in shared memory first, so that a pivot step costs a barrier and a few
// shared-memory reads instead of a chain of dependent global loads; longer segments run from global memory.
constexpr int kImageStage = 4096;
constexpr int kPairCap = 1024;
constexpr size_t kPairBytes = (size_t)kPairCap * (sizeof(Rect) + sizeof(unsigned) + 32 * sizeof(unsigned) + sizeof(float) + 1) + 32 * sizeof(unsigned);
constexpr size_t kImageStageBytes = (size_t)kImageStage * (sizeof(Rect) + sizeof(unsigned) + 1) > kPairBytes
                                        ? (size_t)kImageStage * (sizeof(Rect) + sizeof(unsigned) + 1) : kPairBytes;

__global__ void __launch_bounds__(1024)
nms_cross_class_kernel(const int* members, const int* starts, const int* nseg, int n, const Rect* rect,
                       const unsigned* cls, unsigned char* discard)
{
    extern __shared__ __align__(16) unsigned char stage_raw[];
    Rect* sbox = reinterpret_cast<Rect*>(stage_raw);
    unsigned* scls = reinterpret_cast<unsigned*>(sbox + kImageStage);
    unsigned char* sdead = reinterpret_cast<unsigned char*>(scls + kImageStage);
    const int segs = gld(nseg);
    for (int s = blockIdx.x; s < segs; s += gridDim.x) {
        const int lo = gld(starts + s), hi = s + 1 < segs ? gld(starts + (s + 1)) : n;
        const int cnt = hi - lo;
        if (cnt <= kPairCap) {
            // Up to 1024 boxes: every "q would fall to p" (p before q, other class, IoU above 0.9) is found first, by all
            // warps at once, as one bit of row q of a triangular matrix in shared memory; one warp then walks the rows
            // that have a bit set, in order, and discards q when one of its p is still standing.  That is the loop below
            // -- p discards q only while p stands -- without a barrier per box.
            Rect* pbox = reinterpret_cast<Rect*>(stage_raw);
            unsigned* pcls = reinterpret_cast<unsigned*>(pbox + kPairCap);
            unsigned* mask = pcls + kPairCap;                              // [kPairCap][32] words, row q: bits p < q
            unsigned* deadw = mask + kPairCap * 32;                        // [32]
            float* parea = reinterpret_cast<float*>(deadw + 32);              // [kPairCap]
            unsigned char* rowflag = reinterpret_cast<unsigned char*>(parea + kPairCap);
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
            for (int t = threadIdx.x; t < cnt; t += blockDim.x) {
                const int j = gld(members + (lo + t));
                pbox[t] = gld(rect + j);
                pcls[t] = gld(cls + j);
                // the area, or a NaN (which sends every pair of this box to the exact expression) when the box is so
                // small against its coordinates that the rounding of x + w could change an intersection by a per cent
                const Rect bx = pbox[t];
                const bool plain = fabsf(bx.x) + bx.w <= 16384.0f * bx.w && fabsf(bx.y) + bx.h <= 16384.0f * bx.h;
                parea[t] = plain ? rect_area(bx) : __int_as_float(0x7fc00000);
            }
            __syncthreads();
            for (int q = warp; q < cnt; q += warps) {
                const Rect rq = pbox[q];
                const unsigned cq = pcls[q];
                const float aq = parea[q];
                unsigned any = 0;
                for (int w = 0; 32 * w < q; ++w) {
                    const int pp = 32 * w + lane;
                    bool hit = false;
                    if (pp < q && pcls[pp] != cq) {
                        // Two bounds spare most pairs the exact expression.  IoU <= smaller area / larger area, and
                        // IoU <= (width of the intersection) / (width of q), likewise for the heights: a pair that is
                        // below 0.8 on one of them cannot reach 0.9, with a margin many times the rounding of the exact
                        // expression.  An area that is a NaN (see above) sends the pair to the exact expression.
                        const float ap = parea[pp];
                        const Rect rp = pbox[pp];
                        bool maybe = !(aq < 0.8f * ap || ap < 0.8f * aq);
                        if (maybe && aq == aq && ap == ap) {
                            const float wi = fminf(rq.x + rq.w, rp.x + rp.w) - fmaxf(rq.x, rp.x);
                            const float hi = fminf(rq.y + rq.h, rp.y + rp.h) - fmaxf(rq.y, rp.y);
                            maybe = !(wi < 0.8f * rq.w || hi < 0.8f * rq.h);
                        }
                        if (maybe) hit = rect_iou(rq, rp) > 0.9f;
                    }
                    const unsigned word = __ballot_sync(0xffffffffu, hit);
                    if (lane == 0) mask[q * 32 + w] = word;
                    any |= word;
                }
                if (lane == 0) rowflag[q] = any != 0;
            }
            __syncthreads();
            if (warp == 0) {
                unsigned dead = 0;                                         // lane w: boxes 32w .. 32w + 31
                for (int q = 1; q < cnt; ++q) {
                    if (!rowflag[q]) continue;                             // the same for every lane
                    const unsigned m = 32 * lane < q ? mask[q * 32 + lane] : 0u;
                    if (__any_sync(0xffffffffu, (m & ~dead) != 0u) && lane == (q >> 5)) dead |= 1u << (q & 31);
                }
                deadw[lane] = dead;
            }
            __syncthreads();
            for (int t = threadIdx.x; t < cnt; t += blockDim.x)
                if ((deadw[t >> 5] >> (t & 31)) & 1u) gst(discard + (gld(members + (lo + t))), 1);
            __syncthreads();
            continue;
        }
        if (cnt <= kImageStage) {
            for (int t = threadIdx.x; t < cnt; t += blockDim.x) {
                const int j = gld(members + (lo + t));
                sbox[t] = gld(rect + j);
                scls[t] = gld(cls + j);
                sdead[t] = 0;                              // nothing has been discarded before this step
            }
            __syncthreads();
            for (int p = 0; p < cnt; ++p) {
                if (sdead[p]) continue;                    // block-uniform: written before the last barrier
                const Rect ri = sbox[p];
                const unsigned ci = scls[p];
                for (int q = p + 1 + (int)threadIdx.x; q < cnt; q += blockDim.x)
                    if (scls[q] != ci && !sdead[q] && rect_iou(sbox[q], ri) > 0.9f) sdead[q] = 1;
                __syncthreads();
            }
            for (int t = threadIdx.x; t < cnt; t += blockDim.x)
                if (sdead[t]) gst(discard + (gld(members + (lo + t))), 1);
            __syncthreads();
            continue;
        }
        for (int p = lo; p < hi; ++p) {
            const int i = gld(members + p);
            if (gld(discard + i)) continue;                      // block-uniform: written before the last barrier
            const Rect ri = gld(rect + i);
            const unsigned ci = gld(cls + i);
            for (int q = p + 1 + (int)threadIdx.x; q < hi; q += blockDim.x) {
                const int j = gld(members + q);
                if (gld(cls + j) != ci && !gld(discard + j) && rect_iou(gld(rect + j), ri) > 0.9f) gst(discard + j, 1);
            }
            __syncthreads();
        }
        __syncthreads();
    }
}

// Step 3.  members[start..end) = one (image, class) group in probability order; only its first 1024 positions
// take part (src/Box.cpp:104), records behind them are left as they are.
constexpr int kGroupCap = 1024;

__global__ void __launch_bounds__(kGroupCap)
nms_group_kernel(const int* members, const int* starts, const int* nseg, int n, const Rect* rect, float threshold,
                 unsigned char* discard)
{
    __shared__ Rect box[kGroupCap];
    __shared__ unsigned char dead[kGroupCap];
    const int segs = gld(nseg);
    for (int s = blockIdx.x; s < segs; s += gridDim.x) {
        const int lo = gld(starts + s), hi = s + 1 < segs ? gld(starts + (s + 1)) : n;
        if (hi - lo <= 32) continue;                       // nms_small_group_kernel's
        const int count = min(hi - lo, kGroupCap);
        const int t = threadIdx.x;
        int mine = -1;
        if (t < count) {
            mine = gld(members + (lo + t));
            box[t] = gld(rect + mine);
            dead[t] = gld(discard + mine);
        }
        __syncthreads();
        for (int p = 0; p < count; ++p) {
            if (dead[p]) continue;                         // block-uniform: shared memory, read after a barrier
            if (t > p && t < count && !dead[t] && rect_iou(box[t], box[p]) > threshold) dead[t] = 1;
            __syncthreads();
        }
        if (t < count && dead[t]) gst(discard + mine, 1);
        __syncthreads();
    }
}

// The same rule for groups of up to 32 members (a head with 80 classes leaves a dozen candidates per image and class):
// a warp per group, a lane per member, the pivot's box handed round by shuffles -- no shared memory, no barrier.
__global__ void __launch_bounds__(256)
nms_small_group_kernel(const int* members, const int* starts, const int* nseg, int n, const Rect* rect, float threshold,
                       unsigned char* discard)
{
    const int segs = gld(nseg);
    const int lane = threadIdx.x & 31;
    const int first = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5), step = (int)((gridDim.x * blockDim.x) >> 5);
    for (int s = first; s < segs; s += step) {
        const int lo = gld(starts + s), hi = s + 1 < segs ? gld(starts + (s + 1)) : n;
        const int count = hi - lo;
        if (count > 32 || count < 2) continue;             // the same for the whole warp
        int mine = -1;
        Rect b{0.0f, 0.0f, 0.0f, 0.0f};
        bool dead = true;
        if (lane < count) {
            mine = gld(members + (lo + lane));
            b = gld(rect + mine);
            dead = gld(discard + mine) != 0;
        }
        bool fell = false;
        for (int p = 0; p + 1 < count; ++p) {
            if (__shfl_sync(0xffffffffu, (int)dead, p)) continue;          // a discarded member discards nobody
            Rect bp;
            bp.x = __shfl_sync(0xffffffffu, b.x, p); bp.y = __shfl_sync(0xffffffffu, b.y, p);
            bp.w = __shfl_sync(0xffffffffu, b.w, p); bp.h = __shfl_sync(0xffffffffu, b.h, p);
            if (lane > p && lane < count && !dead && rect_iou(b, bp) > threshold) { dead = true; fell = true; }
        }
        if (fell) gst(discard + mine, 1);
    }
}

// keep[r] = 1 when the r-th record of the probability order survives
__global__ void nms_keep_flags_kernel(const int* order, const unsigned char* discard, int n, unsigned char* keep)
{
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n) gst(keep + r, gld(discard + (gld(order + r))) ? 0 : 1);
}

__global__ void nms_gather_kernel(const pxe_detection* dets, const int* kept_order, const int* kept_count,
                                  pxe_detection* out, long long* out_count)
{
    const int m = gld(kept_count);
    if (blockIdx.x == 0 && threadIdx.x == 0) gst(out_count, m);
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < m; k += gridDim.x * blockDim.x) {
        const float4* src = reinterpret_cast<const float4*>(dets + gld(kept_order + k));
        float4* dst = reinterpret_cast<float4*>(out + k);
        gst(dst, gld(src));
        gst(dst + 1, gld(src + 1));
    }
}

struct Layout {
    size_t key_a, key_b, group_a, group_b, rect, image, cls, order, order_b, order_c, image_a, image_b,
           starts_img, starts_grp, counts, discard, keep, kept, cub, total;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t cub_bytes(int n)
{
    size_t a = 0, b = 0, c = 0, d = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, a, (unsigned long long*)nullptr, (unsigned long long*)nullptr, n);
    cub::DeviceRadixSort::SortPairs(nullptr, b, (unsigned*)nullptr, (unsigned*)nullptr, (int*)nullptr, (int*)nullptr, n);
    cub::DeviceRadixSort::SortPairs(nullptr, c, (unsigned long long*)nullptr, (unsigned long long*)nullptr, (int*)nullptr,
                                    (int*)nullptr, n);
    cub::DeviceSelect::Flagged(nullptr, d, (int*)nullptr, (unsigned char*)nullptr, (int*)nullptr, (int*)nullptr, n);
    size_t m = a > b ? a : b;
    m = m > c ? m : c;
    return m > d ? m : d;
}

Layout layout(int n)
{
    Layout L{};
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t at = off; off += align_up(bytes, 256); return at; };
    const size_t N = (size_t)n;
    L.key_a = take(8 * N); L.key_b = take(8 * N);
    L.group_a = take(8 * N); L.group_b = take(8 * N);
    L.rect = take(16 * N);
    L.image = take(4 * N); L.cls = take(4 * N);
    L.order = take(4 * N); L.order_b = take(4 * N); L.order_c = take(4 * N);
    L.image_a = take(4 * N); L.image_b = take(4 * N);
    L.starts_img = take(4 * N); L.starts_grp = take(4 * N);
    L.counts = take(16);
    L.discard = take(N); L.keep = take(N);
    L.kept = take(4 * N);
    L.cub = take(cub_bytes(n));
    L.total = off;
    return L;
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" size_t pxe_nms_workspace_bytes(long long n)
{
    if (n <= 0 || n > 0x7fffffffLL) return 0;
    return layout((int)n).total;
}

extern "C" int pxe_nms(pxe_stream_t stream, const pxe_detection* dets, long long n, float threshold,
                       pxe_detection* out, long long* out_count, void* workspace, size_t workspace_bytes)
{
    PXE_REQUIRE(out_count != nullptr, "nms: out_count is null");
    PXE_REQUIRE(n >= 0 && n <= 0x7fffffffLL, "nms: n = %lld out of range", n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n == 0) {
        PXE_CUDA_OK(cudaMemsetAsync(out_count, 0, sizeof(long long), s));
        return PXE_OK;
    }
    PXE_REQUIRE(dets && out && workspace, "nms: null pointer");
    PXE_REQUIRE(dets != out, "nms: out must not alias dets");
    PXE_REQUIRE(aligned16(dets) && aligned16(out), "nms: records must be 16-byte aligned");
    PXE_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "nms: workspace must be 256-byte aligned");
    const int N = (int)n;
    const Layout L = layout(N);
    if (workspace_bytes < L.total)
        return set_error(PXE_ERR_WORKSPACE, "nms: workspace %zu bytes, need %zu", workspace_bytes, L.total);
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;

    char* ws = static_cast<char*>(workspace);
    auto* key_a = reinterpret_cast<unsigned long long*>(ws + L.key_a);
    auto* key_b = reinterpret_cast<unsigned long long*>(ws + L.key_b);
    auto* group_a = reinterpret_cast<unsigned long long*>(ws + L.group_a);
    auto* group_b = reinterpret_cast<unsigned long long*>(ws + L.group_b);
    auto* rect = reinterpret_cast<Rect*>(ws + L.rect);
    auto* image = reinterpret_cast<unsigned*>(ws + L.image);
    auto* cls = reinterpret_cast<unsigned*>(ws + L.cls);
    auto* order = reinterpret_cast<int*>(ws + L.order);
    auto* by_image = reinterpret_cast<int*>(ws + L.order_b);
    auto* by_group = reinterpret_cast<int*>(ws + L.order_c);
    auto* image_a = reinterpret_cast<unsigned*>(ws + L.image_a);
    auto* image_b = reinterpret_cast<unsigned*>(ws + L.image_b);
    auto* starts_img = reinterpret_cast<int*>(ws + L.starts_img);
    auto* starts_grp = reinterpret_cast<int*>(ws + L.starts_grp);
    auto* counts = reinterpret_cast<int*>(ws + L.counts);          // [0] images, [1] groups, [2] kept
    auto* discard = reinterpret_cast<unsigned char*>(ws + L.discard);
    auto* keep = reinterpret_cast<unsigned char*>(ws + L.keep);
    auto* kept = reinterpret_cast<int*>(ws + L.kept);
    void* cub_ws = ws + L.cub;
    size_t cub_n = L.total - L.cub;

    const unsigned blocks = (unsigned)((N + 255) / 256);
    PXE_CUDA_OK(cudaMemsetAsync(discard, 0, (size_t)N, s));
    nms_prepare_kernel<<<blocks, 256, 0, s>>>(dets, N, key_a, rect, image, cls);
    PXE_LAUNCH_OK("nms_prepare_kernel");
    PXE_CUDA_OK(cub::DeviceRadixSort::SortKeys(cub_ws, cub_n, key_a, key_b, N, 0, 64, s));
    nms_segment_keys_kernel<<<blocks, 256, 0, s>>>(key_b, image, cls, N, order, image_a, group_a);
    PXE_LAUNCH_OK("nms_segment_keys_kernel");
    PXE_CUDA_OK(cub::DeviceRadixSort::SortPairs(cub_ws, cub_n, image_a, image_b, order, by_image, N, 0, 32, s));
    PXE_CUDA_OK(cub::DeviceRadixSort::SortPairs(cub_ws, cub_n, group_a, group_b, order, by_group, N, 0, 64, s));
    nms_segment_starts_kernel<unsigned><<<1, 1024, 0, s>>>(image_b, N, starts_img, counts + 0);
    PXE_LAUNCH_OK("nms_segment_starts_kernel");
    nms_segment_starts_kernel<unsigned long long><<<1, 1024, 0, s>>>(group_b, N, starts_grp, counts + 1);
    PXE_LAUNCH_OK("nms_segment_starts_kernel");
    const unsigned seg_blocks = (unsigned)(N < 4 * di.sm_count ? N : 4 * di.sm_count);
    PXE_CUDA_OK(cudaFuncSetAttribute(nms_cross_class_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kImageStageBytes));
    nms_cross_class_kernel<<<seg_blocks, 1024, kImageStageBytes, s>>>(by_image, starts_img, counts + 0, N, rect, cls, discard);
    PXE_LAUNCH_OK("nms_cross_class_kernel");
    nms_group_kernel<<<seg_blocks, kGroupCap, 0, s>>>(by_group, starts_grp, counts + 1, N, rect, threshold, discard);
    PXE_LAUNCH_OK("nms_group_kernel");
    const unsigned small_blocks = (unsigned)std::min<long long>(((long long)N + 7) / 8, 8LL * di.sm_count);
    nms_small_group_kernel<<<small_blocks, 256, 0, s>>>(by_group, starts_grp, counts + 1, N, rect, threshold, discard);
    PXE_LAUNCH_OK("nms_small_group_kernel");
    nms_keep_flags_kernel<<<blocks, 256, 0, s>>>(order, discard, N, keep);
    PXE_LAUNCH_OK("nms_keep_flags_kernel");
    PXE_CUDA_OK(cub::DeviceSelect::Flagged(cub_ws, cub_n, order, keep, kept, counts + 2, N, s));
    nms_gather_kernel<<<blocks < 1024 ? blocks : 1024, 256, 0, s>>>(dets, kept, counts + 2, out, out_count);
    PXE_LAUNCH_OK("nms_gather_kernel");
    return PXE_OK;
}
