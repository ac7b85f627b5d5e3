// Detection heads on the device: YOLO activate + decode, CenterNet activate + decode,
// softmax and the YOLOv2 region transform.  The reference decodes on the host after copying the
// whole head tensor back (include/cuda/YoloLayer.h:168-188, include/cuda/CenterNetLayer.h:89-106,
// include/cuda/RegionLayer.h:39-54); here only the compacted detections leave the GPU.
#include <climits>
#include <mutex>

#include "pxe_common.cuh"

namespace pxe {
namespace {

// ============================================================================================
// YOLO
// ============================================================================================
// Work decomposition.  A block covers 32 consecutive cells of one image.  Warp w of the block handles
// mask slot (w / chunks) and class chunk (w % chunks) for those 32 cells, lane = cell, so every
// global load is one coalesced 128-byte row segment of a head plane.  A chunk is at most
// kYoloChunk classes, whose probabilities a thread keeps in registers between counting and emitting.
// The reference emits cell-major, then mask slot, then class (include/YoloLayer.h:668-697); in
// that order thread (lane, w) has rank lane * warps + w inside its block.
constexpr int kYoloCells = 32;
constexpr int kYoloChunk = 16;
constexpr int kYoloMaxWarps = 32;

struct YoloParams {
    pxe_yolo_decode_desc d;
    long long hbs;
    int HW, entries, blocks_per_image;
    int chunks, chunk_len, warps;     // class chunks per mask slot, classes per chunk, warps per block
    pxe_detection* dets;
    long long capacity;
    long long* count;
    int* block_sums;           // [batch*blocks_per_image]
    long long* block_offsets;  // [batch*blocks_per_image]
};

// value of entry `e` of mask slot `n` at `cell`, activated as YoloLayer::forward leaves it
// (logistic on x, y, objectness, classes; w, h raw -- src/YoloKernels.cu:63-71)
__device__ __forceinline__ float yolo_value(const YoloParams& p, const float* img, int n, int e, int cell)
{
    const int ch = n * p.entries + e;
    float v = img[(long long)ch * p.HW + cell];
    if (p.d.head_is_raw) {
        if (p.d.bias) v += p.d.bias[ch];
        if (e < 2 || e >= 4) v = act_logistic(v);
    }
    return v;
}

// Probabilities of this thread's class chunk that reach the threshold; returns their number and
// leaves them in prob[] (negative = not emitted).  obj < threshold skips the slot entirely
// (include/YoloLayer.h:676); a class is emitted when obj * cls >= threshold (:692).
__device__ __forceinline__ int yolo_chunk(const YoloParams& p, const float* img, int n, int chunk, int cell,
                                          float (&prob)[kYoloChunk], float* obj_out)
{
    const float obj = yolo_value(p, img, n, 4, cell);
    *obj_out = obj;
    if (obj < p.d.threshold) return 0;
    int cnt = 0;
    const int c0 = chunk * p.chunk_len;
    const int cend = min(c0 + p.chunk_len, p.d.classes);
    // Raw heads: obj * sigmoid(v) >= thr needs v >= logit(thr / obj).  Values clearly below that bound (by a
    // margin far wider than any rounding in the sigmoid or the product) are skipped without evaluating the
    // sigmoid; everything else goes through the exact expression, so the emitted set is unchanged.
    float skip_below = -INFINITY;
    if (p.d.head_is_raw && p.d.threshold > 0.0f) {
        const float ratio = p.d.threshold / obj;
        if (ratio < 0.999f) {
            const float l = logf(ratio / (1.0f - ratio));
            skip_below = l - 1e-3f - 1e-3f * fabsf(l);
        }
    }
#pragma unroll
    for (int j = 0; j < kYoloChunk; ++j) {
        prob[j] = -1.0f;
        const int cls = c0 + j;
        if (cls < cend) {
            const int ch = n * p.entries + 5 + cls;
            float v = img[(long long)ch * p.HW + cell];
            if (p.d.head_is_raw) {
                if (p.d.bias) v += p.d.bias[ch];
                if (v < skip_below) continue;
                v = act_logistic(v);
            }
            const float pr = obj * v;
            if (pr >= p.d.threshold) { prob[j] = pr; ++cnt; }
        }
    }
    // chunks longer than the register window (very many classes): the rest is only counted here and
    // recomputed when emitting
    for (int cls = c0 + kYoloChunk; cls < cend; ++cls)
        if (obj * yolo_value(p, img, n, 5 + cls, cell) >= p.d.threshold) ++cnt;
    return cnt;
}

__global__ void __launch_bounds__(kYoloCells * kYoloMaxWarps)
yolo_count_kernel(const YoloParams p)
{
    __shared__ int warp_sums[kYoloMaxWarps];
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int cell = blockIdx.x * kYoloCells + lane;
    const float* img = p.d.head + (long long)b * p.hbs;
    int cnt = 0;
    if (cell < p.HW) {
        float prob[kYoloChunk], obj;
        cnt = yolo_chunk(p, img, w / p.chunks, w % p.chunks, cell, prob, &obj);
    }
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_down_sync(0xffffffffu, cnt, o);
    if (lane == 0) warp_sums[w] = cnt;
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int i = 0; i < p.warps; ++i) total += warp_sums[i];
        p.block_sums[b * p.blocks_per_image + blockIdx.x] = total;
    }
}

// Exclusive scan of the per-block sums; starts at the running total *count and advances it.
__global__ void __launch_bounds__(1024)
yolo_scan_kernel(const int* block_sums, long long* block_offsets, int n, long long* count)
{
    __shared__ long long warp_tot[32];
    __shared__ long long carry;
    if (threadIdx.x == 0) carry = *count;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        long long v = i < n ? block_sums[i] : 0;
        long long inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            long long t = __shfl_up_sync(0xffffffffu, inc, o);
            if ((threadIdx.x & 31) >= o) inc += t;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        if (threadIdx.x < 32) {
            long long w = warp_tot[threadIdx.x];
            for (int o = 1; o < 32; o <<= 1) {
                long long t = __shfl_up_sync(0xffffffffu, w, o);
                if (threadIdx.x >= o) w += t;
            }
            warp_tot[threadIdx.x] = w;          // inclusive totals of warps
        }
        __syncthreads();
        const long long warp_excl = (threadIdx.x >> 5) ? warp_tot[(threadIdx.x >> 5) - 1] : 0;
        const long long c = carry;
        if (i < n) block_offsets[i] = c + warp_excl + inc - v;
        __syncthreads();
        if (threadIdx.x == 0) carry = c + warp_tot[31];
        __syncthreads();
    }
    if (threadIdx.x == 0) *count = carry;
}

// One 32-byte record as two 128-bit stores (records are 16-byte aligned).
__device__ __forceinline__ void store_detection(pxe_detection* dst, float x, float y, float w, float h, float prob,
                                                int class_id, int batch_id, int source)
{
    float4* q = reinterpret_cast<float4*>(dst);
    q[0] = make_float4(x, y, w, h);
    q[1] = make_float4(prob, __int_as_float(class_id), __int_as_float(batch_id), __int_as_float(source));
}

// float -> int the way the reference's host decode converts (x86-64 cvttss2si):
// truncation toward zero, INT_MIN for NaN and out-of-range values.
__device__ __forceinline__ int f2i_x86(float v)
{
    if (!(v > -2147483904.0f && v < 2147483648.0f)) return INT_MIN;
    return (int)v;
}

__global__ void __launch_bounds__(kYoloCells * kYoloMaxWarps)
yolo_emit_kernel(const YoloParams p)
{
    __shared__ int ranked[kYoloCells * (kYoloMaxWarps + 1)];   // counts, then exclusive prefixes, in emission order
    __shared__ int warp_tot[kYoloMaxWarps];
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int cell = blockIdx.x * kYoloCells + lane;
    const float* img = p.d.head + (long long)b * p.hbs;
    const int n = w / p.chunks, chunk = w % p.chunks;
    float prob[kYoloChunk], obj = 0.0f;
    int cnt = 0;
    if (cell < p.HW) cnt = yolo_chunk(p, img, n, chunk, cell, prob, &obj);
    // exclusive scan over the block in emission order: rank = lane * warps + w
    const int nthreads = kYoloCells * p.warps;
    ranked[lane * p.warps + w] = cnt;
    __syncthreads();
    {
        const int v = ranked[threadIdx.x];            // thread t now owns rank t
        int inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) warp_tot[w] = inc;
        __syncthreads();
        int before = 0;
        for (int i = 0; i < w; ++i) before += warp_tot[i];
        ranked[threadIdx.x] = before + inc - v;
        (void)nthreads;
    }
    __syncthreads();
    if (cnt == 0) return;
    long long pos = p.block_offsets[b * p.blocks_per_image + blockIdx.x] + ranked[lane * p.warps + w];

    const int W = p.d.width, H = p.d.height;
    const int row = cell / W, col = cell - row * W;
    const bool scaled = p.d.image_width > 0 && p.d.image_height > 0;
    const float tx = yolo_value(p, img, n, 0, cell), ty = yolo_value(p, img, n, 1, cell);
    const float tw = yolo_value(p, img, n, 2, cell), th = yolo_value(p, img, n, 3, cell);
    const int a = p.d.mask[n];
    const int aw = p.d.anchors[2 * a], ah = p.d.anchors[2 * a + 1];
    const int net_w = p.d.net_width, net_h = p.d.net_height;
    float bx, by, bw, bh;
    if (scaled) {
        // scaledYoloBox, include/YoloLayer.h:601-635
        const int iw = p.d.image_width, ih = p.d.image_height;
        int new_w, new_h;
        if (((float)net_w / iw) < ((float)net_h / ih)) { new_w = net_w; new_h = (ih * net_w) / iw; }
        else { new_h = net_h; new_w = (iw * net_h) / ih; }
        float x = (col + tx) / W;
        x = (x - (net_w - new_w) / 2.0f / net_w) / ((float)new_w / net_w);
        float y = (row + ty) / H;
        y = (y - (net_h - new_h) / 2.0f / net_h) / ((float)new_h / net_h);
        float width = expf(tw) * aw / net_w;
        width *= (float)net_w / new_w;
        float height = expf(th) * ah / net_h;
        height *= (float)net_h / new_h;
        int left = f2i_x86(__fmul_rn(__fsub_rn(x, width / 2), (float)iw));    if (left < 0) left = 0;
        int right = f2i_x86(__fmul_rn(__fadd_rn(x, width / 2), (float)iw));   if (right > iw - 1) right = iw - 1;
        int top = f2i_x86(__fmul_rn(__fsub_rn(y, height / 2), (float)ih));    if (top < 0) top = 0;
        int bottom = f2i_x86(__fmul_rn(__fadd_rn(y, height / 2), (float)ih)); if (bottom > ih - 1) bottom = ih - 1;
        bx = (float)left; by = (float)top; bw = (float)(right - left); bh = (float)(bottom - top);
    } else {
        // yoloBox().rect(), include/YoloLayer.h:637-651, src/DarkBox.cpp:84-123
        const float x = (col + tx) / W, y = (row + ty) / H;
        const float wd = expf(tw) * aw / net_w, ht = expf(th) * ah / net_h;
        bx = wd > 0.0f ? __fsub_rn(x, wd / 2.0f) : x;
        by = ht > 0.0f ? __fsub_rn(y, ht / 2.0f) : y;
        bw = wd; bh = ht;
    }
    const int c0 = chunk * p.chunk_len;
#pragma unroll
    for (int j = 0; j < kYoloChunk; ++j) {
        if (prob[j] >= 0.0f) {
            if (pos < p.capacity)
                store_detection(p.dets + pos, bx, by, bw, bh, prob[j], c0 + j, b + p.d.batch_id_offset,
                                cell * p.d.n_masks + n);
            ++pos;
        }
    }
    const int cend = min(c0 + p.chunk_len, p.d.classes);
    for (int cls = c0 + kYoloChunk; cls < cend; ++cls) {
        const float pr = obj * yolo_value(p, img, n, 5 + cls, cell);
        if (pr >= p.d.threshold) {
            if (pos < p.capacity)
                store_detection(p.dets + pos, bx, by, bw, bh, pr, cls, b + p.d.batch_id_offset, cell * p.d.n_masks + n);
            ++pos;
        }
    }
}

// ============================================================================================
// CenterNet
// ============================================================================================
struct CnActParams {
    const float* in; float* out;
    uint32_t total;      // elements (scalar) or float4 vectors
    uint32_t outputs, heat;   // per image, in the same unit as total
    float bias;
    FastDiv div_outputs;
};

template <bool VEC>
__global__ void __launch_bounds__(256)
centernet_activate_kernel(const CnActParams p)
{
    for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < p.total; i += gridDim.x * 256) {
        uint32_t q, within;
        p.div_outputs.divmod(i, q, within);
        const bool heat = within < p.heat;
        if (VEC) {
            float4 v = reinterpret_cast<const float4*>(p.in)[i];
            if (heat) {
                v.x = act_logistic(v.x + p.bias); v.y = act_logistic(v.y + p.bias);
                v.z = act_logistic(v.z + p.bias); v.w = act_logistic(v.w + p.bias);
            }
            reinterpret_cast<float4*>(p.out)[i] = v;
        } else {
            float v = p.in[i];
            if (heat) v = act_logistic(v + p.bias);
            p.out[i] = v;
        }
    }
}

constexpr int kCnTileH = 32, kCnTileW = 64, kCnThreads = 256;
constexpr int kCnCells = kCnTileH * kCnTileW;
constexpr int kCnMaxK = 1024;
constexpr int kCnSlotCap = 256;          // keys one tile may pass on without reducing them (at least K)

struct CnParams {
    pxe_centernet_decode_desc d;
    long long hbs, sbs, obs;
    int tiles_x, tiles_y;
    int K;
    int slots;                       // blocks per image (tiles x classes)
    int slot_cap;                    // keys a block may pass on: block s of image b owns cand[(b*slots+s)*slot_cap ...]
    float lo;                        // pre-filter: a cell with (value >= lo) false cannot reach the threshold
    float lo_list;                   // work-list bound, a margin below lo (see centernet_peaks_kernel)
    unsigned long long* cand;        // [batch][slots][K] sortable keys, unordered inside a slot
    int* cand_cnt;                   // [batch][slots]
    unsigned long long* list;        // [batch][slots*K] per-image compacted list, used when it exceeds shared memory
    pxe_detection* dets; int* counts;
};

// Monotone map float -> uint32 (larger float <=> larger integer), any sign.
__device__ __forceinline__ uint32_t float_order(float f)
{
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float order_float(uint32_t u)
{
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}
// Key orders candidates by score descending, then flat index ascending.  Never 0.
__device__ __forceinline__ unsigned long long cn_key(float score, uint32_t flat)
{
    return ((unsigned long long)float_order(score) << 32) | (unsigned long long)(0xffffffffu - flat);
}

// Finds the k-th largest of n distinct 64-bit keys (1 <= k <= n) by most-significant-digit radix
// selection, 8 bits per pass.  `get(i)` returns key i.  All threads of the block must call; every
// thread returns the key.  hist: 256 ints of shared memory, sh: 2 x u64.  With passes < 8 only the leading
// digits are resolved (see the end of the function).
template <typename Get>
__device__ unsigned long long block_select_kth(Get get, int n, int k, int* hist, unsigned long long* sh,
                                               int passes = 8, int* want_out = nullptr)
{
    unsigned long long prefix = 0, mask = 0;
    int want = k;
    for (int shift = 56; shift > 56 - 8 * passes; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        // Scores of one image share their leading bits, so most keys fall into one or two bins of the
        // early passes: lanes with equal digits are combined before touching shared memory.
        for (int i0 = 0; i0 < n; i0 += blockDim.x) {
            const int i = i0 + threadIdx.x;
            unsigned digit = 0x100u;                      // "no key": its own group, never counted
            if (i < n) {
                const unsigned long long key = get(i);
                if ((key & mask) == prefix) digit = (unsigned)((key >> shift) & 0xff);
            }
            const unsigned same = __match_any_sync(0xffffffffu, digit);
            if (digit < 0x100u && (threadIdx.x & 31) == (unsigned)(__ffs(same) - 1)) atomicAdd(&hist[digit], __popc(same));
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // lane L owns digits 255-8L .. 248-8L; find the digit where the running count from the
            // top first reaches `want`
            const int top = 255 - 8 * (int)threadIdx.x;
            int mine = 0;
            for (int j = 0; j < 8; ++j) mine += hist[top - j];
            int incl = mine;
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)threadIdx.x >= o) incl += t;
            }
            const int before = incl - mine;
            if (before < want && incl >= want) {
                int acc = before, digit = top;
                for (int j = 0; j < 8; ++j) {
                    if (acc + hist[top - j] >= want) { digit = top - j; break; }
                    acc += hist[top - j];
                }
                sh[0] = prefix | ((unsigned long long)digit << shift);
                sh[1] = (unsigned long long)(want - acc);
            }
        }
        __syncthreads();
        prefix = sh[0];
        want = (int)sh[1];
        mask |= 0xffULL << shift;
        __syncthreads();
    }
    // after fewer than 8 passes: `prefix` holds the leading digits of the k-th key and *want_out how many
    // keys with exactly those leading digits still belong to the k largest
    if (want_out) *want_out = want;
    return prefix;
}

// Descending bitonic sort of keys[0..pow2) in shared memory.
__device__ __forceinline__ void block_bitonic_desc(unsigned long long* keys, int pow2)
{
    for (int k = 2; k <= pow2; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < pow2; i += blockDim.x) {
                const int l = i ^ j;
                if (l > i) {
                    const unsigned long long a = keys[i], c = keys[l];
                    const bool desc = (i & k) == 0;
                    if (desc ? (a < c) : (a > c)) { keys[i] = c; keys[l] = a; }
                }
            }
            __syncthreads();
        }
}

__device__ __forceinline__ float cn_score(const CnParams& p, float v)
{
    // the reference's activation expression (src/CenterNetKernels.cu:17), precise math: scores and
    // therefore the kept indices are bit-identical to the reference's CUDA path
    return p.d.heat_is_logit ? 1.0f / (1.0f + expf(-v)) : v;
}

// include/CenterNetLayer.h:217-225: box size and centre offset must be finite and the size positive.
__device__ __forceinline__ bool cn_valid(const float* size, const float* off, long long idx, long long area, int W, int H)
{
    const float bw = size[idx] / W, bh = size[area + idx] / H;
    const float ox = off[idx], oy = off[area + idx];
    return isfinite(bw) && isfinite(bh) && isfinite(ox) && isfinite(oy) && bw > 0.0f && bh > 0.0f;
}

// One block per (32x64 tile, class, image).
//  load   the tile's pre-activation values (logit + bias) with a one-cell halo go to shared memory,
//         128 bits at a time where the row alignment allows; every value that is not clearly below the
//         threshold (in pre-activation space) is put on a work list on the way.  For a typical heatmap
//         that is about one cell in ten.
//  score  the activation (the reference's precise sigmoid) is evaluated once per work-list entry.
//  peak   interior entries at or above the threshold are compared with their 8 neighbours' scores.
//         A neighbour that is not on the work list is clearly below the threshold in pre-activation
//         space; the activation is non-decreasing, so its score cannot exceed that of a cell which
//         reached the threshold ("clearly" = a margin far wider than any rounding in exp()).
//  select a tile with more than K surviving candidates passes on only its K best.
constexpr int kCnRowStride = 72;                      // floats per shared-memory row; interior starts at column 4
constexpr int kCnSmemCells = (kCnTileH + 2) * kCnRowStride;

template <bool VEC>
__global__ void __launch_bounds__(kCnThreads)
centernet_peaks_kernel(const CnParams p)
{
    __shared__ __align__(16) float tile[kCnSmemCells];
    __shared__ __align__(16) float score[kCnSmemCells];
    __shared__ unsigned short work[(kCnTileH + 2) * (kCnTileW + 2)];
    __shared__ unsigned long long keys[kCnCells];
    __shared__ int n_keys, n_out, n_work, base;
    __shared__ int hist[256];
    __shared__ unsigned long long sel[2];

    const int b = blockIdx.z, cls = blockIdx.y;
    const int ty = blockIdx.x / p.tiles_x, tx = blockIdx.x - ty * p.tiles_x;
    const int y0 = ty * kCnTileH, x0 = tx * kCnTileW;
    const int H = p.d.height, W = p.d.width;
    const long long area = (long long)H * W;
    const float* heat = p.d.heat + (long long)b * p.hbs + (long long)cls * area;
    if (threadIdx.x == 0) { n_keys = 0; n_out = 0; n_work = 0; }
    __syncthreads();

    const bool logit = p.d.heat_is_logit != 0;
    const float bias = logit ? p.d.heatmap_bias : 0.0f;
    const float lo_list = p.lo_list;
    constexpr float NEG = -INFINITY;                  // outside the map: never greater than a score

    // ---- load + work list
    if (VEC) {
        // interior: 34 rows x 16 float4
        for (int i = threadIdx.x; i < (kCnTileH + 2) * (kCnTileW / 4); i += kCnThreads) {
            const int row = i / (kCnTileW / 4), vx = i - row * (kCnTileW / 4);
            const int gy = y0 + row - 1, gx = x0 + 4 * vx;
            float4 v = make_float4(NEG, NEG, NEG, NEG);
            if (gy >= 0 && gy < H && gx < W) {
                const float* src = heat + (long long)gy * W + gx;
                if (gx + 3 < W) {
                    v = *reinterpret_cast<const float4*>(src);
                    v.x += bias; v.y += bias; v.z += bias; v.w += bias;
                } else {
                    v.x = src[0] + bias;
                    if (gx + 1 < W) v.y = src[1] + bias;
                    if (gx + 2 < W) v.z = src[2] + bias;
                }
            }
            const int si = row * kCnRowStride + 4 + 4 * vx;
            *reinterpret_cast<float4*>(tile + si) = v;
            *reinterpret_cast<float4*>(score + si) = make_float4(NEG, NEG, NEG, NEG);
            const int hx = v.x >= lo_list, hy = v.y >= lo_list, hz = v.z >= lo_list, hw = v.w >= lo_list;
            const int hits = hx + hy + hz + hw;
            if (hits) {                                  // one reservation per thread, not per element
                int at = atomicAdd(&n_work, hits);
                if (hx) work[at++] = (unsigned short)si;
                if (hy) work[at++] = (unsigned short)(si + 1);
                if (hz) work[at++] = (unsigned short)(si + 2);
                if (hw) work[at] = (unsigned short)(si + 3);
            }
        }
        // halo columns: 34 rows x {left, right}
        for (int i = threadIdx.x; i < (kCnTileH + 2) * 2; i += kCnThreads) {
            const int row = i >> 1, side = i & 1;
            const int gy = y0 + row - 1, gx = side ? x0 + kCnTileW : x0 - 1;
            float v = NEG;
            if (gy >= 0 && gy < H && gx >= 0 && gx < W) v = heat[(long long)gy * W + gx] + bias;
            const int si = row * kCnRowStride + (side ? 4 + kCnTileW : 3);
            tile[si] = v;
            score[si] = NEG;
            if (v >= lo_list) work[atomicAdd(&n_work, 1)] = (unsigned short)si;
        }
    } else {
        for (int i = threadIdx.x; i < (kCnTileH + 2) * (kCnTileW + 2); i += kCnThreads) {
            const int row = i / (kCnTileW + 2), lx = i - row * (kCnTileW + 2);
            const int gy = y0 + row - 1, gx = x0 + lx - 1;
            float v = NEG;
            if (gy >= 0 && gy < H && gx >= 0 && gx < W) v = heat[(long long)gy * W + gx] + bias;
            const int si = row * kCnRowStride + 3 + lx;
            tile[si] = v;
            score[si] = NEG;
            if (v >= lo_list) work[atomicAdd(&n_work, 1)] = (unsigned short)si;
        }
    }
    __syncthreads();

    // ---- score: the reference's activation expression, once per listed cell
    const int todo = n_work;
    for (int wi = threadIdx.x; wi < todo; wi += kCnThreads) {
        const int si = work[wi];
        score[si] = cn_score(p, tile[si]);
    }
    __syncthreads();

    // ---- peak test -> key.  Size / offset validity needs four gathers per candidate from global memory; the
    // common case leaves that to the per-image kernel so that this kernel's only wait on memory is the tile load.
    for (int wi = threadIdx.x; wi < todo; wi += kCnThreads) {
        const int si = work[wi];
        const int row = si / kCnRowStride, col = si - row * kCnRowStride - 4;
        if (row < 1 || row > kCnTileH || col < 0 || col >= kCnTileW) continue;      // halo cell
        const int gy = y0 + row - 1, gx = x0 + col;
        if (gy >= H || gx >= W) continue;
        const float s = score[si];
        // include/CenterNetLayer.h:212: finite, at or above the threshold, no strictly greater neighbour
        if (!(tile[si] >= p.lo) || !isfinite(s) || s < p.d.threshold) continue;
        const float* c = score + si;
        if (c[-kCnRowStride - 1] > s || c[-kCnRowStride] > s || c[-kCnRowStride + 1] > s || c[-1] > s || c[1] > s ||
            c[kCnRowStride - 1] > s || c[kCnRowStride] > s || c[kCnRowStride + 1] > s) continue;
        const int slot = atomicAdd(&n_keys, 1);
        keys[slot] = cn_key(s, (uint32_t)((long long)cls * area + (long long)gy * W + gx));
    }
    __syncthreads();

    int n = n_keys;
    const long long slot_id = (long long)b * p.slots + (long long)cls * (p.tiles_x * p.tiles_y) + blockIdx.x;
    unsigned long long* out = p.cand + slot_id * p.slot_cap;
    if (n <= p.slot_cap) {
        for (int i = threadIdx.x; i < n; i += kCnThreads) out[i] = keys[i];
        if (threadIdx.x == 0) p.cand_cnt[slot_id] = n;
        return;
    }
    // Rare: more candidates than the tile's slot holds (slot_cap >= K).  No image keeps more than K, so the
    // tile's K best are enough -- but only valid candidates may compete for those places, so validity is
    // checked here first.
    const float* size = p.d.size + (long long)b * p.sbs;
    const float* off = p.d.offset + (long long)b * p.obs;
    for (int i = threadIdx.x; i < n; i += kCnThreads) {
        const uint32_t flat = 0xffffffffu - (uint32_t)(keys[i] & 0xffffffffu);
        if (!cn_valid(size, off, (long long)flat - (long long)cls * area, area, W, H)) keys[i] = 0ULL;   // sorts last
    }
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kCnThreads)
        if (keys[i] != 0ULL) atomicAdd(&base, 1);
    __syncthreads();
    const int n_valid = base;
    if (n_valid <= p.K) {
        for (int i = threadIdx.x; i < n; i += kCnThreads)
            if (keys[i] != 0ULL) out[atomicAdd(&n_out, 1)] = keys[i];
        if (threadIdx.x == 0) p.cand_cnt[slot_id] = n_valid;
        return;
    }
    const unsigned long long kth = block_select_kth([&](int i) { return keys[i]; }, n, p.K, hist, sel);
    for (int i = threadIdx.x; i < n; i += kCnThreads)
        if (keys[i] >= kth) out[atomicAdd(&n_out, 1)] = keys[i];
    if (threadIdx.x == 0) p.cand_cnt[slot_id] = p.K;
}

// One block per image: the K best of the image's candidates, sorted, decoded to boxes.
//  1. prefix sums of the slots' counts, so that candidate i of the image is found by a binary search;
//  2. every candidate's size / offset validity (include/CenterNetLayer.h:217-225), all gathers in
//     flight at once; valid keys are compacted into one list (shared memory when it fits);
//  3. a list that fits shared memory is sorted outright (bitonic: no contention, unlike a radix
//     histogram of scores that share their leading bits); a longer one goes through radix
//     selection of the K-th key first.
constexpr int kCnTopkThreads = 1024;
constexpr int kCnStageKeys = 4096;     // candidates per image sorted in shared memory (32 KB)
constexpr int kCnMaxSlots = 2048;      // slots per image whose prefix sums fit shared memory
constexpr int kCnBinShift = 51;        // a key's leading 13 bits (sign, exponent, 4 mantissa bits of the score) ...
constexpr int kCnBins = 1 << 13;       // ... index a histogram that aliases the staging area
static_assert(kCnBins * sizeof(int) <= kCnStageKeys * sizeof(unsigned long long), "histogram must fit the staging area");
static_assert(kCnBins == 8 * kCnTopkThreads, "the top-down scan gives every thread 8 bins");

__global__ void __launch_bounds__(kCnTopkThreads)
centernet_topk_kernel(const CnParams p)
{
    __shared__ unsigned long long stage[kCnStageKeys];
    __shared__ int prefix[kCnMaxSlots + 1];
    __shared__ int hist[256];
    __shared__ unsigned long long sel[2];
    __shared__ int warp_tot[32];
    __shared__ int n_best, n_valid;
    const int b = blockIdx.x;
    const int H = p.d.height, W = p.d.width;
    const long long area = (long long)H * W;
    const float* size = p.d.size + (long long)b * p.sbs;
    const float* off = p.d.offset + (long long)b * p.obs;
    const unsigned long long* cand = p.cand + (long long)b * p.slots * p.slot_cap;
    const int* cnt = p.cand_cnt + (long long)b * p.slots;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { n_valid = 0; n_best = 0; prefix[0] = 0; }

    // 1. inclusive prefix of slot counts -> prefix[s+1]
    int carry = 0;
    for (int base = 0; base < p.slots; base += kCnTopkThreads) {
        const int sidx = base + threadIdx.x;
        const int v = sidx < p.slots ? cnt[sidx] : 0;
        int inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        int before = carry;
        for (int i = 0; i < warp; ++i) before += warp_tot[i];
        if (sidx < p.slots) prefix[sidx + 1] = before + inc;
        int total = 0;
        for (int i = 0; i < 32; ++i) total += warp_tot[i];
        carry += total;
        __syncthreads();
    }
    const int n_total = carry;

    // 2. Short cut.  Far more cells pass the peak test than an image keeps (thousands against K), and the
    // size / offset validity check costs four scattered reads per candidate.  So first find, from a histogram
    // of the keys' leading 13 bits, the bin holding the K-th best candidate; only candidates in that bin or
    // above (at least K, usually a few hundred) are staged and checked.  If K or more of them are valid, the K
    // best valid candidates of the image are among them, because every candidate left out has a smaller key.
    // Otherwise (many invalid boxes, or one bin holding thousands of equal scores) the full path below runs.
    unsigned long long* sorted = stage;
    int m = 0;
    bool done = false;
    {
        int* bins = reinterpret_cast<int*>(stage);                 // kCnBins ints alias the staging area
        for (int i = threadIdx.x; i < kCnBins; i += kCnTopkThreads) bins[i] = 0;
        __syncthreads();
        for (int s0 = 0; s0 < p.slots; s0 += 32) {
            const int sidx = s0 + warp;
            if (sidx >= p.slots) continue;
            const int c = prefix[sidx + 1] - prefix[sidx];
            const unsigned long long* src = cand + (long long)sidx * p.slot_cap;
#pragma unroll 8
            for (int j = lane; j < c; j += 32) atomicAdd(&bins[(int)(src[j] >> kCnBinShift)], 1);
        }
        __syncthreads();
        // thread t owns the 8 bins below kCnBins - 8t, scanned from the top
        const int top = kCnBins - 1 - 8 * (int)threadIdx.x;
        int mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mine += bins[top - j];
        int inc = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) warp_tot[warp] = inc;
        if (threadIdx.x == 0) sel[0] = 0ULL;                       // lead bin 0 = "take everything"
        __syncthreads();
        int before = inc - mine;
        for (int i = 0; i < warp; ++i) before += warp_tot[i];
        if (before < p.K && before + mine >= p.K) {
            int acc = before, bin = top;
            for (int j = 0; j < 8; ++j) {
                if (acc + bins[top - j] >= p.K) { bin = top - j; break; }
                acc += bins[top - j];
            }
            sel[0] = (unsigned long long)bin;
        }
        __syncthreads();
        const int lead = (int)sel[0];
        __syncthreads();                                           // bins are dead from here: stage is reused
        for (int s0 = 0; s0 < p.slots; s0 += 32) {
            const int sidx = s0 + warp;
            if (sidx >= p.slots) continue;
            const int c = prefix[sidx + 1] - prefix[sidx];
            const unsigned long long* src = cand + (long long)sidx * p.slot_cap;
#pragma unroll 8
            for (int j = lane; j < c; j += 32) {
                const unsigned long long key = src[j];
                if ((int)(key >> kCnBinShift) >= lead) {
                    const int at = atomicAdd(&n_best, 1);
                    if (at < kCnStageKeys) stage[at] = key;
                }
            }
        }
        __syncthreads();
        const int n_c = n_best;
        if (n_c <= kCnStageKeys) {
            for (int i = threadIdx.x; i < n_c; i += kCnTopkThreads) {
                const uint32_t flat = 0xffffffffu - (uint32_t)(stage[i] & 0xffffffffu);
                const uint32_t cls = flat / (uint32_t)area;
                if (cn_valid(size, off, (long long)(flat - cls * (uint32_t)area), area, W, H)) atomicAdd(&n_valid, 1);
                else stage[i] = 0ULL;                              // sorts behind every real key
            }
            __syncthreads();
            if (n_valid >= p.K || n_c == n_total) {
                int pow2 = 1;
                while (pow2 < n_c) pow2 <<= 1;
                for (int i = n_c + threadIdx.x; i < pow2; i += kCnTopkThreads) stage[i] = 0ULL;
                __syncthreads();
                block_bitonic_desc(stage, pow2);
                m = n_valid < p.K ? n_valid : p.K;
                done = true;
            }
        }
        __syncthreads();
    }

    if (!done) {
        if (threadIdx.x == 0) { n_valid = 0; n_best = 0; }
        __syncthreads();
        // 2. validity + compaction
        const bool staged = n_total <= kCnStageKeys;
        unsigned long long* list = staged ? stage : p.list + (long long)b * p.slots * p.slot_cap;
        for (int i = threadIdx.x; i < n_total; i += kCnTopkThreads) {
            int lo = 0, hi = p.slots;                    // largest s with prefix[s] <= i
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (prefix[mid] <= i) lo = mid; else hi = mid;
            }
            const unsigned long long key = cand[(long long)lo * p.slot_cap + (i - prefix[lo])];
            const uint32_t flat = 0xffffffffu - (uint32_t)(key & 0xffffffffu);
            const uint32_t cls = flat / (uint32_t)area;
            if (cn_valid(size, off, (long long)(flat - cls * (uint32_t)area), area, W, H)) list[atomicAdd(&n_valid, 1)] = key;
        }
        __syncthreads();
        const int n = n_valid;

        // 3. order the best K
        if (staged) {
            int pow2 = 1;
            while (pow2 < n) pow2 <<= 1;
            for (int i = n + threadIdx.x; i < pow2; i += kCnTopkThreads) stage[i] = 0ULL;
            __syncthreads();
            block_bitonic_desc(stage, pow2);
            m = n < p.K ? n : p.K;
        } else {
            // The list is in global memory.  Two radix passes fix the leading 16 bits of the K-th key; keys above
            // them are certain winners, keys sharing them are the only ones still undecided.  With scores spread
            // over the second byte that is a few hundred keys, which are sorted in shared memory.  If the
            // undecided set does not fit (e.g. a constant heatmap), the full 8-pass selection decides.
            int m_sort = 0;
            if (n > p.K) {
                int want = 0;
                const unsigned long long lead = block_select_kth([&](int i) { return list[i]; }, n, p.K, hist, sel, 2, &want) >> 48;
                const int winners = p.K - want;
                if (threadIdx.x == 0) { n_best = 0; n_valid = 0; }      // n_valid is reused as the tie counter
                __syncthreads();
                for (int i = threadIdx.x; i < n; i += kCnTopkThreads) {
                    const unsigned long long key = list[i];
                    const unsigned long long top = key >> 48;
                    if (top > lead) stage[atomicAdd(&n_best, 1)] = key;
                    else if (top == lead) {
                        const int at = atomicAdd(&n_valid, 1);
                        if (winners + at < kCnStageKeys) stage[winners + at] = key;
                    }
                }
                __syncthreads();
                if (winners + n_valid <= kCnStageKeys) {
                    m_sort = winners + n_valid;
                } else {
                    const unsigned long long kth = block_select_kth([&](int i) { return list[i]; }, n, p.K, hist, sel);
                    if (threadIdx.x == 0) n_best = 0;
                    __syncthreads();
                    for (int i = threadIdx.x; i < n; i += kCnTopkThreads) {
                        const unsigned long long key = list[i];
                        if (key >= kth) stage[atomicAdd(&n_best, 1)] = key;
                    }
                    __syncthreads();
                    m_sort = n_best;
                }
            } else {
                for (int i = threadIdx.x; i < n; i += kCnTopkThreads) stage[i] = list[i];
                m_sort = n;
            }
            __syncthreads();
            int pow2 = 1;
            while (pow2 < m_sort) pow2 <<= 1;
            for (int i = m_sort + threadIdx.x; i < pow2; i += kCnTopkThreads) stage[i] = 0ULL;
            __syncthreads();
            block_bitonic_desc(stage, pow2);
            m = m_sort < p.K ? m_sort : p.K;
        }
    }
    const float image_w = p.d.image_width > 0 ? (float)p.d.image_width : 1.0f;
    const float image_h = p.d.image_height > 0 ? (float)p.d.image_height : 1.0f;
    for (int i = threadIdx.x; i < m; i += blockDim.x) {
        const unsigned long long key = sorted[i];
        const uint32_t flat = 0xffffffffu - (uint32_t)(key & 0xffffffffu);
        const float score = order_float((uint32_t)(key >> 32));
        const int cls = (int)(flat / area);
        const long long idx = flat - (long long)cls * area;
        const int y = (int)(idx / W), x = (int)(idx - (long long)y * W);
        // include/CenterNetLayer.h:217-237, each product and sum rounded separately as on the host
        const float bw = size[idx] / W, bh = size[area + idx] / H;
        const float cx = (x + off[idx]) / W, cy = (y + off[area + idx]) / H;
        store_detection(p.dets + (long long)b * p.K + i, __fmul_rn(__fsub_rn(cx, bw / 2.0f), image_w),
                        __fmul_rn(__fsub_rn(cy, bh / 2.0f), image_h), __fmul_rn(bw, image_w), __fmul_rn(bh, image_h),
                        score, cls, b + p.d.batch_id_offset, (int)flat);
    }
    if (threadIdx.x == 0) p.counts[b] = m;
}

// ============================================================================================
// Softmax / Region
// ============================================================================================
// One block per row of n contiguous values: out = exp(x/temp - max/temp) / sum (src/Math.cpp:77-97).
__global__ void __launch_bounds__(128)
softmax_rows_kernel(const float* in, float* out, int n, float temp)
{
    __shared__ float red[4];
    __shared__ float bcast;
    const float* x = in + (long long)blockIdx.x * n;
    float* y = out + (long long)blockIdx.x * n;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < n; i += 128) m = x[i] > m ? x[i] : m;
    for (int o = 16; o > 0; o >>= 1) { float t = __shfl_xor_sync(0xffffffffu, m, o); m = t > m ? t : m; }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) { float t = red[0]; for (int w = 1; w < 4; ++w) t = red[w] > t ? red[w] : t; bcast = t; }
    __syncthreads();
    const float largest = bcast;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < n; i += 128) {
        const float e = expf(x[i] / temp - largest / temp);
        y[i] = e;
        sum += e;
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) bcast = red[0] + red[1] + red[2] + red[3];
    __syncthreads();
    const float total = bcast;
    for (int i = threadIdx.x; i < n; i += 128) y[i] = y[i] / total;
}

struct RegionParams {
    const float* in; float* out;
    int batch, HW, num, size, coords, classes, softmax;
};

// One thread per predicted box (image, cell, anchor slot).
__global__ void __launch_bounds__(128)
region_forward_kernel(const RegionParams p)
{
    const long long boxes = (long long)p.batch * p.HW * p.num;
    for (long long t = (long long)blockIdx.x * 128 + threadIdx.x; t < boxes; t += (long long)gridDim.x * 128) {
        // thread order: cells fastest so the strided NCHW reads coalesce
        const int cell = (int)(t % p.HW);
        const long long r = t / p.HW;
        const int n = (int)(r % p.num);
        const int b = (int)(r / p.num);
        const long long outputs = (long long)p.HW * p.num * p.size;
        const float* src = p.in + b * outputs + (long long)n * p.size * p.HW + cell;
        float* dst = p.out + b * outputs + ((long long)cell * p.num + n) * p.size;
        for (int e = 0; e < p.size; ++e) {
            float v = src[(long long)e * p.HW];
            if (e == 4) v = act_logistic(v);
            dst[e] = v;
        }
        if (p.softmax) {
            float* cls = dst + p.coords + 1;
            float largest = -FLT_MAX, sum = 0.0f;
            for (int j = 0; j < p.classes; ++j) largest = cls[j] > largest ? cls[j] : largest;
            for (int j = 0; j < p.classes; ++j) { const float e = expf(cls[j] - largest); sum += e; cls[j] = e; }
            for (int j = 0; j < p.classes; ++j) cls[j] = cls[j] / sum;
        }
    }
}

// ============================================================================================
// YOLOv1 detection head (include/DetectLayer.h:166-209)
// ============================================================================================
// One image's predictions are [side*side*classes class scores][side*side*num object scales]
// [side*side*num*coords boxes].  A box is emitted when its scale is finite and positive and
// scale * (its cell's best class score) reaches the threshold; order: image, cell, box.
// The head is a few thousand values, so one block walks all boxes in order with a running count.
struct DetectParams {
    const float* pred; long long pbs;
    int batch, side, num, classes, coords, squared;
    float width, height, threshold;
    pxe_detection* dets; long long capacity; long long* count;
    int batch_id_offset;
};

__global__ void __launch_bounds__(1024)
detect_decode_kernel(const DetectParams p)
{
    __shared__ int warp_tot[32];
    __shared__ long long carry;
    if (threadIdx.x == 0) carry = *p.count;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int locations = p.side * p.side;
    const int per_image = locations * p.num;
    const long long total = (long long)p.batch * per_image;
    for (long long base = 0; base < total; base += 1024) {
        const long long t = base + threadIdx.x;
        int flag = 0, best = 0;
        float best_prob = 0.0f, bx = 0, by = 0, bw = 0, bh = 0;
        int b = 0, slot = 0;
        if (t < total) {
            b = (int)(t / per_image);
            slot = (int)(t - (long long)b * per_image);          // i * num + n
            const int i = slot / p.num;
            const int row = i / p.side, col = i - row * p.side;
            const float* pred = p.pred + (long long)b * p.pbs;
            const float scale = pred[locations * p.classes + slot];
            if (isfinite(scale) && scale > 0.0f) {
                const float* box = pred + (long long)locations * (p.classes + p.num) + (long long)slot * p.coords;
                const float x = __fmul_rn((box[0] + col) / p.side, p.width);
                const float y = __fmul_rn((box[1] + row) / p.side, p.height);
                // the host squares with std::pow(v, 2), glibc's powf: within one ulp of v*v, equal to it for
                // all but ~0.06 % of inputs; one multiplication here
                const float w = __fmul_rn(p.squared ? __fmul_rn(box[2], box[2]) : box[2], p.width);
                const float h = __fmul_rn(p.squared ? __fmul_rn(box[3], box[3]) : box[3], p.height);
                best_prob = -FLT_MAX;
                for (int j = 0; j < p.classes; ++j) {
                    const float pr = __fmul_rn(scale, pred[i * p.classes + j]);
                    if (pr > best_prob) { best = j; best_prob = pr; }
                }
                if (best_prob >= p.threshold) {
                    flag = 1;
                    bx = w > 0.0f ? __fsub_rn(x, w / 2.0f) : x;      // DarkBox::rect, src/DarkBox.cpp:84-123
                    by = h > 0.0f ? __fsub_rn(y, h / 2.0f) : y;
                    bw = w; bh = h;
                }
            }
        }
        int inc = flag;
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += v;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        long long before = carry;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (flag) {
            const long long pos = before + inc - 1;
            if (pos < p.capacity) store_detection(p.dets + pos, bx, by, bw, bh, best_prob, best, b + p.batch_id_offset, slot);
        }
        __syncthreads();
        if (threadIdx.x == 1023) carry = before + inc;
        __syncthreads();
    }
    if (threadIdx.x == 0) *p.count = carry;
}

// ============================================================================================
// Region (YOLOv2) head decode (include/RegionLayer.h:355-395, lightBox src/DarkBox.cpp:191-202)
// ============================================================================================
// pred is the output of pxe_region_forward: [image][cell*num + n][coords + 1 + classes].  Every class of a
// box whose scale * class probability reaches the threshold is one record; order: image, cell, box, class.
// One block walks the boxes in order with a running count (a head is 13x13x5 boxes per image).
constexpr int kRegionMaxBoxes = 32;      // boxes per cell

struct RegionDecodeParams {
    const float* pred;
    int batch, W, H, num, coords, classes, per_image;
    float biases[2 * kRegionMaxBoxes];
    float img_w, img_h, threshold;
    pxe_detection* dets; long long capacity; long long* count;
    int batch_id_offset;
};

__global__ void __launch_bounds__(1024)
region_decode_kernel(const RegionDecodeParams p)
{
    __shared__ int warp_tot[32];
    __shared__ long long carry;
    if (threadIdx.x == 0) carry = *p.count;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int size = p.coords + 1 + p.classes;
    const int per_image = p.W * p.H * p.num;
    const long long total = (long long)p.batch * per_image;
    for (long long base = 0; base < total; base += 1024) {
        const long long t = base + threadIdx.x;
        int cnt = 0, b = 0, index = 0;
        const float* box = nullptr;
        float scale = 0.0f;
        if (t < total) {
            b = (int)(t / per_image);
            index = (int)(t - (long long)b * per_image);
            // RegionLayer.h:363-369 indexes the predictions without the image's offset: every image decodes
            // image 0's boxes.  per_image = 0 keeps that; 1 gives every image its own.
            box = p.pred + ((long long)(p.per_image ? b : 0) * per_image + index) * size;
            scale = box[p.coords];
            for (int j = 0; j < p.classes; ++j)
                if (__fmul_rn(scale, box[p.coords + 1 + j]) >= p.threshold) ++cnt;
        }
        int inc = cnt;
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += v;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        long long before = carry;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (cnt) {
            long long pos = before + inc - cnt;
            const int i = index / p.num, n = index - i * p.num;
            const int row = i / p.W, col = i - row * p.W;
            const float x = (col + 1.0f / (1.0f + expf(-box[0]))) / p.W;
            const float y = (row + 1.0f / (1.0f + expf(-box[1]))) / p.H;
            const float bw = expf(box[2]) * p.biases[2 * n] / p.W;
            const float bh = expf(box[3]) * p.biases[2 * n + 1] / p.H;
            const float x1 = __fmul_rn(x, p.img_w), y1 = __fmul_rn(y, p.img_h);
            const float ww = __fmul_rn(bw, p.img_w), hh = __fmul_rn(bh, p.img_h);
            for (int j = 0; j < p.classes; ++j) {
                const float pr = __fmul_rn(scale, box[p.coords + 1 + j]);
                if (pr >= p.threshold) {
                    if (pos < p.capacity)
                        store_detection(p.dets + pos, __fsub_rn(x1, ww / 2.0f), __fsub_rn(y1, hh / 2.0f), ww, hh, pr, j,
                                        b + p.batch_id_offset, index);
                    ++pos;
                }
            }
        }
        __syncthreads();
        if (threadIdx.x == 1023) carry = before + inc;
        __syncthreads();
    }
    if (threadIdx.x == 0) *p.count = carry;
}

// Softmax (classifier) head: SoftmaxLayer::addDetects, include/SoftmaxLayer.h:182-196.  One record per image
// whose largest probability (first maximum, std::max_element) reaches the threshold: the whole frame as the
// box, the class and its probability.  One warp per image, 32 images per pass, images in order.
__global__ void __launch_bounds__(1024)
softmax_decode_kernel(const float* probs, long long pbs, int batch, int classes, float width, float height,
                      float threshold, pxe_detection* dets, long long capacity, long long* count, int batch_id_offset)
{
    __shared__ int flags[32];
    __shared__ long long carry;
    if (threadIdx.x == 0) carry = *count;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < batch; base += 32) {
        const int b = base + warp;
        // std::max_element: the earliest of the largest values; a NaN never replaces the running maximum, and
        // a NaN in front (element 0) is never replaced.  So: the lowest index among the largest non-NaN values,
        // and no detection at all when element 0 is NaN.
        float best = -INFINITY;
        int arg = 0x7fffffff;
        bool first_is_nan = false;
        if (b < batch) {
            const float* p = probs + (long long)b * pbs;
            first_is_nan = !(p[0] == p[0]);
            for (int j = lane; j < classes; j += 32) {
                const float v = p[j];
                if (v > best || (v == best && j < arg)) { best = v; arg = j; }
            }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ov > best || (ov == best && oa < arg)) { best = ov; arg = oa; }
        }
        if (first_is_nan) best = __int_as_float(0x7fc00000);      // NaN >= threshold is false
        const int flag = (b < batch && best >= threshold) ? 1 : 0;
        if (lane == 0) flags[warp] = flag;
        __syncthreads();
        long long pos = carry;
        int total = 0;
        for (int w = 0; w < 32; ++w) {
            if (w < warp) pos += flags[w];
            total += flags[w];
        }
        if (flag && lane == 0 && pos < capacity)
            store_detection(dets + pos, 0.0f, 0.0f, width, height, best, arg, b + batch_id_offset, 0);
        __syncthreads();
        if (threadIdx.x == 0) carry += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) *count = carry;
}

}  // namespace
}  // namespace pxe

using namespace pxe;

// -------------------------------------------------------------------------------------- YOLO API
extern "C" int pxe_yolo_activate(pxe_stream_t stream, const float* in, float* out, int batch, int masks,
                                 int classes, int area)
{
    PXE_REQUIRE(in && out, "yolo_activate: null pointer");
    PXE_REQUIRE(batch > 0 && masks > 0 && classes >= 0 && area > 0, "yolo_activate: non-positive shape");
    pxe_epilogue_desc d{};
    d.x = in; d.y = out;
    d.batch = batch; d.channels = masks * (classes + 5); d.height = 1; d.width = area;
    d.act = PXE_ACT_YOLO_HEAD; d.yolo_classes = classes;
    return pxe_conv_epilogue(stream, &d);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

extern "C" size_t pxe_yolo_decode_workspace_bytes(int batch, int height, int width)
{
    if (batch <= 0 || height <= 0 || width <= 0) return 0;
    const size_t hw = (size_t)height * width;
    const size_t bpi = (hw + kYoloCells - 1) / kYoloCells;
    return align_up((size_t)batch * bpi * sizeof(int), 256) + align_up((size_t)batch * bpi * sizeof(long long), 256);
}

extern "C" int pxe_yolo_decode(pxe_stream_t stream, const pxe_yolo_decode_desc* dp, pxe_detection* dets,
                               long long capacity, long long* count, void* workspace, size_t workspace_bytes)
{
    PXE_REQUIRE(dp != nullptr, "yolo_decode: null descriptor");
    const pxe_yolo_decode_desc& d = *dp;
    PXE_REQUIRE(d.head && count && workspace, "yolo_decode: null pointer");
    PXE_REQUIRE(capacity >= 0 && (capacity == 0 || dets != nullptr), "yolo_decode: dets is null");
    PXE_REQUIRE(d.batch > 0 && d.height > 0 && d.width > 0 && d.classes >= 0, "yolo_decode: non-positive shape");
    PXE_REQUIRE(d.n_masks > 0 && d.n_masks <= 16, "yolo_decode: n_masks %d outside 1..16", d.n_masks);
    PXE_REQUIRE(d.n_anchor_values > 0 && d.n_anchor_values <= 64 && d.n_anchor_values % 2 == 0,
                "yolo_decode: n_anchor_values %d invalid", d.n_anchor_values);
    for (int n = 0; n < d.n_masks; ++n)
        PXE_REQUIRE(d.mask[n] >= 0 && 2 * d.mask[n] + 1 < d.n_anchor_values, "yolo_decode: mask[%d]=%d has no anchor", n, d.mask[n]);
    PXE_REQUIRE(d.net_width > 0 && d.net_height > 0, "yolo_decode: network size must be positive");
    PXE_REQUIRE((d.image_width > 0) == (d.image_height > 0), "yolo_decode: image_width and image_height must both be set or both be 0");
    PXE_REQUIRE(d.batch <= 65535, "yolo_decode: batch %d exceeds 65535 per call", d.batch);
    PXE_REQUIRE(aligned16(dets), "yolo_decode: dets must be 16-byte aligned");
    const size_t need = pxe_yolo_decode_workspace_bytes(d.batch, d.height, d.width);
    if (workspace_bytes < need)
        return set_error(PXE_ERR_WORKSPACE, "yolo_decode: workspace %zu bytes, need %zu", workspace_bytes, need);
    PXE_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "yolo_decode: workspace must be 256-byte aligned");

    YoloParams p{};
    p.d = d;
    p.HW = d.height * d.width;
    p.entries = d.classes + 5;
    const long long chw = (long long)d.n_masks * p.entries * p.HW;
    PXE_REQUIRE(d.head_batch_stride == 0 || d.head_batch_stride >= chw, "yolo_decode: head_batch_stride too small");
    p.hbs = d.head_batch_stride ? d.head_batch_stride : chw;
    p.blocks_per_image = (p.HW + kYoloCells - 1) / kYoloCells;
    // class chunks of kYoloChunk classes, as many as fit 32 warps per block; with more classes than that
    // the chunks grow beyond the register window (handled in the kernels)
    p.chunks = d.classes > 0 ? (d.classes + kYoloChunk - 1) / kYoloChunk : 1;
    if (p.chunks > kYoloMaxWarps / d.n_masks) p.chunks = kYoloMaxWarps / d.n_masks;
    p.chunk_len = d.classes > 0 ? (d.classes + p.chunks - 1) / p.chunks : 1;
    p.warps = d.n_masks * p.chunks;
    p.dets = dets; p.capacity = capacity; p.count = count;
    char* ws = static_cast<char*>(workspace);
    p.block_sums = reinterpret_cast<int*>(ws);
    ws += align_up((size_t)d.batch * p.blocks_per_image * sizeof(int), 256);
    p.block_offsets = reinterpret_cast<long long*>(ws);

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)p.blocks_per_image, (unsigned)d.batch);
    const unsigned threads = (unsigned)(kYoloCells * p.warps);
    yolo_count_kernel<<<grid, threads, 0, s>>>(p);
    PXE_LAUNCH_OK("yolo_count_kernel");
    yolo_scan_kernel<<<1, 1024, 0, s>>>(p.block_sums, p.block_offsets, d.batch * p.blocks_per_image, count);
    PXE_LAUNCH_OK("yolo_scan_kernel");
    yolo_emit_kernel<<<grid, threads, 0, s>>>(p);
    PXE_LAUNCH_OK("yolo_emit_kernel");
    return PXE_OK;
}

// ------------------------------------------------------------- YOLO decode without a caller workspace
// The scratch of pxe_yolo_decode (per-block sums and offsets) held in the library's
// own device image instead of a buffer the caller allocates.  Every GPU that loads the library
// carries these bytes until the process exits, so the size is kept modest.
static __device__ __align__(256) unsigned char g_yolo_static_scratch[PXE_YOLO_DECODE_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[64];      // device address of the array, per device ordinal
}  // namespace

extern "C" int pxe_yolo_decode_static(pxe_stream_t stream, const pxe_yolo_decode_desc* dp, pxe_detection* dets,
                                      long long capacity, long long* count)
{
    PXE_REQUIRE(dp != nullptr, "yolo_decode_static: null descriptor");
    PXE_REQUIRE(dp->batch > 0 && dp->height > 0 && dp->width > 0, "yolo_decode_static: non-positive shape");
    const size_t need = pxe_yolo_decode_workspace_bytes(dp->batch, dp->height, dp->width);
    if (need > (size_t)PXE_YOLO_DECODE_STATIC_SCRATCH_BYTES)
        return set_error(PXE_ERR_WORKSPACE,
                         "yolo_decode_static: a %d x %d x %d head needs %zu bytes of scratch, the built-in array holds %zu; "
                         "use pxe_yolo_decode with a workspace of your own",
                         dp->batch, dp->height, dp->width, need, (size_t)PXE_YOLO_DECODE_STATIC_SCRATCH_BYTES);
    int dev = 0;
    PXE_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(PXE_ERR_UNSUPPORTED, "yolo_decode_static: device ordinal %d out of range", dev);
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (g_static_scratch_ptr[dev] == nullptr) {
            // In host code the array's name is only a handle; kernels need its address on the current device.
            void* p = nullptr;
            PXE_CUDA_OK(cudaGetSymbolAddress(&p, g_yolo_static_scratch));
            g_static_scratch_ptr[dev] = p;
        }
        scratch = g_static_scratch_ptr[dev];
    }
    return pxe_yolo_decode(stream, dp, dets, capacity, count, scratch, (size_t)PXE_YOLO_DECODE_STATIC_SCRATCH_BYTES);
}

// --------------------------------------------------------------------------------- CenterNet API
extern "C" int pxe_centernet_activate(pxe_stream_t stream, const float* in, float* out, int batch, int classes,
                                      int area, float heatmap_bias)
{
    PXE_REQUIRE(in && out, "centernet_activate: null pointer");
    PXE_REQUIRE(batch > 0 && classes > 0 && area > 0, "centernet_activate: non-positive shape");
    const long long outputs = (long long)(classes + 4) * area, heat = (long long)classes * area;
    const long long total = outputs * batch;
    PXE_REQUIRE(total < (1LL << 32), "centernet_activate: too many elements for one launch");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    CnActParams p{};
    p.in = in; p.out = out; p.bias = heatmap_bias;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (area % 4 == 0 && aligned16(in) && aligned16(out)) {
        p.total = (uint32_t)(total / 4); p.outputs = (uint32_t)(outputs / 4); p.heat = (uint32_t)(heat / 4);
        p.div_outputs = FastDiv(p.outputs);
        centernet_activate_kernel<true><<<grid_for(p.total, 256, di.sm_count, 16), 256, 0, s>>>(p);
    } else {
        p.total = (uint32_t)total; p.outputs = (uint32_t)outputs; p.heat = (uint32_t)heat;
        p.div_outputs = FastDiv(p.outputs);
        centernet_activate_kernel<false><<<grid_for(p.total, 256, di.sm_count, 16), 256, 0, s>>>(p);
    }
    PXE_LAUNCH_OK("centernet_activate_kernel");
    return PXE_OK;
}

static void cn_geometry(int classes, int height, int width, int* tiles_x, int* tiles_y, long long* blocks_per_image)
{
    *tiles_x = (width + kCnTileW - 1) / kCnTileW;
    *tiles_y = (height + kCnTileH - 1) / kCnTileH;
    *blocks_per_image = (long long)classes * *tiles_x * *tiles_y;
}

extern "C" size_t pxe_centernet_decode_workspace_bytes(int batch, int classes, int height, int width,
                                                       int max_detections)
{
    if (batch <= 0 || classes <= 0 || height <= 0 || width <= 0 || max_detections <= 0) return 0;
    int tx, ty;
    long long bpi;
    cn_geometry(classes, height, width, &tx, &ty, &bpi);
    const size_t slot_cap = max_detections > kCnSlotCap ? max_detections : kCnSlotCap;
    return 2 * align_up((size_t)batch * bpi * slot_cap * sizeof(unsigned long long), 256)
           + align_up((size_t)batch * bpi * sizeof(int), 256);
}

// Pre-activation value below which sigmoid(v) < threshold for certain (with a margin far wider
// than any rounding in exp()).
static float centernet_prefilter(const pxe_centernet_decode_desc& d)
{
    if (!d.heat_is_logit) return d.threshold;                 // "(v >= thr) false" is exactly "v < thr or NaN"
    if (!(d.threshold > 0.0f)) return -INFINITY;
    if (d.threshold >= 1.0f) return 15.0f;                    // sigmoid(v) rounds to 1 only for v > 16.6
    const double t = (double)d.threshold;
    const double logit = log(t / (1.0 - t));
    return (float)(logit - 1e-3 - 1e-3 * fabs(logit));
}

extern "C" int pxe_centernet_decode(pxe_stream_t stream, const pxe_centernet_decode_desc* dp,
                                    pxe_detection* dets, int* counts, void* workspace, size_t workspace_bytes)
{
    PXE_REQUIRE(dp != nullptr, "centernet_decode: null descriptor");
    const pxe_centernet_decode_desc& d = *dp;
    PXE_REQUIRE(d.heat && d.size && d.offset && dets && counts && workspace, "centernet_decode: null pointer");
    PXE_REQUIRE(d.batch > 0 && d.classes > 0 && d.height > 0 && d.width > 0, "centernet_decode: non-positive shape");
    PXE_REQUIRE(d.max_detections > 0 && d.max_detections <= kCnMaxK, "centernet_decode: max_detections %d outside 1..%d",
                d.max_detections, kCnMaxK);
    const long long area = (long long)d.height * d.width;
    PXE_REQUIRE(area * d.classes < 0xffffffffLL, "centernet_decode: heatmap has too many cells per image");
    PXE_REQUIRE(d.batch <= 65535 && d.classes <= 65535, "centernet_decode: batch/classes exceed 65535");
    PXE_REQUIRE(d.heat_batch_stride == 0 || d.heat_batch_stride >= area * d.classes, "centernet_decode: heat_batch_stride too small");
    PXE_REQUIRE(d.size_batch_stride == 0 || d.size_batch_stride >= 2 * area, "centernet_decode: size_batch_stride too small");
    PXE_REQUIRE(d.offset_batch_stride == 0 || d.offset_batch_stride >= 2 * area, "centernet_decode: offset_batch_stride too small");
    PXE_REQUIRE(aligned16(dets), "centernet_decode: dets must be 16-byte aligned");
    const size_t need = pxe_centernet_decode_workspace_bytes(d.batch, d.classes, d.height, d.width, d.max_detections);
    if (workspace_bytes < need)
        return set_error(PXE_ERR_WORKSPACE, "centernet_decode: workspace %zu bytes, need %zu", workspace_bytes, need);
    PXE_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "centernet_decode: workspace must be 256-byte aligned");

    CnParams p{};
    p.d = d;
    p.hbs = d.heat_batch_stride ? d.heat_batch_stride : area * d.classes;
    p.sbs = d.size_batch_stride ? d.size_batch_stride : 2 * area;
    p.obs = d.offset_batch_stride ? d.offset_batch_stride : 2 * area;
    long long bpi;
    cn_geometry(d.classes, d.height, d.width, &p.tiles_x, &p.tiles_y, &bpi);
    PXE_REQUIRE(bpi * (d.max_detections > kCnSlotCap ? d.max_detections : kCnSlotCap) < 0x7fffffffLL,
                "centernet_decode: candidate table too large");
    if (bpi > kCnMaxSlots)
        return set_error(PXE_ERR_UNSUPPORTED, "centernet_decode: %lld tiles x classes per image exceed %d", bpi, kCnMaxSlots);
    p.K = d.max_detections;
    p.slots = (int)bpi;
    p.slot_cap = d.max_detections > kCnSlotCap ? d.max_detections : kCnSlotCap;
    p.lo = centernet_prefilter(d);
    p.lo_list = d.heat_is_logit ? p.lo - 2e-4f * fmaxf(1.0f, fabsf(p.lo)) : p.lo;
    char* ws = static_cast<char*>(workspace);
    p.cand = reinterpret_cast<unsigned long long*>(ws);
    ws += align_up((size_t)d.batch * bpi * p.slot_cap * sizeof(unsigned long long), 256);
    p.list = reinterpret_cast<unsigned long long*>(ws);
    ws += align_up((size_t)d.batch * bpi * p.slot_cap * sizeof(unsigned long long), 256);
    p.cand_cnt = reinterpret_cast<int*>(ws);
    p.dets = dets; p.counts = counts;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)(p.tiles_x * p.tiles_y), (unsigned)d.classes, (unsigned)d.batch);
    // 128-bit tile loads need every row segment of a tile to start on a 16-byte boundary
    const bool vec = d.width % 4 == 0 && aligned16(d.heat) && p.hbs % 4 == 0;
    if (vec) centernet_peaks_kernel<true><<<grid, kCnThreads, 0, s>>>(p);
    else centernet_peaks_kernel<false><<<grid, kCnThreads, 0, s>>>(p);
    PXE_LAUNCH_OK("centernet_peaks_kernel");
    centernet_topk_kernel<<<(unsigned)d.batch, kCnTopkThreads, 0, s>>>(p);
    PXE_LAUNCH_OK("centernet_topk_kernel");
    return PXE_OK;
}

// ------------------------------------------------------------------------------ softmax / region
extern "C" int pxe_softmax(pxe_stream_t stream, const float* in, float* out, int batch, int inputs, int groups,
                           float temperature)
{
    PXE_REQUIRE(in && out, "softmax: null pointer");
    PXE_REQUIRE(batch > 0 && inputs > 0 && groups > 0, "softmax: non-positive shape");
    PXE_REQUIRE(inputs % groups == 0, "softmax: inputs %d not divisible by groups %d", inputs, groups);
    PXE_REQUIRE(temperature != 0.0f, "softmax: temperature is zero");
    const long long rows = (long long)batch * groups;
    PXE_REQUIRE(rows <= 0x7fffffffLL, "softmax: too many rows");
    softmax_rows_kernel<<<(unsigned)rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(in, out, inputs / groups, temperature);
    PXE_LAUNCH_OK("softmax_rows_kernel");
    return PXE_OK;
}

extern "C" int pxe_region_forward(pxe_stream_t stream, const float* in, float* out, int batch, int width,
                                  int height, int num, int coords, int classes, int softmax)
{
    PXE_REQUIRE(in && out && in != out, "region_forward: null or aliased pointers");
    PXE_REQUIRE(batch > 0 && width > 0 && height > 0 && num > 0 && coords >= 4 && classes >= 0, "region_forward: bad shape");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PXE_OK) return rc;
    RegionParams p{};
    p.in = in; p.out = out; p.batch = batch; p.HW = width * height; p.num = num;
    p.size = coords + 1 + classes; p.coords = coords; p.classes = classes; p.softmax = softmax;
    const long long boxes = (long long)batch * p.HW * num;
    region_forward_kernel<<<grid_for(boxes, 128, di.sm_count, 16), 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
    PXE_LAUNCH_OK("region_forward_kernel");
    return PXE_OK;
}

// ------------------------------------------------------------------------------- YOLOv1 detect
extern "C" int pxe_detect_decode(pxe_stream_t stream, const float* pred, long long pred_batch_stride, int batch,
                                 int side, int num, int classes, int coords, int squared, float width, float height,
                                 float threshold, pxe_detection* dets, long long capacity, long long* count,
                                 int batch_id_offset)
{
    PXE_REQUIRE(pred && dets && count, "detect_decode: null pointer");
    PXE_REQUIRE(batch > 0 && side > 0 && num > 0 && classes > 0 && coords >= 4, "detect_decode: bad shape");
    PXE_REQUIRE(capacity >= 0, "detect_decode: negative capacity");
    PXE_REQUIRE(aligned16(dets), "detect_decode: dets must be 16-byte aligned");
    const long long outputs = (long long)side * side * (classes + num * (1 + coords));
    PXE_REQUIRE(pred_batch_stride == 0 || pred_batch_stride >= outputs, "detect_decode: pred_batch_stride too small");
    DetectParams p{};
    p.pred = pred; p.pbs = pred_batch_stride ? pred_batch_stride : outputs;
    p.batch = batch; p.side = side; p.num = num; p.classes = classes; p.coords = coords; p.squared = squared;
    p.width = width; p.height = height; p.threshold = threshold;
    p.dets = dets; p.capacity = capacity; p.count = count; p.batch_id_offset = batch_id_offset;
    detect_decode_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(p);
    PXE_LAUNCH_OK("detect_decode_kernel");
    return PXE_OK;
}

// --------------------------------------------------------------------------------- Region decode
extern "C" int pxe_region_decode(pxe_stream_t stream, const float* pred, int batch, int width, int height, int num,
                                 int coords, int classes, const float* anchors, int per_image, float image_width,
                                 float image_height, float threshold, pxe_detection* dets, long long capacity,
                                 long long* count, int batch_id_offset)
{
    PXE_REQUIRE(pred && anchors && dets && count, "region_decode: null pointer");
    PXE_REQUIRE(batch > 0 && width > 0 && height > 0 && num > 0 && coords >= 4 && classes > 0, "region_decode: bad shape");
    PXE_REQUIRE(num <= kRegionMaxBoxes, "region_decode: more than %d boxes per cell", kRegionMaxBoxes);
    PXE_REQUIRE(capacity >= 0, "region_decode: negative capacity");
    PXE_REQUIRE(aligned16(dets), "region_decode: dets must be 16-byte aligned");
    RegionDecodeParams p{};
    p.pred = pred; p.batch = batch; p.W = width; p.H = height; p.num = num; p.coords = coords; p.classes = classes;
    p.per_image = per_image;
    for (int i = 0; i < 2 * num; ++i) p.biases[i] = anchors[i];
    p.img_w = image_width; p.img_h = image_height; p.threshold = threshold;
    p.dets = dets; p.capacity = capacity; p.count = count; p.batch_id_offset = batch_id_offset;
    region_decode_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(p);
    PXE_LAUNCH_OK("region_decode_kernel");
    return PXE_OK;
}

// -------------------------------------------------------------------------------- Softmax decode
extern "C" int pxe_softmax_decode(pxe_stream_t stream, const float* probs, long long probs_batch_stride, int batch,
                                  int classes, float width, float height, float threshold, pxe_detection* dets,
                                  long long capacity, long long* count, int batch_id_offset)
{
    PXE_REQUIRE(probs && dets && count, "softmax_decode: null pointer");
    PXE_REQUIRE(batch > 0 && classes > 0, "softmax_decode: non-positive shape");
    PXE_REQUIRE(probs_batch_stride == 0 || probs_batch_stride >= classes, "softmax_decode: probs_batch_stride too small");
    PXE_REQUIRE(capacity >= 0, "softmax_decode: negative capacity");
    PXE_REQUIRE(aligned16(dets), "softmax_decode: dets must be 16-byte aligned");
    softmax_decode_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        probs, probs_batch_stride ? probs_batch_stride : classes, batch, classes, width, height, threshold, dets, capacity,
        count, batch_id_offset);
    PXE_LAUNCH_OK("softmax_decode_kernel");
    return PXE_OK;
}
