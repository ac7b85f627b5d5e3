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
    int HW, entries, channels, blocks_per_image;
    int groups_per_block;      // consecutive groups of 32 cells one block works through
    int chunks, chunk_len, warps;     // class chunks per mask slot, classes per chunk, warps per block
    pxe_detection* dets;
    long long capacity;
    long long* count;
    int* block_sums;           // [batch*blocks_per_image]
    long long* block_offsets;  // [batch*blocks_per_image]
    unsigned short* masks;     // [batch*blocks_per_image][threads per block]: which classes of a thread's chunk the count
                               // pass found at or above the threshold; NULL = the emit pass finds them again itself
};

// position of channel `ch` at `cell` within one image of the head: planes (the reference's layout) or channels last
__device__ __forceinline__ long long yolo_at(const YoloParams& p, int ch, int cell)
{
    return p.d.head_channels_last ? (long long)cell * p.channels + ch : (long long)ch * p.HW + cell;
}

// value of entry `e` of mask slot `n` at `cell`, activated as YoloLayer::forward leaves it
// (logistic on x, y, objectness, classes; w, h raw -- src/YoloKernels.cu:63-71)
__device__ __forceinline__ float yolo_value(const YoloParams& p, const float* img, int n, int e, int cell)
{
    const int ch = n * p.entries + e;
    float v = gld(img + yolo_at(p, ch, cell));
    if (p.d.head_is_raw) {
        if (p.d.bias) v += gld(p.d.bias + ch);
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
            float v = gld(img + yolo_at(p, ch, cell));
            if (p.d.head_is_raw) {
                if (p.d.bias) v += gld(p.d.bias + ch);
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

// A block takes `groups_per_block` consecutive groups of 32 cells of one image (a launch of one block per group spends
// most of a trained head's decode on starting blocks).  Sums, masks and offsets stay per group.
// MAXW: the most warps a block may have.  Both passes wait on memory, not on registers: with up to 16 warps per block
// (80 classes: 15) they are compiled for four resident blocks per SM -- 32 registers and a few spills -- which
// measured 0.88 ms per YOLOv3-608 step at 64 images against 1.03 with three blocks and 1.23 with two.
template <int MAXW>
__global__ void __launch_bounds__(kYoloCells * MAXW, MAXW <= 16 ? 4 : 1)
yolo_count_kernel(const YoloParams p)
{
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const float* img = p.d.head + (long long)b * p.hbs;
    const int g_end = min((int)(blockIdx.x + 1) * p.groups_per_block, p.blocks_per_image);
    for (int grp = blockIdx.x * p.groups_per_block; grp < g_end; ++grp) {
        const int cell = grp * kYoloCells + lane;
        int cnt = 0;
        unsigned mask = 0;
        if (cell < p.HW) {
            float prob[kYoloChunk], obj;
            cnt = yolo_chunk(p, img, w / p.chunks, w % p.chunks, cell, prob, &obj);
            if (cnt > 0) {                             // prob[] is only filled when the slot's objectness passed
#pragma unroll
                for (int j = 0; j < kYoloChunk; ++j) mask |= prob[j] >= 0.0f ? 1u << j : 0u;
            }
        }
        if (p.masks) gst(p.masks + (((size_t)b * p.blocks_per_image + grp) * blockDim.x + threadIdx.x), (unsigned short)mask);
        // the group's total is an integer: each warp adds its share to the (zeroed) sum, and no warp waits for another
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_down_sync(0xffffffffu, cnt, o);
        int* sum = p.block_sums + (b * p.blocks_per_image + grp);
        if (lane == 0 && cnt != 0 && gcheck(sum)) atomicAdd(sum, cnt);
    }
}

// Exclusive scan of the per-block sums; starts at the running total *count and advances it.
__global__ void __launch_bounds__(1024)
yolo_scan_kernel(const int* block_sums, long long* block_offsets, int n, long long* count)
{
    __shared__ long long warp_tot[32];
    __shared__ long long carry;
    if (threadIdx.x == 0) carry = gld(count);
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        long long v = i < n ? gld(block_sums + i) : 0;
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
        if (i < n) gst(block_offsets + i, c + warp_excl + inc - v);
        __syncthreads();
        if (threadIdx.x == 0) carry = c + warp_tot[31];
        __syncthreads();
    }
    if (threadIdx.x == 0) gst(count, carry);
}

// One 32-byte record as two 128-bit stores (records are 16-byte aligned).
__device__ __forceinline__ void store_detection(pxe_detection* dst, float x, float y, float w, float h, float prob,
                                                int class_id, int batch_id, int source)
{
    float* q = reinterpret_cast<float*>(dst);
    gstv(q, make_float4(x, y, w, h));
    gstv(q + 4, make_float4(prob, __int_as_float(class_id), __int_as_float(batch_id), __int_as_float(source)));
}

// float -> int the way the reference's host decode converts (x86-64 cvttss2si):
// truncation toward zero, INT_MIN for NaN and out-of-range values.
__device__ __forceinline__ int f2i_x86(float v)
{
    if (!(v > -2147483904.0f && v < 2147483648.0f)) return INT_MIN;
    return (int)v;
}

// the records of one thread: box of (cell, mask slot n) and one record per class of its chunk that reached the threshold
__device__ __forceinline__ void yolo_write_records(const YoloParams& p, const float* img, int b, int cell, int n, int chunk,
                                                   unsigned mask, float (&prob)[kYoloChunk], float obj, long long pos)
{
    if (p.masks) {
        obj = yolo_value(p, img, n, 4, cell);
        const int c0m = chunk * p.chunk_len;
#pragma unroll
        for (int j = 0; j < kYoloChunk; ++j)
            prob[j] = (mask >> j) & 1u ? obj * yolo_value(p, img, n, 5 + c0m + j, cell) : -1.0f;
    }

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

template <int MAXW>
__global__ void __launch_bounds__(kYoloCells * MAXW, MAXW <= 16 ? 4 : 1)
yolo_emit_kernel(const YoloParams p)
{
    __shared__ int ranked[kYoloCells * (kYoloMaxWarps + 1)];   // counts, then exclusive prefixes, in emission order
    __shared__ int warp_tot[kYoloMaxWarps];
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const float* img = p.d.head + (long long)b * p.hbs;
    const int n = w / p.chunks, chunk = w % p.chunks;
    const int g_end = min((int)(blockIdx.x + 1) * p.groups_per_block, p.blocks_per_image);
    for (int grp = blockIdx.x * p.groups_per_block; grp < g_end; ++grp) {
        // nothing to write in this group (most groups of a trained head): the same answer for every thread of the block
        if (gld(p.block_sums + (b * p.blocks_per_image + grp)) == 0) continue;
        const int cell = grp * kYoloCells + lane;
        float prob[kYoloChunk], obj = 0.0f;
        int cnt = 0;
        unsigned mask = 0;
        if (p.masks) {
            // the count pass left the classes that reach the threshold: one activation per emitted value, none at all for
            // the threads that emit nothing; the values are loaded after the scan below, so no barrier waits for them
            mask = gld(p.masks + (((size_t)b * p.blocks_per_image + grp) * blockDim.x + threadIdx.x));
            cnt = __popc(mask);
        } else if (cell < p.HW) {
            cnt = yolo_chunk(p, img, n, chunk, cell, prob, &obj);
        }
        // exclusive scan over the block in emission order: rank = lane * warps + w
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
        }
        __syncthreads();
        if (cnt != 0) {
            const long long pos = gld(p.block_offsets + (b * p.blocks_per_image + grp)) + ranked[lane * p.warps + w];
            yolo_write_records(p, img, b, cell, n, chunk, mask, prob, obj, pos);
        }
        __syncthreads();                                  // ranked / warp_tot are reused by the next group
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
            float4 v = gld(reinterpret_cast<const float4*>(p.in) + i);
            if (heat) {
                v.x = act_logistic(v.x + p.bias); v.y = act_logistic(v.y + p.bias);
                v.z = act_logistic(v.z + p.bias); v.w = act_logistic(v.w + p.bias);
            }
            gst(reinterpret_cast<float4*>(p.out) + i, v);
        } else {
            float v = gld(p.in + i);
            if (heat) v = act_logistic(v + p.bias);
            gst(p.out + i, v);
        }
    }
}

constexpr int kCnTileH = 32, kCnTileW = 64, kCnThreads = 256;
constexpr int kCnCells = kCnTileH * kCnTileW;
constexpr int kCnMaxK = 1024;
constexpr int kCnBins = 1024;            // score histogram per image (leading bits of the key above the threshold)
constexpr int kCnListCap = 32768;        // default length of an image's candidate list

struct CnParams {
    pxe_centernet_decode_desc d;
    long long hbs, sbs, obs;
    int K;
    // streaming filter: a group is four consecutive cells of a row; a warp walks groups_per_warp of them
    uint32_t groups, groups_per_warp;  // per image
    FastDiv div_row, div_h;            // by groups per row, by height
    float lo_raw;                    // a cell whose stored value is below this cannot reach the threshold
    float margin;                    // stored values further apart than this have scores in the same order, for certain
    float sat_raw;                   // ... unless the centre value is at or above this (the sigmoid flattens out)
    uint32_t bin_base; int bin_shift;  // activated head: bin = min(kCnBins-1, (score bits - bin_base) >> bin_shift)
    float bin_lo, bin_scale, bin_width;  // logits: bin = (min(value, sat_raw) - bin_lo) * bin_scale, clamped
    int bin_slack;                     // bins below the one holding the K-th candidate that are staged as well
    int sample_stride, sample_want;    // the sampling pass reads every sample_stride-th row and wants this many hot cells
    // tile pass (only for images whose list overflowed or whose raised bound left too few detections)
    int tiles_x, tiles_y;
    float lo;                        // activated-space pre-filter of the tile pass
    float lo_list;                   // its work-list bound, a margin below lo (see centernet_peaks_kernel)
    int cap;                         // keys per image list
    unsigned long long* list;        // [batch][cap] sortable keys, in no particular order
    unsigned long long* list2;       // [batch][cap] valid keys, compacted, when a list does not fit shared memory
    int* count;                      // [batch] keys the streaming filter found (it stores only the first cap)
    int* count2;                     // [batch] keys the tile pass stored for an image it redid
    float* bound;                    // [batch] listing bound of the image: lo_raw, or higher when the sample allowed
    int* redo;                       // images for the tile pass: [0] how many, [1 + i] which (key list overflowed, or a
                                     // raised bound left fewer than K detections)
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
    const float bw = gld(size + idx) / W, bh = gld(size + (area + idx)) / H;
    const float ox = gld(off + idx), oy = gld(off + (area + idx));
    return isfinite(bw) && isfinite(bh) && isfinite(ox) && isfinite(oy) && bw > 0.0f && bh > 0.0f;
}

// The decode runs as a short chain of launches.
//
//  centernet_sample_kernel   one block per image reads every 16th row of the heat map into a histogram of the stored
//                            values and, when the sample holds enough cells above the threshold, raises the
//                            image's listing bound to the histogram bin above which some K/4 sampled cells lie --
//                            about 16 x that many cells of the whole map, several times the K an image keeps.
//  centernet_filter_kernel   streams the heat map once, comparing stored values only (logits, when the head is not
//                            yet activated).  Four consecutive cells none of which reaches the image's listing
//                            bound -- 99 in 100 for a typical head -- cost a 128-bit load and a compare.  The
//                            others are collected and looked at 32 at a time: a cell is listed when it reaches the
//                            bound and no neighbour is larger by more than a margin; it becomes a 64-bit key
//                            (stored value, cell index, and one bit that says whether every neighbour is smaller by
//                            more than the margin) in its image's list.  No exponential is evaluated here.
//  centernet_peaks_kernel    the tile-by-tile pass, which needs no bound and reduces each tile to its best K valid
//                            candidates.  It runs after the selection, only for the images the selection put on
//                            its list: those whose key list overflowed (a plateau makes every cell a maximum) and
//                            those whose raised bound turned out to leave fewer than K detections.
//  centernet_select_kernel   one block per image gives the listed keys the exact treatment -- the reference's
//                            activation expression, the threshold test on the score, the 3x3 test on the
//                            neighbours' exact scores where the margin did not settle it, size / offset validity --
//                            sorts them by (score, index) and writes the K best as boxes.  Run again for the images
//                            the tile pass redid.
//
// Why comparing stored values is enough for most cells.  The activation 1/(1+exp(-v)) is increasing with slope
// s(1-s).  For a centre value v < 8 (in activated units: after the bias) the slope on [v - m, v + m] is at least
// 3.3e-4, so two values at least m = 0.01 apart have true scores at least 3.3e-6 apart, an order of magnitude more
// than the rounding of expf, the add and the division (a few units of 6e-8).  So "a neighbour exceeds the centre by
// more than m" settles "its score is strictly greater", and "every neighbour is below the centre by more than m"
// settles the opposite; only the cases in between, and centres at or above 8 (where the sigmoid flattens out and
// different logits share a score), need the neighbours' exact scores.  The bias is added only where a score is
// evaluated: v + bias rounds monotonically, and its rounding error (1e-6 at these magnitudes) is far inside the
// margin.  A head that is already activated is compared exactly (margin 0).
//
// Why a raised bound loses nothing.  Cells below the bound are never listed.  If at least K of the listed cells
// with a value of bound + m or more turn out to be detections, each of them has a strictly larger score than any
// cell below the bound, so the K best of the image are all listed.  If fewer do, the image is redone by the tile
// pass.  An image whose bound was not raised lists every cell that can reach the threshold.

constexpr int kCnQueueFlush = 64;        // keys a warp collects before it reserves room in the image's list
constexpr int kCnQueueLen = kCnQueueFlush + 32;

// Key written by the filter: stored value (order-preserving bits) | (0x7fffffff - cell index) << 1 | settled bit.
__device__ __forceinline__ unsigned long long cn_raw_key(float value, uint32_t flat, bool settled)
{
    return ((unsigned long long)float_order(value) << 32) | (unsigned long long)(((0x7fffffffu - flat) << 1) | (settled ? 1u : 0u));
}

// Histogram bin of a stored value: linear between bin_lo and the saturation bound for logits (bins are bin_width
// wide in logit units), leading bits of the score for an activated head.  Non-decreasing in the value.
__device__ __forceinline__ int cn_bin(const CnParams& p, float value)
{
    if (p.d.heat_is_logit) {
        const float t = (fminf(value, p.sat_raw) - p.bin_lo) * p.bin_scale;
        return t > 0.0f ? min((int)t, kCnBins - 1) : 0;
    }
    const uint32_t hi = float_order(value);
    const uint32_t bin = hi >= p.bin_base ? (hi - p.bin_base) >> p.bin_shift : 0u;
    return (int)(bin < (uint32_t)kCnBins ? bin : kCnBins - 1);
}

// A value that is not above any value of bin j (j >= 1).
__device__ __forceinline__ float cn_bin_floor(const CnParams& p, int j)
{
    if (p.d.heat_is_logit) return p.bin_lo + (float)(j - 1) * p.bin_width;      // one bin of slack for the rounding of cn_bin
    return order_float(p.bin_base + ((uint32_t)j << p.bin_shift));
}

constexpr int kCnSampleThreads = 512;

template <bool VEC>
__global__ void __launch_bounds__(kCnSampleThreads)
centernet_sample_kernel(const CnParams p)
{
    __shared__ int hist[kCnBins];
    __shared__ int warp_tot[kCnSampleThreads / 32];
    __shared__ int lead_bin;
    const int b = blockIdx.x;
    const int H = p.d.height, W = p.d.width;
    for (int i = threadIdx.x; i < kCnBins; i += kCnSampleThreads) hist[i] = 0;
    if (threadIdx.x == 0) lead_bin = 0;
    __syncthreads();
    const int rows_per_plane = (H + p.sample_stride - 1) / p.sample_stride;
    const int rows = p.d.classes * rows_per_plane;
    const float* heat = p.d.heat + (long long)b * p.hbs;
    const float lo = p.lo_raw;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kWarps = kCnSampleThreads / 32, kRows = 4;      // a warp reads kRows sampled rows at a time
    auto count = [&](float v) { if (v >= lo) atomicAdd(&hist[cn_bin(p, v)], 1); };
    for (int r0 = warp; r0 < rows; r0 += kRows * kWarps) {
        const float* src[kRows];
#pragma unroll
        for (int j = 0; j < kRows; ++j) {
            const int r = min(r0 + j * kWarps, rows - 1);
            const int cls = r / rows_per_plane, gy = (r - cls * rows_per_plane) * p.sample_stride;
            src[j] = heat + ((long long)cls * H + gy) * W;
        }
        if (VEC) {
            for (int x = 4 * lane; x < W; x += 128) {
                float4 v[kRows];
#pragma unroll
                for (int j = 0; j < kRows; ++j) v[j] = gldgv<float4>(src[j] + x);
#pragma unroll
                for (int j = 0; j < kRows; ++j)
                    if (r0 + j * kWarps < rows) { count(v[j].x); count(v[j].y); count(v[j].z); count(v[j].w); }
            }
        } else {
            for (int x = lane; x < W; x += 32) {
                float v[kRows];
#pragma unroll
                for (int j = 0; j < kRows; ++j) v[j] = gldg(src[j] + x);
#pragma unroll
                for (int j = 0; j < kRows; ++j)
                    if (r0 + j * kWarps < rows) count(v[j]);
            }
        }
    }
    __syncthreads();
    // the highest bin with sample_want sampled cells in or above it: thread t owns kCnBins / threads bins, from the top
    constexpr int kPer = kCnBins / kCnSampleThreads;
    const int top = kCnBins - 1 - kPer * (int)threadIdx.x;
    int mine = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) mine += hist[top - j];
    int inc = mine;
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int before = inc - mine;
    for (int i = 0; i < warp; ++i) before += warp_tot[i];
    if (before < p.sample_want && before + mine >= p.sample_want) {
        int acc = before, bin = top;
        for (int j = 0; j < kPer; ++j) {
            if (acc + hist[top - j] >= p.sample_want) { bin = top - j; break; }
            acc += hist[top - j];
        }
        lead_bin = bin;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float bound = lo;
        if (lead_bin >= 2) bound = fmaxf(lo, cn_bin_floor(p, lead_bin));
        gst(p.bound + b, bound);
    }
}

// Writes the first n keys of a warp's queue to the image's list: one reservation (one atomic) per call.  The
// count keeps running past the end of the list, which is how the selection sees that the list overflowed.
__device__ __forceinline__ void cn_flush(const unsigned long long* queue, int n, unsigned long long* list, int cap,
                                         int* count)
{
    const int lane = threadIdx.x & 31;
    int base = 0;
    if (lane == 0 && gcheck(count)) base = atomicAdd(count, n);
    base = __shfl_sync(0xffffffffu, base, 0);
    for (int i = lane; i < n; i += 32)
        if (base + i < cap) gst(list + (base + i), queue[i]);
}

constexpr int kCnFilterWarps = 8;
constexpr int kCnLoads = 8;              // 128-bit loads a lane keeps in flight
constexpr int kCnHotLen = 64;            // hot groups a warp collects before it looks at their neighbourhoods

// The filter in two speeds.  A "group" is four consecutive cells of a row (one 128-bit load).
//  stream   a warp walks its share of the image's groups, eight loads in flight per lane, and only asks whether
//           any of a group's four cells reaches the image's listing bound.  For a typical head one group in a
//           hundred does ("hot"); its index goes to the warp's queue.  Everything else costs a load and a compare.
//  look     once 32 hot groups are queued, each lane takes one: it reads the group's 3 x 6 neighbourhood (from L2,
//           the rows were streamed moments ago), forms the largest neighbour of each of the four cells and lists a
//           cell when it reaches the bound and no neighbour is larger by more than the margin.  A listed cell
//           becomes a key in the warp's key queue, which is written to the image's list 64 keys at a time.
template <bool VEC>
__global__ void __launch_bounds__(kCnFilterWarps * 32)
centernet_filter_kernel(const CnParams p)
{
    __shared__ unsigned long long key_queues[kCnFilterWarps][kCnQueueLen];
    __shared__ uint32_t hot_queues[kCnFilterWarps][kCnHotLen];
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const uint32_t wi = blockIdx.x * kCnFilterWarps + (threadIdx.x >> 5);
    const uint32_t g_begin = wi * (uint32_t)p.groups_per_warp;
    if (g_begin >= p.groups) return;
    const uint32_t g_end = min(p.groups, g_begin + (uint32_t)p.groups_per_warp);
    const int H = p.d.height, W = p.d.width;
    const float* heat = p.d.heat + (long long)b * p.hbs;
    const float lo = gld(p.bound + b), m = p.margin, sat = p.sat_raw;
    // outside the map: never listed (NaN >= x is false), never greater than anything (fmaxf skips NaN)
    const float OUT = __int_as_float(0x7fffffff);
    unsigned long long* key_queue = key_queues[threadIdx.x >> 5];
    uint32_t* hot_queue = hot_queues[threadIdx.x >> 5];
    unsigned long long* list = p.list + (long long)b * p.cap;
    int qn = 0, hn = 0;                                           // keys / hot groups queued, the same in every lane

    // the four cells of group g (row g / groups_per_row over all classes, columns 4 * (g % groups_per_row) ...)
    auto load_group = [&](uint32_t g) {
        if (VEC) return gldgv<float4>(heat + 4 * (size_t)g);
        uint32_t row, gx;
        p.div_row.divmod(g, row, gx);
        const int x = 4 * (int)gx;
        const float* src = heat + (size_t)row * W + x;
        float4 v = make_float4(OUT, OUT, OUT, OUT);
        v.x = gldg(src);
        if (x + 1 < W) v.y = gldg(src + 1);
        if (x + 2 < W) v.z = gldg(src + 2);
        if (x + 3 < W) v.w = gldg(src + 3);
        return v;
    };

    // look at up to 32 queued hot groups, one per lane
    auto look = [&](int n) {
        const bool active = lane < n;
        float4 c = make_float4(OUT, OUT, OUT, OUT);
        float nbx = OUT, nby = OUT, nbz = OUT, nbw = OUT;
        uint32_t flat = 0;
        if (active) {
            const uint32_t g = hot_queue[lane];
            uint32_t row, gx;
            p.div_row.divmod(g, row, gx);                          // row over all classes: class * H + y
            const uint32_t cls = p.div_h.div(row);
            const int gy = (int)(row - cls * (uint32_t)H), x = 4 * (int)gx;
            flat = row * (uint32_t)W + (uint32_t)x;                // (class * H + y) * W + x
            float4 r[3];
            float l[3], rt[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const int ny = gy + k - 1;
                r[k] = make_float4(OUT, OUT, OUT, OUT);
                l[k] = OUT; rt[k] = OUT;
                if (ny >= 0 && ny < H) {
                    const float* src = heat + ((size_t)row + k - 1) * W + x;
                    if (VEC) {
                        r[k] = gldgv<float4>(src);
                    } else {
                        r[k].x = gldg(src);
                        if (x + 1 < W) r[k].y = gldg(src + 1);
                        if (x + 2 < W) r[k].z = gldg(src + 2);
                        if (x + 3 < W) r[k].w = gldg(src + 3);
                    }
                    if (x > 0) l[k] = gldg(src - 1);
                    if (x + 4 < W) rt[k] = gldg(src + 4);
                }
            }
            c = r[1];
            const float4 u = r[0], d = r[2];
            // largest neighbour of each of the four cells: three above, three below, two beside
            const float ux = fmaxf(fmaxf(l[0], u.x), u.y), uy = fmaxf(fmaxf(u.x, u.y), u.z);
            const float uz = fmaxf(fmaxf(u.y, u.z), u.w), uw = fmaxf(fmaxf(u.z, u.w), rt[0]);
            const float dx = fmaxf(fmaxf(l[2], d.x), d.y), dy = fmaxf(fmaxf(d.x, d.y), d.z);
            const float dz = fmaxf(fmaxf(d.y, d.z), d.w), dw = fmaxf(fmaxf(d.z, d.w), rt[2]);
            nbx = fmaxf(fmaxf(ux, dx), fmaxf(l[1], c.y)); nby = fmaxf(fmaxf(uy, dy), fmaxf(c.x, c.z));
            nbz = fmaxf(fmaxf(uz, dz), fmaxf(c.y, c.w)); nbw = fmaxf(fmaxf(uw, dw), fmaxf(c.z, rt[1]));
        }
        // listed: reaches the bound, and not (a neighbour larger by more than the margin while the centre is
        // below the saturation bound, where a larger neighbour may still have the same score)
        unsigned fm = (c.x >= lo && !(nbx > c.x + m && c.x < sat) ? 1u : 0u) |
                      (c.y >= lo && !(nby > c.y + m && c.y < sat) ? 2u : 0u) |
                      (c.z >= lo && !(nbz > c.z + m && c.z < sat) ? 4u : 0u) |
                      (c.w >= lo && !(nbw > c.w + m && c.w < sat) ? 8u : 0u);
        while (__any_sync(0xffffffffu, fm != 0u)) {               // one cell per lane and round
            const bool has = fm != 0u;
            const int col = has ? __ffs(fm) - 1 : 0;
            const float me = col == 0 ? c.x : col == 1 ? c.y : col == 2 ? c.z : c.w;
            const float nb = col == 0 ? nbx : col == 1 ? nby : col == 2 ? nbz : nbw;
            const unsigned mask = __ballot_sync(0xffffffffu, has);
            if (has) {
                const bool settled = nb <= me - m && me < sat;     // every neighbour's score is smaller, for certain
                key_queue[qn + __popc(mask & ((1u << lane) - 1u))] = cn_raw_key(me, flat + (uint32_t)col, settled);
            }
            qn += __popc(mask);
            fm &= fm - 1u;
            __syncwarp();
            if (qn >= kCnQueueFlush) {
                cn_flush(key_queue, kCnQueueFlush, list, p.cap, p.count + b);
                const unsigned long long rest = key_queue[kCnQueueFlush + lane];   // at most 31 keys lie beyond
                __syncwarp();
                if (lane < qn - kCnQueueFlush) key_queue[lane] = rest;
                __syncwarp();
                qn -= kCnQueueFlush;
            }
        }
    };

    for (uint32_t g0 = g_begin; g0 < g_end; g0 += 32 * kCnLoads) {
        float4 v[kCnLoads];
#pragma unroll
        for (int k = 0; k < kCnLoads; ++k) {
            const uint32_t g = g0 + 32 * k + lane;
            v[k] = g < g_end ? load_group(g) : make_float4(OUT, OUT, OUT, OUT);
        }
#pragma unroll
        for (int k = 0; k < kCnLoads; ++k) {
            const bool hot = v[k].x >= lo || v[k].y >= lo || v[k].z >= lo || v[k].w >= lo;
            const unsigned mask = __ballot_sync(0xffffffffu, hot);
            if (mask) {
                if (hot) hot_queue[hn + __popc(mask & ((1u << lane) - 1u))] = g0 + 32 * k + lane;
                hn += __popc(mask);
                __syncwarp();
                if (hn >= 32) {
                    look(32);
                    const uint32_t rest = hot_queue[32 + lane];    // at most 31 groups lie beyond the ones looked at
                    __syncwarp();
                    if (lane < hn - 32) hot_queue[lane] = rest;
                    __syncwarp();
                    hn -= 32;
                }
            }
        }
    }
    if (hn > 0) look(hn);
    if (qn > 0) cn_flush(key_queue, qn, list, p.cap, p.count + b);
}

// The exact treatment of one key of the filter: size / offset validity (include/CenterNetLayer.h:217-225), the
// reference's activation expression (src/CenterNetKernels.cu:17), the threshold test on the score and, unless the
// filter settled it, the 3x3 test on the neighbours' scores (include/CenterNetLayer.h:181-194, 212).  Returns the
// final key (score, index) or 0 when the cell is not a detection.
__device__ __forceinline__ unsigned long long cn_exact(const CnParams& p, const float* heat, const float* size,
                                                       const float* off, unsigned long long key)
{
    const int H = p.d.height, W = p.d.width;
    const uint32_t area = (uint32_t)H * (uint32_t)W;               // cells per image < 2^31
    const uint32_t low = (uint32_t)(key & 0xffffffffu);
    const uint32_t flat = 0x7fffffffu - (low >> 1);
    const bool settled = (low & 1u) != 0u;
    const float c = order_float((uint32_t)(key >> 32));
    const uint32_t cls = flat / area;
    const uint32_t idx = flat - cls * area;
    if (!cn_valid(size, off, (long long)idx, (long long)area, W, H)) return 0ULL;
    const bool logit = p.d.heat_is_logit != 0;
    const float bias = p.d.heatmap_bias;
    const float s = logit ? 1.0f / (1.0f + expf(-(c + bias))) : c;
    if (!isfinite(s) || s < p.d.threshold) return 0ULL;
    if (logit && !settled) {
        const float m = p.margin, sat = p.sat_raw;
        const float* plane = heat + (size_t)cls * area;
        const int gy = (int)(idx / (uint32_t)W), gx = (int)(idx - (uint32_t)gy * (uint32_t)W);
        const float NONE = __int_as_float(0x7fffffff);             // outside the map: compares false
        float nv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int dy = (k < 3) ? -1 : (k < 5 ? 0 : 1);
            const int dx = (k < 3) ? k - 1 : (k == 3 ? -1 : (k == 4 ? 1 : k - 6));
            const int ny = gy + dy, nx = gx + dx;
            nv[k] = (ny >= 0 && ny < H && nx >= 0 && nx < W) ? gldg(plane + (size_t)ny * W + nx) : NONE;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            // a neighbour below the centre by more than the margin cannot have a larger score (centre < sat)
            if (nv[k] > c - m || (!(c < sat) && nv[k] == nv[k])) {
                const float ns = 1.0f / (1.0f + expf(-(nv[k] + bias)));
                if (ns > s) return 0ULL;
            }
        }
    }
    return cn_key(s, flat);
}

// The tile pass, for the images on the list `todo` ([0]: how many, [1 + i]: which).  One block per (32x64 tile,
// class) walks those images.
//  load   the tile's pre-activation values (logit + bias) with a one-cell halo go to shared memory,
//         128 bits at a time where the row alignment allows; every value that is not clearly below the
//         threshold (in pre-activation space) is put on a work list on the way.
//  score  the activation (the reference's precise sigmoid) is evaluated once per work-list entry.
//  peak   interior entries at or above the threshold are compared with their 8 neighbours' scores.
//         A neighbour that is not on the work list is clearly below the threshold in pre-activation
//         space; the activation is non-decreasing, so its score cannot exceed that of a cell which
//         reached the threshold ("clearly" = a margin far wider than any rounding in exp()).
//  select a tile with more than K surviving candidates passes on only its K best valid ones, so an image's
//         list (at least tiles x classes x K keys long) always holds what this pass appends.
constexpr int kCnRowStride = 72;                      // floats per shared-memory row; interior starts at column 4
constexpr int kCnSmemCells = (kCnTileH + 2) * kCnRowStride;

template <bool VEC>
__global__ void __launch_bounds__(kCnThreads)
centernet_peaks_kernel(const CnParams p, const int* todo)
{
    __shared__ __align__(16) float tile[kCnSmemCells];
    __shared__ __align__(16) float score[kCnSmemCells];
    __shared__ unsigned short work[(kCnTileH + 2) * (kCnTileW + 2)];
    __shared__ unsigned long long keys[kCnCells];
    __shared__ int n_keys, n_out, n_work, base;
    __shared__ int hist[256];
    __shared__ unsigned long long sel[2];

    const int cls = blockIdx.y;
    const int ty = blockIdx.x / p.tiles_x, tx = blockIdx.x - ty * p.tiles_x;
    const int y0 = ty * kCnTileH, x0 = tx * kCnTileW;
    const int H = p.d.height, W = p.d.width;
    const long long area = (long long)H * W;
    const bool logit = p.d.heat_is_logit != 0;
    const float bias = logit ? p.d.heatmap_bias : 0.0f;
    const float lo_list = p.lo_list;
    constexpr float NEG = -INFINITY;                  // outside the map: never greater than a score
    const int n_over = min(gld(todo), p.d.batch);

    for (int oi = blockIdx.z; oi < n_over; oi += gridDim.z) {
    const int b = gld(todo + (1 + oi));
    const float* heat = p.d.heat + (long long)b * p.hbs + (long long)cls * area;
    __syncthreads();                                  // the previous image's shared state is dead
    if (threadIdx.x == 0) { n_keys = 0; n_out = 0; n_work = 0; }
    __syncthreads();

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
                    v = gldv<float4>(src);
                    v.x += bias; v.y += bias; v.z += bias; v.w += bias;
                } else {
                    v.x = gld(src) + bias;
                    if (gx + 1 < W) v.y = gld(src + 1) + bias;
                    if (gx + 2 < W) v.z = gld(src + 2) + bias;
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
            if (gy >= 0 && gy < H && gx >= 0 && gx < W) v = gld(heat + ((long long)gy * W + gx)) + bias;
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
            if (gy >= 0 && gy < H && gx >= 0 && gx < W) v = gld(heat + ((long long)gy * W + gx)) + bias;
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

    // ---- peak test -> key
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

    const int n = n_keys;
    unsigned long long* out = p.list + (long long)b * p.cap;
    if (n <= p.K) {
        if (threadIdx.x == 0) base = n && gcheck(p.count2 + b) ? atomicAdd(p.count2 + b, n) : 0;
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += kCnThreads) gst(out + (base + i), keys[i]);
        continue;
    }
    // More candidates than an image keeps: the tile's K best are enough -- but only valid candidates may
    // compete for those places, so validity is checked here first.
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
    __syncthreads();
    unsigned long long kth = 1ULL;                     // every valid key
    if (n_valid > p.K) kth = block_select_kth([&](int i) { return keys[i]; }, n, p.K, hist, sel);
    const int n_pass = n_valid > p.K ? p.K : n_valid;
    if (threadIdx.x == 0) base = n_pass && gcheck(p.count2 + b) ? atomicAdd(p.count2 + b, n_pass) : 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kCnThreads)
        if (keys[i] >= kth) gst(out + (base + atomicAdd(&n_out, 1)), keys[i]);
    }
}

// One block per image: the K best of the image's candidates, sorted, decoded to boxes.
//  1. a short list (up to about 2.5 K keys) is staged whole.  A longer one is counted into a histogram of the
//     stored values first; the bin in or above which at least K + K/4 + 32 keys lie, less bin_slack bins whose
//     scores are not separated from it for certain, bounds what is staged;
//  2. staged keys get the exact treatment (cn_exact).  If K or more of the keys in or above the bin turn out to
//     be detections, the K best of the list are among the staged ones, because every key left out has a strictly
//     smaller score;
//  3. otherwise (many invalid boxes, one bin holding thousands of equal scores, or an image the tile pass redid)
//     every key is treated, the detections are compacted and the K-th key is found by radix selection;
//  4. the staged keys are sorted (bitonic, shared memory) and the first K become records -- unless the image's
//     listing bound was raised and fewer than K detections lie clear above it: then the list may be missing some
//     of the K best, and the image goes on the list of images to redo.
// `only` == nullptr: block b treats image b.  Otherwise the blocks walk the images listed in `only`, which the tile
// pass has redone.
constexpr int kCnSelThreads = 512;
constexpr int kCnStageKeys = 4096;     // candidates per image sorted in shared memory (32 KB)
constexpr int kCnRankKeys = 128;       // up to this many, keys are placed by counting instead of sorted
static_assert(kCnBins == 2 * kCnSelThreads, "the top-down scan gives every thread 2 bins");

__global__ void __launch_bounds__(kCnSelThreads)
centernet_select_kernel(const CnParams p, const int* only)
{
    __shared__ unsigned long long stage[kCnStageKeys];
    __shared__ int bins[kCnBins];
    __shared__ int hist[256];
    __shared__ unsigned long long sel[2];
    __shared__ int warp_tot[kCnSelThreads / 32];
    __shared__ int n_best, n_valid, n_top, n_above, lead_bin;
    const int H = p.d.height, W = p.d.width;
    const long long area = (long long)H * W;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_items = only ? min(gld(only), p.d.batch) : p.d.batch;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int b = only ? gld(only + (1 + item)) : item;
    const float* heat = p.d.heat + (long long)b * p.hbs;
    const float* size = p.d.size + (long long)b * p.sbs;
    const float* off = p.d.offset + (long long)b * p.obs;
    const unsigned long long* cand = p.list + (long long)b * p.cap;
    const int found = gld(p.count + b);
    if (only == nullptr && found > p.cap) {
        // the filter found more keys than the list holds (a plateau): the tile pass redoes this image
        if (threadIdx.x == 0) {
            if (gcheck(p.redo)) gst(p.redo + (1 + atomicAdd(p.redo, 1)), b);
            gst(p.counts + b, 0);
        }
        continue;
    }
    // an image on the list was redone by the tile pass, which stored count2 final keys (at most cap)
    const bool redone = only != nullptr;
    const int n_total = redone ? min(gld(p.count2 + b), p.cap) : found;
    const float bound = gld(p.bound + b);
    const bool raised = !redone && bound > p.lo_raw;
    const float clear = bound + p.margin;              // a detection at or above this beats every cell below the bound
    __syncthreads();                                   // the previous image's shared state is dead
    if (threadIdx.x == 0) { n_valid = 0; n_best = 0; n_top = 0; n_above = 0; lead_bin = 0; }
    __syncthreads();

    unsigned long long* sorted = stage;
    int m = 0;
    bool done = false;
    if (!redone) {
        int lead = 0, lead_staged = 0;
        if (n_total > 2 * (p.K + p.K / 4 + 32)) {
            // 1. histogram of the stored values; thread t owns bins kCnBins-1-2t and the one below, from the top
            for (int i = threadIdx.x; i < kCnBins; i += kCnSelThreads) bins[i] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < n_total; i += kCnSelThreads)
                atomicAdd(&bins[cn_bin(p, order_float((uint32_t)(gld(cand + i) >> 32)))], 1);
            __syncthreads();
            const int want = p.K + p.K / 4 + 32;
            const int top = kCnBins - 1 - 2 * (int)threadIdx.x;
            const int h0 = bins[top], h1 = bins[top - 1];
            const int mine = h0 + h1;
            int inc = mine;
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            if (lane == 31) warp_tot[warp] = inc;
            __syncthreads();
            int before = inc - mine;
            for (int i = 0; i < warp; ++i) before += warp_tot[i];
            if (before < want && before + mine >= want) lead_bin = before + h0 >= want ? top : top - 1;
            __syncthreads();
            lead = lead_bin;
            lead_staged = lead > p.bin_slack ? lead - p.bin_slack : 0;
        }

        // 2. stage, then the exact treatment
#pragma unroll 4
        for (int i = threadIdx.x; i < n_total; i += kCnSelThreads) {
            const unsigned long long key = gld(cand + i);
            if (lead_staged == 0 || cn_bin(p, order_float((uint32_t)(key >> 32))) >= lead_staged) {
                const int at = atomicAdd(&n_best, 1);
                if (at < kCnStageKeys) stage[at] = key;
            }
        }
        __syncthreads();
        const int n_c = n_best;
        if (n_c <= kCnStageKeys) {
            for (int i0 = 0; i0 < n_c; i0 += kCnSelThreads) {     // all threads of a warp take part in the votes
                const int i = i0 + threadIdx.x;
                bool ok = false, top = false, above = false;
                if (i < n_c) {
                    const unsigned long long key = stage[i];
                    const unsigned long long fin = cn_exact(p, heat, size, off, key);
                    stage[i] = fin;                                // 0 sorts behind every real key
                    if (fin != 0ULL) {
                        const float value = order_float((uint32_t)(key >> 32));
                        ok = true;
                        top = lead == 0 || cn_bin(p, value) >= lead;
                        above = value >= clear;
                    }
                }
                const unsigned v_ok = __ballot_sync(0xffffffffu, ok), v_top = __ballot_sync(0xffffffffu, top);
                const unsigned v_above = __ballot_sync(0xffffffffu, above);
                if (lane == 0 && v_ok) {
                    atomicAdd(&n_valid, __popc(v_ok));
                    if (v_top) atomicAdd(&n_top, __popc(v_top));
                    if (v_above) atomicAdd(&n_above, __popc(v_above));
                }
            }
            __syncthreads();
            if (n_top >= p.K || n_c == n_total) {
                m = n_valid < p.K ? n_valid : p.K;
                if (n_c <= kCnRankKeys) {
                    // few keys: every thread finds the place of its key by counting the larger ones; the first
                    // K places are written to the front of a second area
                    unsigned long long* out = stage + kCnStageKeys / 2;
                    for (int i = threadIdx.x; i < n_c; i += kCnSelThreads) {
                        const unsigned long long mine = stage[i];
                        if (mine == 0ULL) continue;
                        int rank = 0;
                        for (int j = 0; j < n_c; ++j) rank += stage[j] > mine ? 1 : 0;
                        if (rank < m) out[rank] = mine;
                    }
                    sorted = out;
                    __syncthreads();
                } else {
                    int pow2 = 1;
                    while (pow2 < n_c) pow2 <<= 1;
                    for (int i = n_c + threadIdx.x; i < pow2; i += kCnSelThreads) stage[i] = 0ULL;
                    __syncthreads();
                    block_bitonic_desc(stage, pow2);
                }
                done = true;
            }
        }
        __syncthreads();
    }

    if (!done) {
        if (threadIdx.x == 0) { n_valid = 0; n_best = 0; n_above = 0; }
        __syncthreads();
        // 3. the exact treatment of every key + compaction
        const bool staged = n_total <= kCnStageKeys;
        unsigned long long* list = staged ? stage : p.list2 + (long long)b * p.cap;
        for (int i = threadIdx.x; i < n_total; i += kCnSelThreads) {
            unsigned long long key = gld(cand + i);
            if (redone) {                                  // final keys of the tile pass: only validity is open
                const uint32_t flat = 0xffffffffu - (uint32_t)(key & 0xffffffffu);
                const uint32_t cls = flat / (uint32_t)area;
                if (!cn_valid(size, off, (long long)(flat - cls * (uint32_t)area), area, W, H)) key = 0ULL;
            } else {
                const float value = order_float((uint32_t)(key >> 32));
                key = cn_exact(p, heat, size, off, key);
                if (key != 0ULL && value >= clear) atomicAdd(&n_above, 1);
            }
            if (key != 0ULL) gst(list + (atomicAdd(&n_valid, 1)), key);
        }
        __syncthreads();
        const int n = n_valid;

        if (staged) {
            int pow2 = 1;
            while (pow2 < n) pow2 <<= 1;
            for (int i = n + threadIdx.x; i < pow2; i += kCnSelThreads) stage[i] = 0ULL;
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
                const unsigned long long lead16 = block_select_kth([&](int i) { return gld(list + i); }, n, p.K, hist, sel, 2, &want) >> 48;
                const int winners = p.K - want;
                if (threadIdx.x == 0) { n_best = 0; n_valid = 0; }      // n_valid is reused as the tie counter
                __syncthreads();
                for (int i = threadIdx.x; i < n; i += kCnSelThreads) {
                    const unsigned long long key = gld(list + i);
                    const unsigned long long top = key >> 48;
                    if (top > lead16) stage[atomicAdd(&n_best, 1)] = key;
                    else if (top == lead16) {
                        const int at = atomicAdd(&n_valid, 1);
                        if (winners + at < kCnStageKeys) stage[winners + at] = key;
                    }
                }
                __syncthreads();
                if (winners + n_valid <= kCnStageKeys) {
                    m_sort = winners + n_valid;
                } else {
                    const unsigned long long kth = block_select_kth([&](int i) { return gld(list + i); }, n, p.K, hist, sel);
                    if (threadIdx.x == 0) n_best = 0;
                    __syncthreads();
                    for (int i = threadIdx.x; i < n; i += kCnSelThreads) {
                        const unsigned long long key = gld(list + i);
                        if (key >= kth) stage[atomicAdd(&n_best, 1)] = key;
                    }
                    __syncthreads();
                    m_sort = n_best;
                }
            } else {
                for (int i = threadIdx.x; i < n; i += kCnSelThreads) stage[i] = gld(list + i);
                m_sort = n;
            }
            __syncthreads();
            int pow2 = 1;
            while (pow2 < m_sort) pow2 <<= 1;
            for (int i = m_sort + threadIdx.x; i < pow2; i += kCnSelThreads) stage[i] = 0ULL;
            __syncthreads();
            block_bitonic_desc(stage, pow2);
            m = m_sort < p.K ? m_sort : p.K;
        }
    }
    __syncthreads();
    if (raised && n_above < p.K) {
        // the raised bound may have kept some of the K best off the list: the tile pass redoes this image
        if (threadIdx.x == 0) {
            if (gcheck(p.redo)) gst(p.redo + (1 + atomicAdd(p.redo, 1)), b);
            gst(p.counts + b, 0);
        }
        continue;
    }
    const float image_w = p.d.image_width > 0 ? (float)p.d.image_width : 1.0f;
    const float image_h = p.d.image_height > 0 ? (float)p.d.image_height : 1.0f;
    for (int i = threadIdx.x; i < m; i += blockDim.x) {
        const unsigned long long key = sorted[i];
        const uint32_t flat = 0xffffffffu - (uint32_t)(key & 0xffffffffu);
        const float score = order_float((uint32_t)(key >> 32));
        const int cls = (int)(flat / (uint32_t)area);
        const uint32_t idx = flat - (uint32_t)cls * (uint32_t)area;
        const int y = (int)(idx / (uint32_t)W), x = (int)(idx - (uint32_t)y * (uint32_t)W);
        // include/CenterNetLayer.h:217-237, each product and sum rounded separately as on the host
        const float bw = gld(size + idx) / W, bh = gld(size + (area + idx)) / H;
        const float cx = (x + gld(off + idx)) / W, cy = (y + gld(off + (area + idx))) / H;
        store_detection(p.dets + (long long)b * p.K + i, __fmul_rn(__fsub_rn(cx, bw / 2.0f), image_w),
                        __fmul_rn(__fsub_rn(cy, bh / 2.0f), image_h), __fmul_rn(bw, image_w), __fmul_rn(bh, image_h),
                        score, cls, b + p.d.batch_id_offset, (int)flat);
    }
    if (threadIdx.x == 0) gst(p.counts + b, m);
    }
}

// ============================================================================================
// Softmax / Region
// ============================================================================================
// One block per row of n contiguous values: out = exp(x/temp - max/temp) / sum (src/Math.cpp:77-97).
// PER > 0: rows of up to 128 * PER values stay in registers between the three passes (same operations in the same
// order as the form that re-reads the row, so the same bits); PER == 0: any length.
template <int PER>
__global__ void __launch_bounds__(128)
softmax_rows_kernel(const float* in, float* out, int n, float temp)
{
    __shared__ float red[4];
    __shared__ float bcast;
    const float* x = in + (long long)blockIdx.x * n;
    float* y = out + (long long)blockIdx.x * n;
    constexpr int R = PER > 0 ? PER : 1;
    float xv[R];
    float m = -FLT_MAX;
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const int i = threadIdx.x + 128 * k;
            xv[k] = i < n ? gld(x + i) : -FLT_MAX;
            m = xv[k] > m ? xv[k] : m;
        }
    } else {
        for (int i = threadIdx.x; i < n; i += 128) m = gld(x + i) > m ? gld(x + i) : m;
    }
    for (int o = 16; o > 0; o >>= 1) { float t = __shfl_xor_sync(0xffffffffu, m, o); m = t > m ? t : m; }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) { float t = red[0]; for (int w = 1; w < 4; ++w) t = red[w] > t ? red[w] : t; bcast = t; }
    __syncthreads();
    const float largest = bcast;
    float sum = 0.0f;
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (threadIdx.x + 128 * k < n) {
                xv[k] = expf(xv[k] / temp - largest / temp);
                sum += xv[k];
            }
        }
    } else {
        for (int i = threadIdx.x; i < n; i += 128) {
            const float e = expf(gld(x + i) / temp - largest / temp);
            gst(y + i, e);
            sum += e;
        }
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) bcast = red[0] + red[1] + red[2] + red[3];
    __syncthreads();
    const float total = bcast;
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < R; ++k)
            if (threadIdx.x + 128 * k < n) gst(y + (threadIdx.x + 128 * k), xv[k] / total);
    } else {
        for (int i = threadIdx.x; i < n; i += 128) gst(y + i, gld(y + i) / total);
    }
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
            float v = gld(src + ((long long)e * p.HW));
            if (e == 4) v = act_logistic(v);
            gst(dst + e, v);
        }
        if (p.softmax) {
            float* cls = dst + p.coords + 1;
            float largest = -FLT_MAX, sum = 0.0f;
            for (int j = 0; j < p.classes; ++j) largest = gld(cls + j) > largest ? gld(cls + j) : largest;
            for (int j = 0; j < p.classes; ++j) { const float e = expf(gld(cls + j) - largest); sum += e; gst(cls + j, e); }
            for (int j = 0; j < p.classes; ++j) gst(cls + j, gld(cls + j) / sum);
        }
    }
}

// The same result from coalesced traffic: a warp takes 32 consecutive cells of one (image, box slot).  It reads the
// slot's `size` planes row by row (32 consecutive cells = one 128-byte request) into a shared-memory tile, each lane
// then does its own cell's objectness and softmax on its column of the tile (the operations and their order are the
// thread-per-box kernel's, so the bits are), and the warp writes the 32 records out, each as consecutive floats.  The
// thread-per-box form reads with a stride of HW floats and writes with a stride of `size` floats per lane, and runs
// its three softmax passes over global memory.  Rows are 33 floats apart: no bank conflicts in any of the phases.
constexpr int kRegionWarps = 4;

__global__ void __launch_bounds__(kRegionWarps * 32)
region_forward_tile_kernel(const RegionParams p, int tiles_per_plane, long long tiles)
{
    extern __shared__ float region_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* tile = region_smem + (size_t)warp * p.size * 33;
    const long long outputs = (long long)p.HW * p.num * p.size;
    for (long long t = (long long)blockIdx.x * kRegionWarps + warp; t < tiles; t += (long long)gridDim.x * kRegionWarps) {
        const int tp = (int)(t % tiles_per_plane);
        const long long r = t / tiles_per_plane;
        const int n = (int)(r % p.num), b = (int)(r / p.num);
        const int cell0 = tp * 32, cell = cell0 + lane;
        const bool live = cell < p.HW;
        const float* src = p.in + b * outputs + (long long)n * p.size * p.HW + cell;
        for (int e0 = 0; e0 < p.size; e0 += 16) {              // sixteen rows in flight per lane
            float r[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) r[k] = (live && e0 + k < p.size) ? gld(src + (long long)(e0 + k) * p.HW) : 0.0f;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (e0 + k < p.size) tile[(e0 + k) * 33 + lane] = r[k];
        }
        if (live) {
            float* col = tile + lane;
            col[4 * 33] = act_logistic(col[4 * 33]);
            if (p.softmax) {
                float* cls = col + (p.coords + 1) * 33;
                float largest = -FLT_MAX, sum = 0.0f;
                for (int j = 0; j < p.classes; ++j) largest = cls[j * 33] > largest ? cls[j * 33] : largest;
                for (int j = 0; j < p.classes; ++j) { const float e = expf(cls[j * 33] - largest); sum += e; cls[j * 33] = e; }
                for (int j = 0; j < p.classes; ++j) cls[j * 33] = cls[j * 33] / sum;
            }
        }
        __syncwarp();
        const int live_cells = min(32, p.HW - cell0);
        for (int c = 0; c < live_cells; ++c) {
            float* dst = p.out + b * outputs + ((long long)(cell0 + c) * p.num + n) * p.size;
            for (int e = lane; e < p.size; e += 32) gst(dst + e, tile[e * 33 + c]);
        }
        __syncwarp();
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
    if (threadIdx.x == 0) carry = gld(p.count);
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
            const float scale = gld(pred + (locations * p.classes + slot));
            if (isfinite(scale) && scale > 0.0f) {
                const float* box = pred + (long long)locations * (p.classes + p.num) + (long long)slot * p.coords;
                const float x = __fmul_rn((gld(box) + col) / p.side, p.width);
                const float y = __fmul_rn((gld(box + 1) + row) / p.side, p.height);
                // the host squares with std::pow(v, 2), glibc's powf: within one ulp of v*v, equal to it for
                // all but ~0.06 % of inputs; one multiplication here
                const float w = __fmul_rn(p.squared ? __fmul_rn(gld(box + 2), gld(box + 2)) : gld(box + 2), p.width);
                const float h = __fmul_rn(p.squared ? __fmul_rn(gld(box + 3), gld(box + 3)) : gld(box + 3), p.height);
                best_prob = -FLT_MAX;
                for (int j = 0; j < p.classes; ++j) {
                    const float pr = __fmul_rn(scale, gld(pred + (i * p.classes + j)));
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
    if (threadIdx.x == 0) gst(p.count, carry);
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
    if (threadIdx.x == 0) carry = gld(p.count);
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
            scale = gld(box + p.coords);
            for (int j = 0; j < p.classes; ++j)
                if (__fmul_rn(scale, gld(box + (p.coords + 1 + j))) >= p.threshold) ++cnt;
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
            const float x = (col + 1.0f / (1.0f + expf(-gld(box)))) / p.W;
            const float y = (row + 1.0f / (1.0f + expf(-gld(box + 1)))) / p.H;
            const float bw = expf(gld(box + 2)) * p.biases[2 * n] / p.W;
            const float bh = expf(gld(box + 3)) * p.biases[2 * n + 1] / p.H;
            const float x1 = __fmul_rn(x, p.img_w), y1 = __fmul_rn(y, p.img_h);
            const float ww = __fmul_rn(bw, p.img_w), hh = __fmul_rn(bh, p.img_h);
            for (int j = 0; j < p.classes; ++j) {
                const float pr = __fmul_rn(scale, gld(box + (p.coords + 1 + j)));
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
    if (threadIdx.x == 0) gst(p.count, carry);
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
    if (threadIdx.x == 0) carry = gld(count);
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
            first_is_nan = !(gld(p) == gld(p));
            for (int j = lane; j < classes; j += 32) {
                const float v = gld(p + j);
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
    if (threadIdx.x == 0) gst(count, carry);
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

extern "C" size_t pxe_yolo_decode_fast_workspace_bytes(int batch, int height, int width)
{
    if (batch <= 0 || height <= 0 || width <= 0) return 0;
    const size_t hw = (size_t)height * width;
    const size_t bpi = (hw + kYoloCells - 1) / kYoloCells;
    return pxe_yolo_decode_workspace_bytes(batch, height, width) +
           align_up((size_t)batch * bpi * kYoloCells * kYoloMaxWarps * sizeof(unsigned short), 256);
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
    p.channels = d.n_masks * p.entries;
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
    ws += align_up((size_t)d.batch * p.blocks_per_image * sizeof(long long), 256);
    // with room for them, the count pass leaves per-thread class masks and the emit pass evaluates only what it
    // emits (chunks longer than the register window keep the plain form: their tail is not in the mask)
    p.masks = nullptr;
    if (workspace_bytes >= pxe_yolo_decode_fast_workspace_bytes(d.batch, d.height, d.width) && p.chunk_len <= kYoloChunk)
        p.masks = reinterpret_cast<unsigned short*>(ws);

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    // enough blocks to fill the machine sixteen times over, each working through up to eight groups of 32 cells
    const long long groups_total = (long long)p.blocks_per_image * d.batch;
    long long gpb = (groups_total + (long long)di.sm_count * 16 - 1) / ((long long)di.sm_count * 16);
    p.groups_per_block = (int)(gpb < 1 ? 1 : (gpb > 8 ? 8 : gpb));
    dim3 grid((unsigned)((p.blocks_per_image + p.groups_per_block - 1) / p.groups_per_block), (unsigned)d.batch);
    const unsigned threads = (unsigned)(kYoloCells * p.warps);
    PXE_CUDA_OK(cudaMemsetAsync(p.block_sums, 0, sizeof(int) * (size_t)d.batch * p.blocks_per_image, s));
    if (p.warps <= 16) yolo_count_kernel<16><<<grid, threads, 0, s>>>(p);
    else yolo_count_kernel<kYoloMaxWarps><<<grid, threads, 0, s>>>(p);
    PXE_LAUNCH_OK("yolo_count_kernel");
    yolo_scan_kernel<<<1, 1024, 0, s>>>(p.block_sums, p.block_offsets, d.batch * p.blocks_per_image, count);
    PXE_LAUNCH_OK("yolo_scan_kernel");
    if (p.warps <= 16) yolo_emit_kernel<16><<<grid, threads, 0, s>>>(p);
    else yolo_emit_kernel<kYoloMaxWarps><<<grid, threads, 0, s>>>(p);
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
#ifdef PXE_BOUNDS_CHECK
            if (const int rc = pxe::bounds_add_internal(p, sizeof(g_yolo_static_scratch))) return rc;
#endif
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

// Keys per image list: enough for what the tile pass may append (tiles x classes x K), by default kCnListCap,
// never more than the image has cells.
static long long cn_list_cap(int classes, int height, int width, int max_detections, long long* floor_out)
{
    int tx, ty;
    long long bpi;
    cn_geometry(classes, height, width, &tx, &ty, &bpi);
    const long long cells = (long long)classes * height * width;
    long long floor_cap = bpi * max_detections;
    if (floor_cap > cells) floor_cap = cells;
    long long cap = floor_cap > kCnListCap ? floor_cap : kCnListCap;
    if (cap > cells) cap = cells;
    if (floor_out) *floor_out = floor_cap;
    return cap;
}

static size_t cn_counter_ints(int batch)
{
    return 2 * (size_t)batch + (size_t)batch + 1;                // count, count2, redo list
}

extern "C" size_t pxe_centernet_decode_workspace_bytes(int batch, int classes, int height, int width,
                                                       int max_detections)
{
    if (batch <= 0 || classes <= 0 || height <= 0 || width <= 0 || max_detections <= 0) return 0;
    const long long cap = cn_list_cap(classes, height, width, max_detections, nullptr);
    return 2 * align_up((size_t)batch * cap * sizeof(unsigned long long), 256)
           + align_up(cn_counter_ints(batch) * sizeof(int), 256) + align_up((size_t)batch * sizeof(float), 256);
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

static uint32_t host_float_order(float f)
{
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
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
    PXE_REQUIRE(area * d.classes < 0x7fffffffLL, "centernet_decode: heatmap has too many cells per image");
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
    long long bpi, floor_cap;
    cn_geometry(d.classes, d.height, d.width, &p.tiles_x, &p.tiles_y, &bpi);
    const long long full_cap = cn_list_cap(d.classes, d.height, d.width, d.max_detections, &floor_cap);
    PXE_REQUIRE(full_cap < 0x7fffffffLL && bpi < 0x7fffffffLL, "centernet_decode: candidate table too large");
    PXE_REQUIRE(d.candidate_capacity >= 0 && d.candidate_capacity <= full_cap,
                "centernet_decode: candidate_capacity %d outside 0..%lld", d.candidate_capacity, full_cap);
    p.K = d.max_detections;
    p.cap = (int)(d.candidate_capacity == 0 ? full_cap : (d.candidate_capacity < floor_cap ? floor_cap : d.candidate_capacity));
    p.lo = centernet_prefilter(d);
    p.lo_list = d.heat_is_logit ? p.lo - 2e-4f * fmaxf(1.0f, fabsf(p.lo)) : p.lo;
    if (d.heat_is_logit) {
        // the filter compares stored logits; the bias is added only where a score is evaluated
        const float shifted = p.lo - d.heatmap_bias;
        p.lo_raw = isfinite(shifted) ? shifted - 1e-3f * fmaxf(1.0f, fabsf(p.lo) + fabsf(d.heatmap_bias)) : shifted;
        p.margin = 0.01f;
        p.sat_raw = 8.0f - d.heatmap_bias;
        if (!isfinite(p.sat_raw)) p.sat_raw = -INFINITY;        // a non-finite bias: every listed cell takes the exact test
    } else {
        p.lo_raw = d.threshold;
        p.margin = 0.0f;
        p.sat_raw = INFINITY;
    }
    // histogram bins (sampling pass; long lists in the selection).  Logits: linear from the listing bound (at
    // most 64 below the saturation bound) to the saturation bound; bins are bin_width wide, so keys bin_slack
    // bins apart differ by more than the margin.  Activated head: leading bits of the score between the
    // threshold and the largest float.
    p.bin_base = host_float_order(d.threshold);
    const uint32_t top = host_float_order(FLT_MAX);
    p.bin_shift = 0;
    while (top > p.bin_base && ((top - p.bin_base) >> p.bin_shift) >= (uint32_t)kCnBins) ++p.bin_shift;
    p.bin_lo = 0.0f; p.bin_scale = 0.0f; p.bin_width = 0.0f; p.bin_slack = 0;
    if (d.heat_is_logit) {
        p.bin_lo = fmaxf(p.lo_raw, p.sat_raw - 64.0f);
        const float width = (p.sat_raw - p.bin_lo) / (float)(kCnBins - 1);
        if (isfinite(width) && width > 0.0f) {
            p.bin_width = width;
            p.bin_scale = 1.0f / width;
            p.bin_slack = (int)ceilf(p.margin / width) + 1;
        } else {
            p.bin_lo = 0.0f;                                     // degenerate bounds: one bin, every key staged
            p.bin_slack = kCnBins;
        }
    }
    // the sampling pass: every 16th row; it raises an image's bound when some 4K cells of the whole map lie above
    p.sample_stride = d.height >= 32 ? 16 : 1;
    p.sample_want = 4 * p.K / p.sample_stride + 16;
    // groups of four cells; a warp's share is a multiple of what its lanes load at once, sized for a few waves
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    const bool vec = d.width % 4 == 0 && aligned16(d.heat) && p.hbs % 4 == 0;   // 128-bit loads: rows start on 16 bytes
    const uint32_t groups_per_row = (uint32_t)((d.width + 3) / 4);
    p.groups = (uint32_t)d.classes * (uint32_t)d.height * groups_per_row;     // < 2^31
    p.div_row = FastDiv(groups_per_row);
    p.div_h = FastDiv((uint32_t)d.height);
    const uint32_t step = 32 * kCnLoads;
    uint32_t share = 8 * step;
    while (share > step && (long long)d.batch * ((p.groups + share - 1) / share) < 4LL * 24 * di.sm_count) share >>= 1;
    p.groups_per_warp = share;
    const long long wpi = (p.groups + share - 1) / share;

    char* ws = static_cast<char*>(workspace);
    const size_t list_bytes = align_up((size_t)d.batch * full_cap * sizeof(unsigned long long), 256);
    p.list = reinterpret_cast<unsigned long long*>(ws);
    p.list2 = reinterpret_cast<unsigned long long*>(ws + list_bytes);
    int* ints = reinterpret_cast<int*>(ws + 2 * list_bytes);
    p.count = ints;
    p.count2 = ints + d.batch;
    p.redo = ints + 2 * (size_t)d.batch;
    p.bound = reinterpret_cast<float*>(ws + 2 * list_bytes + align_up(cn_counter_ints(d.batch) * sizeof(int), 256));
    p.dets = dets; p.counts = counts;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PXE_CUDA_OK(cudaMemsetAsync(ints, 0, cn_counter_ints(d.batch) * sizeof(int), s));
    if (vec) centernet_sample_kernel<true><<<(unsigned)d.batch, kCnSampleThreads, 0, s>>>(p);
    else centernet_sample_kernel<false><<<(unsigned)d.batch, kCnSampleThreads, 0, s>>>(p);
    PXE_LAUNCH_OK("centernet_sample_kernel");
    dim3 fgrid((unsigned)((wpi + kCnFilterWarps - 1) / kCnFilterWarps), (unsigned)d.batch);
    if (vec) centernet_filter_kernel<true><<<fgrid, kCnFilterWarps * 32, 0, s>>>(p);
    else centernet_filter_kernel<false><<<fgrid, kCnFilterWarps * 32, 0, s>>>(p);
    PXE_LAUNCH_OK("centernet_filter_kernel");
    centernet_select_kernel<<<(unsigned)d.batch, kCnSelThreads, 0, s>>>(p, nullptr);
    PXE_LAUNCH_OK("centernet_select_kernel");
    // The selection puts two kinds of image on a list that is empty in the normal case: those whose key list
    // overflowed and those whose raised bound left fewer than K detections.  The tile pass redoes them (its
    // blocks return at once when there are none) and the selection runs again for them.
    const unsigned walkers = (unsigned)(d.batch < 2 ? d.batch : 2);
    dim3 tgrid((unsigned)(p.tiles_x * p.tiles_y), (unsigned)d.classes, walkers);
    if (vec) centernet_peaks_kernel<true><<<tgrid, kCnThreads, 0, s>>>(p, p.redo);
    else centernet_peaks_kernel<false><<<tgrid, kCnThreads, 0, s>>>(p, p.redo);
    PXE_LAUNCH_OK("centernet_peaks_kernel");
    centernet_select_kernel<<<walkers, kCnSelThreads, 0, s>>>(p, p.redo);
    PXE_LAUNCH_OK("centernet_select_kernel");
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
    const int row = inputs / groups;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (row <= 128) softmax_rows_kernel<1><<<(unsigned)rows, 128, 0, s>>>(in, out, row, temperature);
    else if (row <= 256) softmax_rows_kernel<2><<<(unsigned)rows, 128, 0, s>>>(in, out, row, temperature);
    else if (row <= 512) softmax_rows_kernel<4><<<(unsigned)rows, 128, 0, s>>>(in, out, row, temperature);
    else if (row <= 1024) softmax_rows_kernel<8><<<(unsigned)rows, 128, 0, s>>>(in, out, row, temperature);
    else if (row <= 2048) softmax_rows_kernel<16><<<(unsigned)rows, 128, 0, s>>>(in, out, row, temperature);
    else softmax_rows_kernel<0><<<(unsigned)rows, 128, 0, s>>>(in, out, row, temperature);
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
    const size_t tile_bytes = (size_t)kRegionWarps * p.size * 33 * sizeof(float);
    if (tile_bytes <= (size_t)di.max_smem_optin) {
        if (tile_bytes > 48 * 1024)
            PXE_CUDA_OK(cudaFuncSetAttribute(region_forward_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_bytes));
        const int tiles_per_plane = (p.HW + 31) / 32;
        const long long tiles = (long long)batch * num * tiles_per_plane;
        const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (size_t)(200 * 1024) / tile_bytes));
        region_forward_tile_kernel<<<grid_for(tiles, kRegionWarps, di.sm_count, per_sm), kRegionWarps * 32, tile_bytes,
                                     static_cast<cudaStream_t>(stream)>>>(p, tiles_per_plane, tiles);
        PXE_LAUNCH_OK("region_forward_tile_kernel");
        return PXE_OK;
    }
    // records too long for a shared-memory tile: a thread per box
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
