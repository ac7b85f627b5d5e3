// The loss kernels of the two detector heads, which PixieNN's CUDA layers call at the end of a training (or
// validating) forward pass:
//   px::yoloLossGpu        src/YoloKernels.cu:73-252   (regionLossKernel, objectLossKernel, squaredNormKernel,
//                                                        lossComponentsKernel: four launches, three passes over delta)
//   px::centerNetLossGpu   src/CenterNetKernels.cu:20-139 (heat-map focal loss, size / offset L1 loss)
// Here the YOLO loss is one launch: a thread owns one box slot (image, mask slot, cell), decides its deltas the way
// the region kernel and then the object kernel would, and adds the squares of the slot's final deltas to the cost
// and the loss components while it still holds them -- delta is read once and written where it changes.  Sums
// are reduced inside the block first (one atomicAdd per block and statistic instead of one per thread or element),
// so they agree with the reference's sums to rounding; every delta value is computed by the same expressions and
// is identical to the reference's.
#include <cfloat>
#include <stdint.h>

#include "pxe_common.cuh"

namespace pxe {
namespace {

constexpr int kLossThreads = 256;

// Block-wide sum of one value per thread; the total lands in thread 0.
__device__ __forceinline__ float block_sum(float v, float* shared /* kLossThreads / 32 floats */)
{
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    __syncthreads();                                   // the previous use of `shared` is over
    if ((threadIdx.x & 31) == 0) shared[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
    if (threadIdx.x == 0)
        for (int i = 0; i < kLossThreads / 32; ++i) total += shared[i];
    return total;
}

// ---------------------------------------------------------------- YOLO
__device__ __forceinline__ float overlap(float x1, float w1, float x2, float w2)
{
    return fminf(x1 + w1 / 2.0f, x2 + w2 / 2.0f) - fmaxf(x1 - w1 / 2.0f, x2 - w2 / 2.0f);
}

__device__ __forceinline__ float box_iou(const float* a, const float* b)
{
    const float w = overlap(gld(a), gld(a + 2), gld(b), gld(b + 2));
    const float h = overlap(gld(a + 1), gld(a + 3), gld(b + 1), gld(b + 3));
    const float intersection = w > 0.0f && h > 0.0f ? w * h : 0.0f;
    const float union_area = fmaxf(0.0f, gld(a + 2) * gld(a + 3) + gld(b + 2) * gld(b + 3) - intersection);
    return union_area > 0.0f ? intersection / union_area : 0.0f;
}

struct YoloLossParams {
    const float* output; float* delta;
    const float* truths; const int* truth_counts; int max_truth;
    const int* assigned_classes; const int* assigned_anchors; const float* assigned_boxes;
    const int* masks; const float* anchors;
    float* stats; float* cost;
    int slots, mask_count, classes, width, height, net_width, net_height;
    float ignore_threshold, truth_threshold, coord_scale, object_scale, no_object_scale, class_scale;
};

// stats[0] sum of IoU of assigned slots, [1] / [2] how many of them exceed 0.5 / 0.75, [3] their class scores,
// [4] their objectness, [5] objectness of every slot, [6], [7] number of assigned slots, [8] box loss,
// [9] / [10] objectness loss of non-negative / negative deltas, [11] class loss (src/YoloKernels.cu:73-214).
__global__ void __launch_bounds__(kLossThreads)
yolo_loss_kernel(const YoloLossParams p)
{
    __shared__ float red[kLossThreads / 32];
    const int area = p.width * p.height;
    const int entries = p.classes + 5;
    float s_iou = 0.0f, s_r50 = 0.0f, s_r75 = 0.0f, s_cat = 0.0f, s_obj = 0.0f, s_any = 0.0f, s_n = 0.0f;
    float l_box = 0.0f, l_pos = 0.0f, l_neg = 0.0f, l_cls = 0.0f, l_all = 0.0f;
    const int slot = blockIdx.x * kLossThreads + threadIdx.x;
    if (slot < p.slots) {
        const int batch = slot / (p.mask_count * area);
        const int within = slot - batch * (p.mask_count * area);
        const int mask_slot = within / area;
        const int cell = within - mask_slot * area;
        const int x = cell % p.width, y = cell / p.width;
        const int base = batch * p.mask_count * entries * area + mask_slot * entries * area + cell;   // entry 0
        const float* out = p.output + base;
        float* del = p.delta + base;
        const float o0 = gld(out), o1 = gld(out + area), o2 = gld(out + (2 * area)), o3 = gld(out + (3 * area));
        const float objectness = gld(out + (4 * area));

        // what the slot's deltas end up as; entries not decided below keep what delta holds
        float d_box[4];
        float d_obj = gld(del + (4 * area));
        bool write_box = false, write_obj = false, write_cls = false;
        int cls_truth = -1;

        // ---- region part: the prediction against every truth of the image (:73-124)
        {
            const int a = gld(p.masks + mask_slot);
            float pred[4];
            pred[0] = (x + o0) / p.width;
            pred[1] = (y + o1) / p.height;
            pred[2] = expf(o2) * gld(p.anchors + (2 * a)) / p.net_width;
            pred[3] = expf(o3) * gld(p.anchors + (2 * a + 1)) / p.net_height;
            float best_iou = -FLT_MAX;
            int best = -1;
            const int n_truth = gld(p.truth_counts + batch);
            for (int t = 0; t < n_truth; ++t) {
                const int ti = (batch * p.max_truth + t) * 5;
                const float iou = box_iou(pred, p.truths + ti);
                if (iou > best_iou) { best_iou = iou; best = ti; }
            }
            s_any = objectness;
            if (best < 0 || best_iou < p.ignore_threshold) { d_obj = -p.no_object_scale * objectness; write_obj = true; }
            if (best >= 0 && best_iou > p.truth_threshold) {
                d_obj = p.object_scale * (1.0f - objectness);
                write_obj = true;
                cls_truth = (int)gld(p.truths + (best + 4));
                write_cls = true;
                const float* truth = p.truths + best;
                const float scale = p.coord_scale * (2.0f - gld(truth + 2) * gld(truth + 3));
                const float tx = gld(truth) * p.width - x;
                const float ty = gld(truth + 1) * p.height - y;
                const float tw = logf(fmaxf(1e-9f, gld(truth + 2) * p.net_width / gld(p.anchors + (2 * a))));
                const float th = logf(fmaxf(1e-9f, gld(truth + 3) * p.net_height / gld(p.anchors + (2 * a + 1))));
                d_box[0] = scale * (tx - o0); d_box[1] = scale * (ty - o1);
                d_box[2] = scale * (tw - o2); d_box[3] = scale * (th - o3);
                write_box = true;
            }
        }
        // ---- object part: a slot a truth was assigned to (:126-168); overrides the region part
        const int assigned = gld(p.assigned_classes + slot);
        float cat_score = 0.0f;
        if (assigned >= 0) {
            const float* truth = p.assigned_boxes + (size_t)slot * 4;
            const int a = gld(p.assigned_anchors + slot);
            float pred[4];
            pred[0] = (x + o0) / p.width;
            pred[1] = (y + o1) / p.height;
            pred[2] = expf(o2) * gld(p.anchors + (2 * a)) / p.net_width;
            pred[3] = expf(o3) * gld(p.anchors + (2 * a + 1)) / p.net_height;
            const float iou = box_iou(pred, truth);
            const float scale = p.coord_scale * (2.0f - gld(truth + 2) * gld(truth + 3));
            const float tx = gld(truth) * p.width - x;
            const float ty = gld(truth + 1) * p.height - y;
            const float tw = logf(fmaxf(1e-9f, gld(truth + 2) * p.net_width / gld(p.anchors + (2 * a))));
            const float th = logf(fmaxf(1e-9f, gld(truth + 3) * p.net_height / gld(p.anchors + (2 * a + 1))));
            d_box[0] = scale * (tx - o0); d_box[1] = scale * (ty - o1);
            d_box[2] = scale * (tw - o2); d_box[3] = scale * (th - o3);
            write_box = true;
            d_obj = p.object_scale * (1.0f - objectness);
            write_obj = true;
            cls_truth = assigned;
            write_cls = true;
            s_obj = objectness;
            s_iou = iou;
            s_r50 = iou > 0.5f ? 1.0f : 0.0f;
            s_r75 = iou > 0.75f ? 1.0f : 0.0f;
            s_n = 1.0f;
            if (assigned < p.classes) cat_score = fminf(1.0f, gld(out + ((5 + assigned) * area)));
        }
        s_cat = cat_score;

        // ---- store what changed; squares of the slot's final deltas (:170-214)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float v;
            if (write_box) { v = d_box[k]; gst(del + (k * area), v); } else { v = gld(del + (k * area)); }
            l_box += v * v;
        }
        if (write_obj) gst(del + (4 * area), d_obj);
        const float o_sq = d_obj * d_obj;
        if (d_obj >= 0.0f) l_pos = o_sq; else l_neg = o_sq;
        for (int c = 0; c < p.classes; ++c) {
            float v;
            if (write_cls) {
                const float truth_class = c == cls_truth ? 1.0f : 0.0f;
                v = p.class_scale * (truth_class - gld(out + ((5 + c) * area)));
                gst(del + ((5 + c) * area), v);
            } else {
                v = gld(del + ((5 + c) * area));
            }
            l_cls += v * v;
        }
        l_all = l_box + o_sq + l_cls;
    }
    float t;
    t = block_sum(s_iou, red); if (threadIdx.x == 0 && t != 0.0f) gatomic_add(p.stats + 0, t);
    t = block_sum(s_r50, red); if (threadIdx.x == 0 && t != 0.0f) gatomic_add(p.stats + 1, t);
    t = block_sum(s_r75, red); if (threadIdx.x == 0 && t != 0.0f) gatomic_add(p.stats + 2, t);
    t = block_sum(s_cat, red); if (threadIdx.x == 0 && t != 0.0f) gatomic_add(p.stats + 3, t);
    t = block_sum(s_obj, red); if (threadIdx.x == 0 && t != 0.0f) gatomic_add(p.stats + 4, t);
    t = block_sum(s_any, red); if (threadIdx.x == 0) gatomic_add(p.stats + 5, t);
    t = block_sum(s_n, red);   if (threadIdx.x == 0 && t != 0.0f) { gatomic_add(p.stats + 6, t); gatomic_add(p.stats + 7, t); }
    t = block_sum(l_box, red); if (threadIdx.x == 0) gatomic_add(p.stats + 8, t);
    t = block_sum(l_pos, red); if (threadIdx.x == 0) gatomic_add(p.stats + 9, t);
    t = block_sum(l_neg, red); if (threadIdx.x == 0) gatomic_add(p.stats + 10, t);
    t = block_sum(l_cls, red); if (threadIdx.x == 0) gatomic_add(p.stats + 11, t);
    t = block_sum(l_all, red); if (threadIdx.x == 0) gatomic_add(p.cost, t);
}

// ---------------------------------------------------------------- CenterNet
struct CnLossParams {
    const float* output; float* delta;
    const float* target_heat; const float* target_size; const float* target_offset; const float* target_mask;
    float* costs;
    size_t heat_elements, cells;
    int classes, area;
    float normalizer, alpha, beta, size_weight;
};

// Penalty-reduced focal loss on the heat map (src/CenterNetKernels.cu:20-61): costs[0] += the loss,
// delta = normalizer * d(-loss)/d(prediction) at every heat-map element.
__global__ void __launch_bounds__(kLossThreads)
centernet_heat_loss_kernel(const CnLossParams p)
{
    __shared__ float red[kLossThreads / 32];
    const int outputs = (p.classes + 4) * p.area, heat = p.classes * p.area;
    float loss = 0.0f;
    for (size_t i = (size_t)blockIdx.x * kLossThreads + threadIdx.x; i < p.heat_elements; i += (size_t)gridDim.x * kLossThreads) {
        const size_t batch = i / heat;
        const size_t at = batch * outputs + (i - batch * heat);
        const float prediction = fminf(fmaxf(gld(p.output + at), 1e-4f), 1.0f - 1e-4f);
        const float truth = gld(p.target_heat + i);
        if (truth >= 1.0f - 1e-6f) {
            const float one_minus = 1.0f - prediction;
            loss += -powf(one_minus, p.alpha) * logf(prediction);
            gst(p.delta + at, p.normalizer * (powf(one_minus, p.alpha + 1.0f)
                                          - p.alpha * prediction * powf(one_minus, p.alpha) * logf(prediction)));
        } else {
            const float weight = powf(1.0f - truth, p.beta);
            loss += -weight * powf(prediction, p.alpha) * logf(1.0f - prediction);
            gst(p.delta + at, p.normalizer * weight * (p.alpha * powf(prediction, p.alpha) * (1.0f - prediction)
                                                   * logf(1.0f - prediction) - powf(prediction, p.alpha + 1.0f)));
        }
    }
    const float t = block_sum(loss, red);
    if (threadIdx.x == 0) gatomic_add(p.costs, t);
}

// L1 loss on size and offset at the cells a target marks (src/CenterNetKernels.cu:63-122): costs[1], costs[2].
__global__ void __launch_bounds__(kLossThreads)
centernet_regression_loss_kernel(const CnLossParams p)
{
    __shared__ float red[kLossThreads / 32];
    const int outputs = (p.classes + 4) * p.area, heat = p.classes * p.area;
    float size_loss = 0.0f, offset_loss = 0.0f;
    for (size_t i = (size_t)blockIdx.x * kLossThreads + threadIdx.x; i < p.cells; i += (size_t)gridDim.x * kLossThreads) {
        if (gld(p.target_mask + i) == 0.0f) continue;
        const size_t batch = i / p.area, cell = i - batch * p.area;
        const size_t tbase = batch * 2 * p.area, obase = batch * outputs;
        for (int channel = 0; channel < 2; ++channel) {
            const size_t map = (size_t)channel * p.area + cell;
            const size_t si = obase + heat + map, oi = obase + heat + 2 * (size_t)p.area + map;
            const float size_error = gld(p.target_size + (tbase + map)) - gld(p.output + si);
            const float offset_error = gld(p.target_offset + (tbase + map)) - gld(p.output + oi);
            size_loss += fabsf(size_error);
            offset_loss += fabsf(offset_error);
            gst(p.delta + si, p.size_weight * p.normalizer * ((size_error > 0.0f) - (size_error < 0.0f)));
            gst(p.delta + oi, p.normalizer * ((offset_error > 0.0f) - (offset_error < 0.0f)));
        }
    }
    float t = block_sum(size_loss, red);
    if (threadIdx.x == 0) gatomic_add(p.costs + 1, t);
    t = block_sum(offset_loss, red);
    if (threadIdx.x == 0) gatomic_add(p.costs + 2, t);
}

}  // namespace
}  // namespace pxe

using namespace pxe;

extern "C" int pxe_yolo_loss(pxe_stream_t stream, const pxe_yolo_loss_desc* dp)
{
    PXE_REQUIRE(dp != nullptr, "yolo_loss: null descriptor");
    const pxe_yolo_loss_desc& d = *dp;
    PXE_REQUIRE(d.output && d.delta && d.truths && d.truth_counts && d.assigned_classes && d.assigned_anchors &&
                d.assigned_boxes && d.masks && d.anchors && d.stats && d.cost, "yolo_loss: null pointer");
    PXE_REQUIRE(d.batch > 0 && d.mask_count > 0 && d.classes >= 0 && d.width > 0 && d.height > 0 && d.max_truth >= 0,
                "yolo_loss: non-positive shape");
    PXE_REQUIRE(d.network_width > 0 && d.network_height > 0, "yolo_loss: network size must be positive");
    const long long slots = (long long)d.batch * d.mask_count * d.width * d.height;
    PXE_REQUIRE(slots * (d.classes + 5) < 0x7fffffffLL, "yolo_loss: head has too many elements");
    YoloLossParams p{};
    p.output = d.output; p.delta = d.delta; p.truths = d.truths; p.truth_counts = d.truth_counts; p.max_truth = d.max_truth;
    p.assigned_classes = d.assigned_classes; p.assigned_anchors = d.assigned_anchors; p.assigned_boxes = d.assigned_boxes;
    p.masks = d.masks; p.anchors = d.anchors; p.stats = d.stats; p.cost = d.cost;
    p.slots = (int)slots; p.mask_count = d.mask_count; p.classes = d.classes; p.width = d.width; p.height = d.height;
    p.net_width = d.network_width; p.net_height = d.network_height;
    p.ignore_threshold = d.ignore_threshold; p.truth_threshold = d.truth_threshold; p.coord_scale = d.coord_scale;
    p.object_scale = d.object_scale; p.no_object_scale = d.no_object_scale; p.class_scale = d.class_scale;
    yolo_loss_kernel<<<(unsigned)((slots + kLossThreads - 1) / kLossThreads), kLossThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    PXE_LAUNCH_OK("yolo_loss_kernel");
    return PXE_OK;
}

extern "C" int pxe_centernet_loss(pxe_stream_t stream, const float* output, float* delta, const float* target_heatmap,
                                  const float* target_size, const float* target_offset, const float* target_mask,
                                  float* costs, int batch, int classes, int area, float normalizer, float focal_alpha,
                                  float focal_beta, float size_weight)
{
    PXE_REQUIRE(output && delta && target_heatmap && target_size && target_offset && target_mask && costs,
                "centernet_loss: null pointer");
    PXE_REQUIRE(batch > 0 && classes > 0 && area > 0, "centernet_loss: non-positive shape");
    PXE_REQUIRE((long long)(classes + 4) * area < 0x7fffffffLL, "centernet_loss: too many elements per image");
    DeviceInfo di;
    { const int rc = device_info(&di); if (rc != PXE_OK) return rc; }
    CnLossParams p{};
    p.output = output; p.delta = delta; p.target_heat = target_heatmap; p.target_size = target_size;
    p.target_offset = target_offset; p.target_mask = target_mask; p.costs = costs;
    p.heat_elements = (size_t)batch * classes * area; p.cells = (size_t)batch * area;
    p.classes = classes; p.area = area; p.normalizer = normalizer; p.alpha = focal_alpha; p.beta = focal_beta;
    p.size_weight = size_weight;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    centernet_heat_loss_kernel<<<grid_for((long long)p.heat_elements, kLossThreads, di.sm_count, 8), kLossThreads, 0, s>>>(p);
    PXE_LAUNCH_OK("centernet_heat_loss_kernel");
    centernet_regression_loss_kernel<<<grid_for((long long)p.cells, kLossThreads, di.sm_count, 8), kLossThreads, 0, s>>>(p);
    PXE_LAUNCH_OK("centernet_regression_loss_kernel");
    return PXE_OK;
}
