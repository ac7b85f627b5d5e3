/*
 * pxe_shim.h -- the glue a patched PixieNN needs around libpxe.so's fused tier.
 *
 * Include it from the headers under include/cuda/ (after Error.h, which supplies PX_CHECK).  The bodies in this folder's
 * *.inl files are meant to be #included INSIDE the member functions they replace, where the layer's private
 * members are visible:
 *
 *   conv_forward_epilogue.inl    ConvLayer<Device::CUDA>::forward, in place of include/cuda/ConvLayer.h:284-307
 *   route_forward.inl            RouteLayer<Device::CUDA>::forward, in place of include/cuda/RouteLayer.h:25-43
 *   maxpool_forward.inl          MaxPoolLayer<Device::CUDA>::forward, in place of include/cuda/MaxPoolLayer.h:39-41
 *   upsample_forward.inl         UpsampleLayer<Device::CUDA>::forward, in place of include/cuda/UpsampleLayer.h:37-38
 *   shortcut_forward.inl         ShortcutLayer<Device::CUDA>::forward, in place of include/cuda/ShortcutLayer.h:27-33
 *   yolo_add_detects.inl         YoloLayer<Device::CUDA>::addDetects, in place of include/cuda/YoloLayer.h:171-176
 *   centernet_add_detects.inl    CenterNetLayer<Device::CUDA>::addDetects, in place of include/cuda/CenterNetLayer.h:92-95
 *   region_forward.inl           RegionLayer<Device::CUDA>::forward (inferring), in place of include/cuda/RegionLayer.h:43-53
 *   region_add_detects.inl       RegionLayer<Device::CUDA>::addDetects, in place of include/cuda/RegionLayer.h:76-82
 *   softmax_forward.inl          SoftmaxLayer<Device::CUDA>::forward, in place of include/cuda/SoftmaxLayer.h:72-74
 *   avgpool_forward.inl          AvgPoolLayer<Device::CUDA>::forward, in place of include/cuda/AvgPoolLayer.h:71-73
 *   conn_forward_epilogue.inl    ConnLayer<Device::CUDA>::forward (inferring), in place of include/cuda/ConnLayer.h:187-216
 *   detect_add_detects.inl       DetectLayer<Device::CUDA>::addDetects, in place of include/cuda/DetectLayer.h:81-86
 *
 * What the fragments expect from the surrounding class beyond the reference's own members is listed at the top of
 * each; it comes to: a `const pxe_shim::PlanView& pxePlan()` on the model (built once after parseModel, see
 * build_plan below), a non-const `float* pxeOutput()` on Layer (today only `output() const` exists,
 * include/Layer.h:77), and the layer's activation as an int (`pxeActivation_`, from activation_from_name).
 */
#ifndef PXE_SHIM_H
#define PXE_SHIM_H

#include <cstddef>
#include <string>
#include <vector>

#include "pxe.h"
#include "pxe_plan.h"

#ifndef PXE_CHECK
#define PXE_CHECK(call)                                                    \
    do {                                                                   \
        int pxe_rc_ = (call);                                              \
        PX_CHECK(pxe_rc_ == PXE_OK, "pxe: %s", pxe_last_error_string());   \
    } while (0)
#endif

namespace pxe_shim {

/* The YAML `activation:` string -> PXE_ACT_* (the values of ActivationType, include/ActivationTypes.h:19-30). */
inline int activation_from_name(const std::string& name)
{
    static const char* const names[] = {"leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"};
    for (int i = 0; i < 9; ++i)
        if (name == names[i]) return i;
    return -1;
}

/* The plan plus the index from a layer to the step that produces it (a layer folded into an earlier step has none). */
struct PlanView {
    pxe_plan* plan = nullptr;
    std::vector<int> step_of;                      /* layer -> step index, or -1 */

    const pxe_step* step(int layer) const
    {
        const int s = layer >= 0 && layer < (int)step_of.size() ? step_of[layer] : -1;
        return s >= 0 ? pxe_plan_step(plan, s) : nullptr;
    }
};

/* Built once at the end of Model<D>::parseModel (include/Model.h:1596-1641) from one pxe_layer_desc per layer.
 * raw_heads = 0: the convolution in front of a YOLO layer keeps its epilogue (bias, linear), YoloLayer<CUDA>::forward
 * activates into output_ as in the reference -- output() is public -- and yolo_add_detects.inl decodes that tensor.
 * (With raw_heads = 1 the plan marks those convolutions head_raw: no epilogue, and the decode must then be given the
 * raw convolution output, the bias and head_is_raw = 1 instead; the fragments here do not take that route.) */
inline int build_plan(const std::vector<pxe_layer_desc>& descs, bool inferring, PlanView* out)
{
    const int rc = pxe_plan_build(descs.data(), (int)descs.size(), inferring ? 1 : 0, /*raw_heads=*/0, &out->plan);
    if (rc != PXE_OK) return rc;
    out->step_of.assign(descs.size(), -1);
    for (int s = 0; s < pxe_plan_step_count(out->plan); ++s) {
        const pxe_step* st = pxe_plan_step(out->plan, s);
        out->step_of[st->layer] = s;
        if (st->fused_shortcut >= 0) out->step_of[st->fused_shortcut] = s;
        if (st->fused_pool >= 0) out->step_of[st->fused_pool] = s;
        for (int g = 1; g < st->n_spp; ++g) out->step_of[st->spp_layers[g]] = s;
    }
    return PXE_OK;
}

/* Where a planned destination lives: a dense tensor of `own` elements per image, or a channel slot of a route's
 * concat buffer (`route_output` = that route layer's output_, `route_outputs` = its elements per image). */
struct Slot {
    float* ptr;
    long long batch_stride;
};

inline Slot resolve(const pxe_dest& d, float* own_output, long long own_outputs, float* route_output,
                    long long route_outputs, long long plane /* H*W of the stored tensor */)
{
    if (d.kind == 0) return Slot{own_output, own_outputs};
    return Slot{route_output + (long long)d.channel_offset * plane, route_outputs};
}

/* One tensor copied into a further destination (a step stores up to two destinations itself; a tensor that still more
 * routes read is copied from the first). */
inline int copy_to(const float* src, long long src_batch_stride, int channels, const Slot& dst, int batch, int height, int width)
{
    return pxe_concat(nullptr, 1, &src, &src_batch_stride, &channels, dst.ptr, dst.batch_stride, batch, height, width);
}

}   // namespace pxe_shim

#endif /* PXE_SHIM_H */
