"""ctypes declarations for ``libpxe.so`` (the C ABI in ``include/pxe.h``).

This module only loads the library and declares prototypes.  It fails loudly when the library
has not been built: there is no CPU or PyTorch fallback for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libpxe.so")

PXE_OK, PXE_ERR_BAD_ARG, PXE_ERR_UNSUPPORTED, PXE_ERR_CUDA, PXE_ERR_WORKSPACE = range(5)

ACT = {"leaky": 0, "linear": 1, "loggy": 2, "logistic": 3, "mish": 4, "relu": 5, "softplus": 6,
       "swish": 7, "tanh": 8, "yolo_head": 100}
EPS_CUDNN, EPS_CPU = 0, 1


class PxeError(RuntimeError):
    """A C-ABI call returned a non-zero status (the counterpart of px::Error / px::CudaError)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"pxe status {status}: {message}")
        self.status = status


class Detection(C.Structure):
    _fields_ = [("x", C.c_float), ("y", C.c_float), ("w", C.c_float), ("h", C.c_float),
                ("prob", C.c_float), ("class_id", C.c_int32), ("batch_id", C.c_int32),
                ("source", C.c_int32)]


class EpilogueDesc(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("x_batch_stride", C.c_longlong),
        ("y", C.c_void_p), ("y_batch_stride", C.c_longlong),
        ("y2", C.c_void_p), ("y2_batch_stride", C.c_longlong),
        ("batch", C.c_int), ("channels", C.c_int), ("height", C.c_int), ("width", C.c_int),
        ("gamma", C.c_void_p), ("beta", C.c_void_p), ("mean", C.c_void_p), ("var", C.c_void_p),
        ("eps", C.c_float), ("eps_mode", C.c_int),
        ("bias", C.c_void_p), ("act", C.c_int), ("yolo_classes", C.c_int),
        ("residual", C.c_void_p), ("residual_batch_stride", C.c_longlong),
        ("res_alpha", C.c_float), ("res_beta", C.c_float), ("res_act", C.c_int),
        ("pool_kernel", C.c_int), ("pool_stride", C.c_int), ("pool_padding", C.c_int),
        ("y_pool", C.c_void_p), ("y_pool_batch_stride", C.c_longlong), ("pool_variant", C.c_int),
        ("folded_a", C.c_void_p), ("folded_b", C.c_void_p),
    ]


class EpilogueNhwcDesc(C.Structure):
    """pxe_epilogue_nhwc_desc of include/pxe.h."""
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("y2", C.c_void_p), ("residual", C.c_void_p),
                ("x_pixel_stride", C.c_longlong), ("y_pixel_stride", C.c_longlong), ("y2_pixel_stride", C.c_longlong),
                ("residual_pixel_stride", C.c_longlong), ("pixels", C.c_longlong), ("channels", C.c_int),
                ("a", C.c_void_p), ("b", C.c_void_p), ("act", C.c_int), ("res_alpha", C.c_float), ("res_beta", C.c_float),
                ("res_act", C.c_int), ("pool_kernel", C.c_int), ("pool_stride", C.c_int), ("pool_padding", C.c_int),
                ("batch", C.c_int), ("height", C.c_int), ("width", C.c_int), ("y_pool", C.c_void_p),
                ("y_pool_pixel_stride", C.c_longlong)]


class StemDesc(C.Structure):
    """pxe_stem_desc of include/pxe.h."""
    _fields_ = [("x", C.c_void_p), ("x_batch_stride", C.c_longlong), ("weights", C.c_void_p), ("a", C.c_void_p),
                ("b", C.c_void_p), ("y", C.c_void_p), ("y_is_nhwc", C.c_int), ("y_stride", C.c_longlong),
                ("batch", C.c_int), ("in_channels", C.c_int), ("out_channels", C.c_int), ("height", C.c_int),
                ("width", C.c_int), ("act", C.c_int)]


class YoloDecodeDesc(C.Structure):
    _fields_ = [
        ("head", C.c_void_p), ("head_batch_stride", C.c_longlong),
        ("head_is_raw", C.c_int), ("bias", C.c_void_p),
        ("batch", C.c_int), ("height", C.c_int), ("width", C.c_int), ("classes", C.c_int),
        ("n_masks", C.c_int), ("mask", C.c_int * 16),
        ("n_anchor_values", C.c_int), ("anchors", C.c_int * 64),
        ("net_width", C.c_int), ("net_height", C.c_int),
        ("image_width", C.c_int), ("image_height", C.c_int),
        ("threshold", C.c_float), ("batch_id_offset", C.c_int), ("head_channels_last", C.c_int),
    ]


class CenterNetDecodeDesc(C.Structure):
    _fields_ = [
        ("heat", C.c_void_p), ("heat_batch_stride", C.c_longlong),
        ("size", C.c_void_p), ("size_batch_stride", C.c_longlong),
        ("offset", C.c_void_p), ("offset_batch_stride", C.c_longlong),
        ("heat_is_logit", C.c_int), ("heatmap_bias", C.c_float),
        ("batch", C.c_int), ("classes", C.c_int), ("height", C.c_int), ("width", C.c_int),
        ("image_width", C.c_int), ("image_height", C.c_int),
        ("threshold", C.c_float), ("max_detections", C.c_int), ("batch_id_offset", C.c_int),
        ("candidate_capacity", C.c_int),
    ]


POOL_AUTO, POOL_GENERAL = 0, 1            # enum pxe_pool_variant
class YoloLossDesc(C.Structure):
    """pxe_yolo_loss_desc of include/pxe.h."""
    _fields_ = [("output", C.c_void_p), ("delta", C.c_void_p), ("truths", C.c_void_p), ("truth_counts", C.c_void_p),
                ("max_truth", C.c_int), ("assigned_classes", C.c_void_p), ("assigned_anchors", C.c_void_p),
                ("assigned_boxes", C.c_void_p), ("masks", C.c_void_p), ("anchors", C.c_void_p), ("stats", C.c_void_p),
                ("cost", C.c_void_p), ("batch", C.c_int), ("mask_count", C.c_int), ("classes", C.c_int),
                ("width", C.c_int), ("height", C.c_int), ("network_width", C.c_int), ("network_height", C.c_int),
                ("ignore_threshold", C.c_float), ("truth_threshold", C.c_float), ("coord_scale", C.c_float),
                ("object_scale", C.c_float), ("no_object_scale", C.c_float), ("class_scale", C.c_float)]


class BnTrainDesc(C.Structure):
    """pxe_bn_train_desc of include/pxe.h."""
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("y_act", C.c_void_p), ("act", C.c_int),
                ("batch", C.c_int), ("channels", C.c_int), ("height", C.c_int), ("width", C.c_int),
                ("gamma", C.c_void_p), ("beta", C.c_void_p), ("running_mean", C.c_void_p), ("running_var", C.c_void_p),
                ("exp_avg_factor", C.c_float), ("eps", C.c_float), ("eps_mode", C.c_int),
                ("save_mean", C.c_void_p), ("save_scale", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t)]


class BnBackwardDesc(C.Structure):
    """pxe_bn_backward_desc of include/pxe.h."""
    _fields_ = [("x", C.c_void_p), ("dy", C.c_void_p), ("dx", C.c_void_p),
                ("batch", C.c_int), ("channels", C.c_int), ("height", C.c_int), ("width", C.c_int),
                ("gamma", C.c_void_p), ("dgamma", C.c_void_p), ("dbeta", C.c_void_p),
                ("save_mean", C.c_void_p), ("save_scale", C.c_void_p), ("eps", C.c_float), ("eps_mode", C.c_int),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


PLAN_MAX_SOURCES, PLAN_MAX_DESTS, PLAN_MAX_SPP = 16, 8, 4


class LayerDesc(C.Structure):
    """pxe_layer_desc of include/pxe_plan.h."""
    _fields_ = [("type", C.c_int), ("out_channels", C.c_int), ("out_height", C.c_int), ("out_width", C.c_int),
                ("kernel", C.c_int), ("stride", C.c_int), ("padding", C.c_int), ("batch_norm", C.c_int),
                ("activation", C.c_int), ("n_sources", C.c_int), ("sources", C.c_int * PLAN_MAX_SOURCES)]


class PlanDest(C.Structure):
    _fields_ = [("kind", C.c_int), ("route", C.c_int), ("channel_offset", C.c_int)]


class PlanStep(C.Structure):
    """pxe_step of include/pxe_plan.h."""
    _fields_ = [("op", C.c_int), ("layer", C.c_int), ("n_inputs", C.c_int), ("inputs", C.c_int * 2),
                ("n_dests", C.c_int), ("dests", PlanDest * PLAN_MAX_DESTS),
                ("fused_shortcut", C.c_int), ("fused_pool", C.c_int), ("keep_full", C.c_int),
                ("n_pool_dests", C.c_int), ("pool_dests", PlanDest * PLAN_MAX_DESTS), ("head_raw", C.c_int),
                ("n_spp", C.c_int), ("spp_layers", C.c_int * PLAN_MAX_SPP), ("n_spp_dests", C.c_int * PLAN_MAX_SPP),
                ("spp_dests", (PlanDest * PLAN_MAX_DESTS) * PLAN_MAX_SPP)]


class PlanStats(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("fused_shortcut", "fused_pool", "routes_eliminated", "routes_aliased",
                                       "spp_blocks", "raw_heads", "concat_copies")]


# name -> (restype, argtypes); every name here must be declared in include/pxe.h
_vp, _ll, _i, _f, _sz = C.c_void_p, C.c_longlong, C.c_int, C.c_float, C.c_size_t
PROTOTYPES = {
    "pxe_version": (_i, []),
    "pxe_last_error_string": (C.c_char_p, []),
    "pxe_status_string": (C.c_char_p, [_i]),
    "pxe_conv_epilogue": (_i, [_vp, C.POINTER(EpilogueDesc)]),
    "pxe_activate": (_i, [_vp, _i, _vp, _sz]),
    "pxe_add_bias": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "pxe_maxpool": (_i, [_vp, _vp, _ll, _vp, _ll, _vp, _i, _i, _i, _i, _i, _i, _i]),
    "pxe_maxpool_out_dim": (_i, [_i, _i, _i, _i]),
    "pxe_spp": (_i, [_vp, _vp, _ll, _i, _i, _i, _i, _i, C.POINTER(_i), C.POINTER(_vp), C.POINTER(_ll)]),
    "pxe_spp_epilogue": (_i, [_vp, _vp, _ll, _i, _i, _i, _i, _vp, _vp, _i, _vp, _ll, _i, C.POINTER(_i), C.POINTER(_vp),
                              C.POINTER(_ll)]),
    "pxe_upsample": (_i, [_vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _i, _f]),
    "pxe_shortcut": (_i, [_vp, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _f, _f, _i]),
    "pxe_shortcut_general": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _i, _i, _f, _f, _vp]),
    "pxe_concat": (_i, [_vp, _i, C.POINTER(_vp), C.POINTER(_ll), C.POINTER(_i), _vp, _ll, _i, _i, _i]),
    "pxe_yolo_activate": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "pxe_yolo_decode_workspace_bytes": (_sz, [_i, _i, _i]),
    "pxe_yolo_decode_fast_workspace_bytes": (_sz, [_i, _i, _i]),
    "pxe_yolo_decode": (_i, [_vp, C.POINTER(YoloDecodeDesc), _vp, _ll, _vp, _vp, _sz]),
    "pxe_yolo_decode_static": (_i, [_vp, C.POINTER(YoloDecodeDesc), _vp, _ll, _vp]),
    "pxe_centernet_activate": (_i, [_vp, _vp, _vp, _i, _i, _i, _f]),
    "pxe_centernet_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "pxe_centernet_decode": (_i, [_vp, C.POINTER(CenterNetDecodeDesc), _vp, _vp, _vp, _sz]),
    "pxe_softmax": (_i, [_vp, _vp, _vp, _i, _i, _i, _f]),
    "pxe_region_forward": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i]),
    "pxe_conv_stem": (_i, [_vp, C.POINTER(StemDesc)]),
    "pxe_fold_bn": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _vp, _vp]),
    "pxe_conv_epilogue_nhwc": (_i, [_vp, C.POINTER(EpilogueNhwcDesc)]),
    "pxe_upsample_nhwc": (_i, [_vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _i, _f]),
    "pxe_maxpool_nhwc": (_i, [_vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _i, _i, _i]),
    "pxe_nhwc_to_nchw": (_i, [_vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i]),
    "pxe_avgpool": (_i, [_vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i]),
    "pxe_detect_decode": (_i, [_vp, _vp, _ll, _i, _i, _i, _i, _i, _i, _f, _f, _f, _vp, _ll, _vp, _i]),
    "pxe_softmax_decode": (_i, [_vp, _vp, _ll, _i, _i, _f, _f, _f, _vp, _ll, _vp, _i]),
    "pxe_region_decode": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, C.POINTER(C.c_float), _i, _f, _f, _f, _vp, _ll, _vp, _i]),
    "pxe_nms_host": (_ll, [_vp, _ll, _f, _vp]),
    "pxe_nms_workspace_bytes": (_sz, [_ll]),
    "pxe_nms": (_i, [_vp, _vp, _ll, _f, _vp, _vp, _vp, _sz]),
    "pxe_activation_gradient": (_i, [_vp, _i, _vp, _sz, _vp]),
    "pxe_backward_bias": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "pxe_maxpool_backward": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "pxe_upsample_backward": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f]),
    "pxe_constrain": (_i, [_vp, _vp, _sz, _f]),
    "pxe_mul": (_i, [_vp, _vp, _vp, _sz]),
    "pxe_random_uniform": (_i, [_vp, _vp, _sz, _f, _f]),
    "pxe_random_normal": (_i, [_vp, _vp, _sz, _f, _f]),
    "pxe_yolo_loss": (_i, [_vp, C.POINTER(YoloLossDesc)]),
    "pxe_centernet_loss": (_i, [_vp] + [_vp] * 7 + [_i] * 3 + [_f] * 4),
    "pxe_adam_update": (_i, [_vp, C.c_size_t, _vp, _vp, _vp, _f, _f, _f, _f, _i]),
    "pxe_softmax_cross_entropy": (_i, [_vp, C.c_size_t, _vp, _vp, _vp, _vp]),
    "pxe_batchnorm_workspace_bytes": (C.c_size_t, [_i] * 4),
    "pxe_batchnorm_forward_training": (_i, [_vp, C.POINTER(BnTrainDesc)]),
    "pxe_batchnorm_backward": (_i, [_vp, C.POINTER(BnBackwardDesc)]),
}

# the planner of include/pxe_plan.h (host code)
PLAN_PROTOTYPES = {
    "pxe_plan_build": (_i, [C.POINTER(LayerDesc), _i, _i, _i, C.POINTER(_vp)]),
    "pxe_plan_destroy": (None, [_vp]),
    "pxe_plan_step_count": (_i, [_vp]),
    "pxe_plan_step": (C.POINTER(PlanStep), [_vp, _i]),
    "pxe_plan_alias": (_i, [_vp, _i]),
    "pxe_plan_concat_channels": (_i, [_vp, _i]),
    "pxe_plan_last_use": (_i, [_vp, _i]),
    "pxe_plan_get_stats": (None, [_vp, C.POINTER(PlanStats)]),
}

# mangled names of the link-compatible tier (include/pxe_compat.hpp)
COMPAT_SYMBOLS = [
    "_ZN2px8activateE14ActivationTypePfm",
    "_ZN2px10addBiasGpuEPfPKfiii",
    "_ZN2px17maxPoolForwardGpuEPKfPfPiiiiiiiiii",
    "_ZN2px11upsampleGpuEPKfiiiiiifPfS2_",
    "_ZN2px11shortcutGpuEiiiiPKfiiiffPf",
    "_ZN2px15yoloActivateGpuEPKfPfiiii",
    "_ZN2px20centerNetActivateGpuEPKfPfiiif",
    "_ZN2px7fillGpuEPfmf",
    "_ZN2px7fillGpuEPimi",
    "_ZN2px8gradientE14ActivationTypePKfmPf",
    "_ZN2px15backwardBiasGpuEPfPKfiii",
    "_ZN2px18maxPoolBackwardGpuEPKfPKiPfi",
    "_ZN2px12constrainGpuEifPf",
    "_ZN2px12cudaGridsizeEj",
    "_ZN2px6mulGpuEiPfS0_",
    "_ZN2px9randomGpuEPfmff",
    "_ZN2px15randomNormalGpuEPfmff",
    "_ZN2px11yoloLossGpuEPKfPfS1_PKiiS4_S4_S1_S4_S1_S2_S2_iiiiiiiiffffff",
    "_ZN2px16centerNetLossGpuEPKfPfS1_S1_S1_S1_S2_iiiffff",
    "_ZN2px7adamGpuEiPfS0_S0_ffffi",
    "_ZN2px19softmaxCrossEntropyEiPKfS1_PfS2_",
]

class BoundsReport(C.Structure):
    """pxe_bounds_report of include/pxe_debug.h."""
    _fields_ = [("violations", C.c_uint), ("bytes", C.c_int), ("address", C.c_ulonglong), ("line", C.c_int),
                ("is_store", C.c_int), ("misaligned", C.c_int), ("reserved", C.c_int), ("file", C.c_char * 48)]


# include/pxe_debug.h: present in both builds of the library
DEBUG_PROTOTYPES = {
    "pxe_debug_bounds_checked": (C.c_int, []),
    "pxe_debug_set_allocations": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), C.c_int]),
    "pxe_debug_read_report": (C.c_int, [C.POINTER(BoundsReport), C.c_int]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (run ``python -m pixienn_b200._build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m pixienn_b200._build` "
                "(needs nvcc); there is no fallback implementation")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in list(PROTOTYPES.items()) + list(PLAN_PROTOTYPES.items()) + list(DEBUG_PROTOTYPES.items()):
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != PXE_OK:
        raise PxeError(status, lib().pxe_last_error_string().decode(errors="replace"))
