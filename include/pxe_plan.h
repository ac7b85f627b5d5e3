/* pxe_plan.h -- the fusion plan of the epilogue path, built once per model.
 *
 * The reference decides nothing ahead of time: Model<D>::forward (include/Model.h:1748-1756) walks
 * the layers in index order and every layer runs its own passes (conv epilogue, then the maxpool /
 * shortcut / route layer that follows as separate full-tensor launches and copies).  Cross-layer
 * fusion needs one object that knows the whole graph: which conv epilogue absorbs the shortcut
 * (include/cuda/ShortcutLayer.h:23-34) or the 2x2 stride-2 max pool (include/cuda/MaxPoolLayer.h:36-42)
 * that follows it, which producers store straight into a route's concat buffer
 * (include/cuda/RouteLayer.h:21-44) so that the route runs nothing, which stride-1 pools form an SPP
 * block that reads its input once, and which YOLO heads are decoded from the raw conv output
 * (include/cuda/YoloLayer.h:70-96, 168-188).
 *
 * A caller describes its layers (after shape propagation, as Model<D>::parseModel leaves them,
 * include/Model.h:1596-1641) with pxe_layer_desc records, builds the plan once, and consults it in
 * each layer's forward: the step of a layer says which libpxe call to make and where its output
 * goes.  Host code only; no CUDA call is made here.
 *
 * There is no counterpart in the reference: this header is the additive piece a maintainer adds
 * next to Model.h.
 */
#ifndef PXE_PLAN_H
#define PXE_PLAN_H

#include "pxe.h"   /* PXE_API, status codes, PXE_ACT_* */

#ifdef __cplusplus
extern "C" {
#endif

#define PXE_PLAN_MAX_SOURCES 16   /* fan-in of a route layer */
#define PXE_PLAN_MAX_DESTS 8      /* one dense tensor + the concat slots a tensor is stored into */
#define PXE_PLAN_MAX_SPP 4        /* stride-1 pools read in one pass */

/* layer types, in the reference's YAML vocabulary (include/Model.h:1596-1641) */
enum {
    PXE_LAYER_CONV = 0,
    PXE_LAYER_MAXPOOL = 1,
    PXE_LAYER_UPSAMPLE = 2,
    PXE_LAYER_ROUTE = 3,
    PXE_LAYER_SHORTCUT = 4,
    PXE_LAYER_YOLO = 5,
    PXE_LAYER_CENTERNET = 6,
    PXE_LAYER_REGION = 7,
    PXE_LAYER_SOFTMAX = 8,
    PXE_LAYER_AVGPOOL = 9,
    PXE_LAYER_DROPOUT = 10,
    PXE_LAYER_CONNECTED = 11,
    PXE_LAYER_DETECTION = 12      /* the YOLOv1 head, `type: detection` */
};

/* step operations */
enum {
    PXE_STEP_CONV = 0,       /* convolution + pxe_conv_epilogue (with the fusions named in the step) */
    PXE_STEP_ALIAS = 1,      /* nothing runs: the layer's output is another tensor / an already filled concat buffer */
    PXE_STEP_MAXPOOL = 2,    /* pxe_maxpool */
    PXE_STEP_SPP = 3,        /* pxe_spp over spp_layers */
    PXE_STEP_UPSAMPLE = 4,   /* pxe_upsample */
    PXE_STEP_SHORTCUT = 5,   /* pxe_shortcut (a shortcut that could not be folded into a conv) */
    PXE_STEP_CONCAT = 6,     /* pxe_concat (unfused plans only) */
    PXE_STEP_HEAD = 7        /* yolo / centernet / region / softmax / avgpool / dropout / connected / detection: see layer type */
};

typedef struct pxe_layer_desc {
    int type;                              /* PXE_LAYER_* */
    int out_channels, out_height, out_width;
    int kernel, stride, padding;           /* conv, maxpool (padding as the layer stores it: total padding for maxpool) */
    int batch_norm;                        /* conv: non-zero when followed by batch normalisation */
    int activation;                        /* conv, shortcut: PXE_ACT_* of pxe.h */
    int n_sources;                         /* 1 for most layers; 2 for shortcut (previous, from); fan-in for route */
    int sources[PXE_PLAN_MAX_SOURCES];     /* absolute layer indices; -1 = the network input */
} pxe_layer_desc;

typedef struct pxe_dest {
    int kind;                              /* 0: a dense tensor of the layer's own; 1: a channel slot of a concat buffer */
    int route;                             /* kind 1: the route layer that owns the concat buffer */
    int channel_offset;                    /* kind 1: first channel of the slot */
} pxe_dest;

typedef struct pxe_step {
    int op;                                /* PXE_STEP_* */
    int layer;                             /* the layer whose output this step produces (SPP: the first pool) */
    int n_inputs;
    int inputs[2];                         /* tensors read (layer indices, aliases resolved); conv + fused shortcut: {input, from} */
    int n_dests;
    pxe_dest dests[PXE_PLAN_MAX_DESTS];    /* where the (full-resolution) output is stored; dests beyond the second need pxe_concat */
    int fused_shortcut;                    /* conv: index of the shortcut layer folded into the epilogue, or -1 */
    int fused_pool;                        /* conv: index of the maxpool layer folded into the epilogue, or -1 */
    int keep_full;                         /* with fused_pool: is the full-resolution output needed as well */
    int n_pool_dests;
    pxe_dest pool_dests[PXE_PLAN_MAX_DESTS];
    int head_raw;                          /* conv: skip the epilogue; yolo: decode the raw conv output (bias + logistic inside the decode) */
    int n_spp;
    int spp_layers[PXE_PLAN_MAX_SPP];
    int n_spp_dests[PXE_PLAN_MAX_SPP];
    pxe_dest spp_dests[PXE_PLAN_MAX_SPP][PXE_PLAN_MAX_DESTS];
} pxe_step;

typedef struct pxe_plan_stats {
    int fused_shortcut, fused_pool, routes_eliminated, routes_aliased, spp_blocks, raw_heads, concat_copies;
} pxe_plan_stats;

typedef struct pxe_plan pxe_plan;

/* Builds the plan.  fuse = 0 gives the layer-by-layer schedule (one step per layer, every route a real
 * copy), used as the unfused comparison.  raw_heads = 0 keeps the epilogue of convs that feed a YOLO layer.
 * Returns a pxe.h status code; on success *out owns the plan until pxe_plan_destroy. */
PXE_API int pxe_plan_build(const pxe_layer_desc* layers, int n_layers, int fuse, int raw_heads, pxe_plan** out);
PXE_API void pxe_plan_destroy(pxe_plan* plan);

PXE_API int pxe_plan_step_count(const pxe_plan* plan);
/* Step i in execution order, or NULL when i is out of range.  The pointer stays valid until destroy. */
PXE_API const pxe_step* pxe_plan_step(const pxe_plan* plan, int i);
/* The layer whose tensor `layer` shares (fan-in-1 routes, convs folded into their shortcut), or -1. */
PXE_API int pxe_plan_alias(const pxe_plan* plan, int layer);
/* Total channels of the concat buffer owned by route layer `route`, or 0 when the route owns none. */
PXE_API int pxe_plan_concat_channels(const pxe_plan* plan, int route);
/* Index of the last step that reads tensor `layer`, or -1: its buffer may be released after that step. */
PXE_API int pxe_plan_last_use(const pxe_plan* plan, int layer);
PXE_API void pxe_plan_get_stats(const pxe_plan* plan, pxe_plan_stats* stats);

#ifdef __cplusplus
}
#endif
#endif /* PXE_PLAN_H */
