/*
 * pxe.h -- C ABI of the B200 (sm_100a) epilogue kernels for PixieNN.
 *
 * Every entry point replaces one step that PixieNN's CUDA layers run between
 * convolutions.  The comment above each declaration names the reference call
 * site(s) it stands in for, by path inside the trieck/pixienn tree.
 *
 * Conventions
 *  - All tensors are fp32, NCHW.  A "batch stride" is the distance in ELEMENTS
 *    between consecutive images of a tensor; 0 means "densely packed"
 *    (channels*height*width).  A non-dense stride lets a kernel read from or
 *    write into a channel slot of a wider concat buffer, which is how route
 *    (concat) layers are eliminated.
 *  - The caller owns every buffer.  No entry point allocates or frees device
 *    memory, and none synchronises: work is enqueued on `stream` (0 = the
 *    legacy default stream the reference uses everywhere).
 *  - Every entry point returns PXE_OK (0) or an error code, validates its
 *    arguments before launching anything, never throws and never aborts.
 *    pxe_last_error_string() returns the message of the calling thread's most
 *    recent failure.
 *  - Functions are re-entrant; there is no global mutable state apart from a
 *    per-device cache of immutable device properties (and, for
 *    pxe_yolo_decode_static only, the shared scratch array its comment describes).
 */
#ifndef PXE_H
#define PXE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define PXE_API
#else
#define PXE_API __attribute__((visibility("default")))
#endif

typedef void* pxe_stream_t;   /* a cudaStream_t */

enum pxe_status {
    PXE_OK = 0,
    PXE_ERR_BAD_ARG = 1,       /* null pointer, non-positive size, misaligned or overlapping buffer */
    PXE_ERR_UNSUPPORTED = 2,   /* valid request this build has no kernel for */
    PXE_ERR_CUDA = 3,          /* a CUDA runtime call failed; see pxe_last_error_string() */
    PXE_ERR_WORKSPACE = 4      /* caller-provided workspace is too small */
};

/* Same values as the reference's ActivationType (include/ActivationTypes.h:19-30). */
enum pxe_activation {
    PXE_ACT_LEAKY = 0,      /* x > 0 ? x : 0.1 x   (slope fixed, include/Activation.h:45) */
    PXE_ACT_LINEAR = 1,
    PXE_ACT_LOGGY = 2,
    PXE_ACT_LOGISTIC = 3,
    PXE_ACT_MISH = 4,
    PXE_ACT_RELU = 5,
    PXE_ACT_SOFTPLUS = 6,
    PXE_ACT_SWISH = 7,      /* beta fixed to 1, include/Activation.h:195 */
    PXE_ACT_TANH = 8,
    /* Not a reference activation: the YOLO head's per-entry rule (logistic on x, y,
     * objectness and class entries, identity on w, h) so that bias add and
     * yoloActivateGpu run as one pass.  Needs pxe_epilogue_desc.yolo_classes. */
    PXE_ACT_YOLO_HEAD = 100
};

/* How epsilon enters the batch-norm denominator. */
enum pxe_bn_eps_mode {
    PXE_BN_EPS_CUDNN = 0,   /* sqrt(var + eps): cudnnBatchNormalizationForwardInference, the CUDA path */
    PXE_BN_EPS_CPU = 1      /* sqrt(var) + eps: normalizeCpu, src/CpuUtil.cpp:288 */
};

/* One detection, the fields of px::Detection (include/Detection.h:23-40) plus the emitting slot. */
typedef struct pxe_detection {
    float x, y, w, h;       /* cv::Rect2f: left, top, width, height */
    float prob;
    int32_t class_id;
    int32_t batch_id;
    int32_t source;         /* YOLO: cell*masks + mask slot; CenterNet: (class*H + y)*W + x;
                               Region: cell*num + n; Softmax: class */
} pxe_detection;

PXE_API int pxe_version(void);
PXE_API const char* pxe_last_error_string(void);
PXE_API const char* pxe_status_string(int status);

/* ------------------------------------------------------------------------------------------
 * Fused convolution epilogue.
 *
 * Replaces, in one pass over the conv output, the sequence in
 * ConvLayer<Device::CUDA>::forward (include/cuda/ConvLayer.h:284-307):
 *   cudnnBatchNormalizationForwardInference (eps 1e-5)  OR  addBiasGpu (src/BiasKernels.cu:86-93),
 *   the preActivation_ device copy (skipped: inference never reads it),
 *   activation_->apply == px::activate (src/Activation.cu:126-133),
 * and, when requested, the layers that follow it in the graph:
 *   ShortcutLayer<CUDA>::forward (include/cuda/ShortcutLayer.h:23-34): residual add + activation,
 *   MaxPoolLayer<CUDA>::forward  (include/cuda/MaxPoolLayer.h:36-42) for kernel 2 / stride 2,
 *   RouteLayer<CUDA>::forward    (include/cuda/RouteLayer.h:21-44): the result is stored straight
 *                                into its slot of the concat buffer (y or y2 with a batch stride),
 *   yoloActivateGpu              (src/YoloKernels.cu:216-221) via PXE_ACT_YOLO_HEAD.
 *
 * v = x; if gamma: v = gamma*(v-mean)/denom(var,eps) + beta; if bias: v += bias; v = act(v);
 * if residual: v = res_act(res_alpha*v + res_beta*residual);
 * y (and y2) receive v; y_pool receives the 2x2/stride-2 max of v (window origin
 * -pool_padding/2 == 0, out-of-range taps skipped, first maximum wins).
 * ------------------------------------------------------------------------------------------ */
typedef struct pxe_epilogue_desc {
    const float* x;             /* conv output [batch, channels, height, width] */
    long long x_batch_stride;
    float* y;                   /* destination; may equal x (in place).  May be NULL only when y_pool is set */
    long long y_batch_stride;
    float* y2;                  /* optional second destination (e.g. a concat slot), or NULL */
    long long y2_batch_stride;
    int batch, channels, height, width;

    const float* gamma;         /* scales_;      NULL = no batch norm */
    const float* beta;          /* biases_ (BN shift) */
    const float* mean;          /* rollingMean_ */
    const float* var;           /* rollingVar_ */
    float eps;                  /* the reference passes 1e-5 */
    int eps_mode;               /* enum pxe_bn_eps_mode */
    const float* bias;          /* per-channel bias added after BN, or the conv bias when gamma is NULL; may be NULL */
    int act;                    /* enum pxe_activation */
    int yolo_classes;           /* PXE_ACT_YOLO_HEAD only: channels % (yolo_classes + 5) must be 0 */

    const float* residual;      /* from_->output() of a following shortcut layer, or NULL */
    long long residual_batch_stride;
    float res_alpha, res_beta;  /* ShortcutLayer alpha_, beta_ (include/ShortcutLayer.h:51-52) */
    int res_act;                /* the shortcut layer's activation */

    int pool_kernel;            /* 0 = no pooling; otherwise must be 2 */
    int pool_stride;            /* must be 2 */
    int pool_padding;           /* 0 or 1 (the MaxPoolLayer default is kernel-1 = 1) */
    float* y_pool;              /* [batch, channels, OH, OW], OH = (height + pad - 2)/2 + 1 */
    long long y_pool_batch_stride;
    int pool_variant;           /* 0: the library picks the pooled kernel for the shape (what callers want);
                                   PXE_POOL_GENERAL: always the general pooled kernel -- the specialised forms
                                   (even heights, small odd planes) must equal it bit for bit, which is how
                                   the tests hold them to it */
    const float* folded_a;      /* optional: a[c], b[c] of y = act(a * x + b), folded once per layer by pxe_fold_bn from */
    const float* folded_b;      /* the same gamma / beta / mean / var / bias (which are then ignored).  Same results bit
                                   for bit; the kernels then build no per-block coefficient table and meet no barrier,
                                   which is what tensors under about 200 MB spend a visible share of a launch on */
} pxe_epilogue_desc;

enum pxe_pool_variant { PXE_POOL_AUTO = 0, PXE_POOL_GENERAL = 1 };

PXE_API int pxe_conv_epilogue(pxe_stream_t stream, const pxe_epilogue_desc* desc);

/* px::activate(type, x, n), include/Activation.cuh:26 / src/Activation.cu:126-133: in-place activation. */
PXE_API int pxe_activate(pxe_stream_t stream, int act, float* x, size_t n);

/* px::addBiasGpu, include/BiasKernels.cuh:21 / src/BiasKernels.cu:86-93: out[b, j, :] += bias[j]. */
PXE_API int pxe_add_bias(pxe_stream_t stream, float* out, const float* bias, int batch, int n, int size);

/* ------------------------------------------------------------------------------------------
 * Max pooling: px::maxPoolForwardGpu (include/MaxPoolKernels.cuh:5, src/MaxPoolKernels.cu:10-59).
 * Output extent (in + padding - kernel)/stride + 1 (include/MaxPoolLayer.h:61-62), window origin
 * -padding/2 with C truncation, out-of-range taps skipped, first maximum wins.  `indexes`
 * (int32 flat index into a DENSE input tensor, -1 for an empty window) may be NULL.
 * ------------------------------------------------------------------------------------------ */
PXE_API int pxe_maxpool(pxe_stream_t stream, const float* x, long long x_batch_stride, float* y,
                        long long y_batch_stride, int* indexes, int batch, int channels, int height,
                        int width, int kernel, int stride, int padding);
PXE_API int pxe_maxpool_out_dim(int in, int kernel, int stride, int padding);

/* SPP block: several stride-1 max pools of the SAME input (e.g. kernels 5, 9, 13 with the default
 * padding kernel-1), each written to its own destination, in one launch that reads the input once.
 * Stands in for consecutive MaxPoolLayer<CUDA>::forward calls joined by route layers. */
PXE_API int pxe_spp(pxe_stream_t stream, const float* x, long long x_batch_stride, int batch, int channels,
                    int height, int width, int n_pools, const int* kernels, float* const* ys,
                    const long long* y_batch_strides);

/* The conv epilogue folded into the SPP block that follows it (ConvLayer<CUDA>::forward lines
 * include/cuda/ConvLayer.h:284-307, then the MaxPoolLayer<CUDA>::forward calls of the block,
 * include/cuda/MaxPoolLayer.h:36-42, and the route that concatenates them, include/cuda/RouteLayer.h:21-44):
 * x is the RAW convolution output; v = act(a[c] * x + b[c]) (a, b: the table of pxe_fold_bn, or NULL for
 * the activation alone) is computed once while the plane is staged, stored to y_identity (the block's
 * pass-through slot; may be NULL) and pooled with every kernel size.  One read of the conv output instead of
 * an epilogue pass plus the SPP's read.  Values equal pxe_conv_epilogue followed by pxe_spp bit for bit.
 * PXE_ERR_UNSUPPORTED when a plane (2 * height * width floats) does not fit shared memory. */
PXE_API int pxe_spp_epilogue(pxe_stream_t stream, const float* x, long long x_batch_stride, int batch, int channels,
                             int height, int width, const float* a, const float* b, int act, float* y_identity,
                             long long y_identity_batch_stride, int n_pools, const int* kernels, float* const* ys,
                             const long long* y_batch_strides);

/* px::upsampleGpu forward (include/UpsampleKernels.cuh:21, src/UpsampleKernels.cu:25-63):
 * nearest-neighbour x stride, y = scale * x (assigned, as the CPU layer does). */
PXE_API int pxe_upsample(pxe_stream_t stream, const float* x, long long x_batch_stride, float* y,
                         long long y_batch_stride, int batch, int channels, int height, int width,
                         int stride, float scale);

/* ShortcutLayer<CUDA>::forward (include/cuda/ShortcutLayer.h:23-34) for equal shapes:
 * y = act(alpha * x + beta * from).  y may alias x. */
PXE_API int pxe_shortcut(pxe_stream_t stream, const float* x, long long x_batch_stride, const float* from,
                         long long from_batch_stride, float* y, long long y_batch_stride, float* y2,
                         long long y2_batch_stride, int batch, int channels, int height, int width,
                         float alpha, float beta, int act);

/* px::shortcutGpu (include/ShortcutKernel.cuh:21, src/ShortcutKernel.cu:25-66), any shapes:
 * out = s1 * out + s2 * add with the reference's stride/sample index rule. */
PXE_API int pxe_shortcut_general(pxe_stream_t stream, int batch, int w1, int h1, int c1, const float* add,
                                 int w2, int h2, int c2, float s1, float s2, float* out);

/* RouteLayer<CUDA>::forward (include/cuda/RouteLayer.h:21-44) as one launch instead of
 * batch x fan-in blocking copies.  Source s is [batch, src_channels[s], height, width] with its own
 * batch stride; it lands at channel offset sum(src_channels[0..s)) of y.  n_src <= 8. */
PXE_API int pxe_concat(pxe_stream_t stream, int n_src, const float* const* srcs,
                       const long long* src_batch_strides, const int* src_channels, float* y,
                       long long y_batch_stride, int batch, int height, int width);

/* ------------------------------------------------------------------------------------------
 * YOLO head
 * ------------------------------------------------------------------------------------------ */
/* px::yoloActivateGpu (include/YoloKernels.cuh:7, src/YoloKernels.cu:63-71, 216-221). */
PXE_API int pxe_yolo_activate(pxe_stream_t stream, const float* in, float* out, int batch, int masks,
                              int classes, int area);

typedef struct pxe_yolo_decode_desc {
    const float* head;          /* [batch, masks*(5+classes), height, width] (or channels last, see below) */
    long long head_batch_stride;
    int head_is_raw;            /* 0: already activated (YoloLayer output_); 1: raw conv output,
                                   the decode applies `bias` and the head's logistic rule itself */
    const float* bias;          /* per-channel conv bias for head_is_raw, or NULL */
    int batch, height, width;
    int classes;
    int n_masks;                /* <= 16 */
    int mask[16];               /* YoloLayer mask_ */
    int n_anchor_values;        /* 2*num, <= 64 */
    int anchors[64];            /* YoloLayer anchors_, ints as the reference parses them (include/YoloLayer.h:93) */
    int net_width, net_height;  /* model().width(), model().height() */
    int image_width, image_height;  /* > 0: scaledYoloBox (letterbox-corrected integer pixel boxes,
                                       include/YoloLayer.h:601-635); 0: normalised yoloBox().rect() */
    float threshold;
    int batch_id_offset;        /* added to batch_id (batch-sharded multi-GPU runs) */
    int head_channels_last;     /* 1: `head` is [batch, height, width, masks*(5+classes)] (the channels-last tier's
                                   conv output, no transposition first); same records in the same order */
} pxe_yolo_decode_desc;

/* Bytes of device workspace pxe_yolo_decode needs for this head (12 bytes per 32 cells per image). */
PXE_API size_t pxe_yolo_decode_workspace_bytes(int batch, int height, int width);
/* With this many bytes (about 2 KB per 32 cells per image more) the decode's first pass leaves, per box slot and
 * class chunk, a mask of the classes that reached the threshold, and the second pass evaluates only those: one
 * logistic per emitted value, and no second read of the head where nothing is emitted.  Same records either way. */
PXE_API size_t pxe_yolo_decode_fast_workspace_bytes(int batch, int height, int width);

/*
 * YoloLayer<CUDA>::addDetects (include/cuda/YoloLayer.h:168-188 -> include/YoloLayer.h:659-698):
 * threshold on objectness, box decode, per-class probability, on the device instead of a
 * full-tensor device-to-host copy and a host loop.  Records are appended to `dets` starting at
 * position *count (a device counter the caller zeroes once per forward) in exactly the
 * reference's emission order (image, cell, mask slot, class), so chaining the heads in layer order
 * reproduces Model::detections().  *count keeps counting past `capacity`; records beyond it are
 * dropped, so count > capacity tells the caller to retry with more room.
 */
PXE_API int pxe_yolo_decode(pxe_stream_t stream, const pxe_yolo_decode_desc* desc, pxe_detection* dets,
                            long long capacity, long long* count, void* workspace,
                            size_t workspace_bytes);

/*
 * pxe_yolo_decode with no workspace argument.  This entry point has no counterpart in the
 * reference; it exists for callers that have no way to obtain device memory at the point where
 * they decode: PixieNN's own addDetects runs inside Model::detections(), a per-frame call on
 * objects that are not meant to grow there, and a host application that handed the engine a fixed
 * memory budget at start-up (or forbids allocation once its real-time loop runs, since cudaMalloc
 * stalls the whole device) cannot satisfy a "bring a scratch buffer" contract either.
 *
 * The scratch lives in a fixed array inside the library (PXE_YOLO_DECODE_STATIC_SCRATCH_BYTES,
 * resident on every GPU that loads the library for the life of the process).  A head whose
 * pxe_yolo_decode_workspace_bytes() exceeds that size is refused with PXE_ERR_WORKSPACE; the
 * decode needs 12 bytes per 32 cells per image, so 4 MiB covers e.g. 64 images of a 76x76 head
 * (140 KB) many times over.  Nothing is allocated or freed, by this function or by anything it calls.
 *
 * - The first call on each device looks up the array's device address (that device must be
 *   current); make that first call before starting any stream capture.
 * - All calls on a device share the one array.  The decode overwrites every scratch word it later
 *   reads, so leftovers of an earlier call are harmless, but two decodes that may run at the same
 *   time on the GPU (different streams) would corrupt each other: serialise them, or give the
 *   concurrent ones their own workspace through pxe_yolo_decode.
 */
#define PXE_YOLO_DECODE_STATIC_SCRATCH_BYTES (4u << 20)
PXE_API int pxe_yolo_decode_static(pxe_stream_t stream, const pxe_yolo_decode_desc* desc, pxe_detection* dets,
                                   long long capacity, long long* count);

/* ------------------------------------------------------------------------------------------
 * CenterNet head
 * ------------------------------------------------------------------------------------------ */
/* px::centerNetActivateGpu (include/CenterNetKernels.cuh:5, src/CenterNetKernels.cu:9-18, 110-118). */
PXE_API int pxe_centernet_activate(pxe_stream_t stream, const float* in, float* out, int batch, int classes,
                                   int area, float heatmap_bias);

typedef struct pxe_centernet_decode_desc {
    const float* heat;          /* [batch, classes, height, width] heatmap */
    long long heat_batch_stride;
    const float* size;          /* [batch, 2, height, width]: box width, height in cells */
    long long size_batch_stride;
    const float* offset;        /* [batch, 2, height, width]: centre offset x, y */
    long long offset_batch_stride;
    int heat_is_logit;          /* 1: heat holds logits, sigmoid(heat + heatmap_bias) is applied here;
                                   0: heat is already activated (CenterNetLayer output_) */
    float heatmap_bias;
    int batch, classes, height, width;
    int image_width, image_height;   /* <= 0 means 1 (normalised boxes) */
    float threshold;
    int max_detections;         /* CenterNetLayer max_detections (default 100), <= 1024 */
    int batch_id_offset;
    int candidate_capacity;     /* 0 = default.  Local maxima one image may list before it is redone by the
                                   tile-by-tile pass, which reduces every tile to its best max_detections (the
                                   result is the same either way; a heat map with plateaus, where every cell is a
                                   maximum, is the case that overflows).  Values below tiles x classes x
                                   max_detections are raised to that; values above the default are refused. */
} pxe_centernet_decode_desc;

PXE_API size_t pxe_centernet_decode_workspace_bytes(int batch, int classes, int height, int width,
                                                    int max_detections);

/*
 * CenterNetLayer<CUDA>::addDetects (include/cuda/CenterNetLayer.h:89-106 ->
 * include/CenterNetLayer.h:181-247): 3x3 strict local-maximum test on the activated scores,
 * threshold, validity of size/offset, box rebuild, and the max_detections best per image ordered
 * by score descending with ties to the lower flat index (class*H + y)*W + x.
 * dets holds batch*max_detections records (image b at dets + b*max_detections); counts[b]
 * receives the number of valid records of image b.
 */
PXE_API int pxe_centernet_decode(pxe_stream_t stream, const pxe_centernet_decode_desc* desc,
                                 pxe_detection* dets, int* counts, void* workspace,
                                 size_t workspace_bytes);

/* ------------------------------------------------------------------------------------------
 * Softmax and Region heads
 * ------------------------------------------------------------------------------------------ */
/* SoftmaxLayer forward.  CPU semantics (include/SoftmaxLayer.h:86-99, src/Math.cpp:77-108):
 * each image's `inputs` values are split into `groups` contiguous groups, softmax with
 * temperature inside each.  The CUDA layer's cudnnSoftmaxForward(MODE_CHANNEL)
 * (include/cuda/SoftmaxLayer.h:67-85) equals groups = 1, temperature = 1 when height*width == 1. */
PXE_API int pxe_softmax(pxe_stream_t stream, const float* in, float* out, int batch, int inputs, int groups,
                        float temperature);

/* RegionLayer forward, inference part (include/RegionLayer.h:271-300), replacing the
 * device->host->device round trip of include/cuda/RegionLayer.h:39-54: NCHW ->
 * [cell*num + n][coords+1+classes] transpose (flatten, src/CpuUtil.cpp:364-384), logistic on the
 * objectness entry, optional softmax over each box's classes.  in != out. */
PXE_API int pxe_region_forward(pxe_stream_t stream, const float* in, float* out, int batch, int width,
                               int height, int num, int coords, int classes, int softmax);

/* ------------------------------------------------------------------------------------------
 * Channels-last (NHWC) tier.  The reference describes every tensor to cuDNN as NCHW
 * (include/Cudnn.h:103-108; include/cuda/ConvLayer.h:278-283), and cuDNN then converts to and from the NHWC
 * layout of its tensor-core kernels around every convolution.  A caller that sets its descriptors to
 * CUDNN_TENSOR_NHWC (and stores its filters that way) avoids those conversions; these entry points are the
 * epilogue path for such tensors.  Element (image b, row r, column c, channel k) of a tensor lives at
 * ((b*H + r)*W + c) * pixel_stride + k; pixel_stride is the channel count of the buffer the tensor lives in
 * (0 = the tensor's own channel count), so a channel slot of a route's concat buffer is a tensor with a
 * larger pixel stride and a pointer advanced by the slot's first channel.
 * ------------------------------------------------------------------------------------------ */

/* Folds batch-norm inference and bias into y = a[k]*x + b[k] (include/cuda/ConvLayer.h:294-303;
 * CPU form src/BatchNorm.cpp:61-66 with eps_mode = PXE_BN_EPS_CPU): a = gamma / denom(var, eps),
 * b = beta - mean*a (+ bias).  gamma == NULL: a = 1, b = bias (or 0).  Run once per layer when the weights
 * are loaded; a, b: device arrays of `channels` floats. */
PXE_API int pxe_fold_bn(pxe_stream_t stream, const float* gamma, const float* beta, const float* mean,
                        const float* var, const float* bias, float eps, int eps_mode, int channels, float* a,
                        float* b);

typedef struct pxe_epilogue_nhwc_desc {
    const float* x;               /* conv output, NHWC */
    float* y;                     /* destination (may be x) */
    float* y2;                    /* optional second destination, e.g. a route slot */
    const float* residual;        /* optional: the `from` tensor of a following shortcut layer */
    long long x_pixel_stride, y_pixel_stride, y2_pixel_stride, residual_pixel_stride;   /* 0 = channels */
    long long pixels;             /* batch * height * width */
    int channels;
    const float* a;               /* folded coefficients from pxe_fold_bn, or NULL (with b) for none */
    const float* b;
    int act;                      /* pxe_activation */
    float res_alpha, res_beta;    /* y = res_act(res_alpha * act(a*x+b) + res_beta * residual) */
    int res_act;
    /* optional folded 2x2 stride-2 max pool (as in pxe_epilogue_desc): needs the geometry as well */
    int pool_kernel, pool_stride, pool_padding;   /* 0 = none; 2 / 2 / 0|1 */
    int batch, height, width;                     /* batch * height * width == pixels */
    float* y_pool;                                /* [batch, OH, OW, channels]; y may then be NULL */
    long long y_pool_pixel_stride;
} pxe_epilogue_nhwc_desc;

/* The fused conv epilogue of pxe_conv_epilogue for NHWC tensors; with a = b = NULL and act linear it is
 * the shortcut layer (include/cuda/ShortcutLayer.h:23-34) or a copy into a route slot. */
PXE_API int pxe_conv_epilogue_nhwc(pxe_stream_t stream, const pxe_epilogue_nhwc_desc* desc);

/* UpsampleLayer (src/UpsampleKernels.cu:25-63) and MaxPoolLayer (src/MaxPoolKernels.cu:10-43, values only)
 * for NHWC tensors; same geometry and tie rules as pxe_upsample / pxe_maxpool. */
PXE_API int pxe_upsample_nhwc(pxe_stream_t stream, const float* in, long long in_pixel_stride, float* out,
                              long long out_pixel_stride, int batch, int channels, int height, int width,
                              int stride, float scale);
PXE_API int pxe_maxpool_nhwc(pxe_stream_t stream, const float* in, long long in_pixel_stride, float* out,
                             long long out_pixel_stride, int batch, int channels, int height, int width,
                             int kernel, int stride, int padding);

/* NHWC -> dense NCHW (batch stride 0 = channels*height*width): hands a head to the decoders, which read the
 * reference's [B][C][H*W] layout. */
PXE_API int pxe_nhwc_to_nchw(pxe_stream_t stream, const float* in, long long in_pixel_stride, float* out,
                             long long out_batch_stride, int batch, int channels, int height, int width);

/* ------------------------------------------------------------------------------------------
 * The network's first convolution fused with its epilogue (ConvLayer<CUDA>::forward in one launch,
 * include/cuda/ConvLayer.h:278-307): 3x3, stride 1, padding 1, dilation 1, one group, 1..4 input channels,
 * 8..64 output channels in multiples of 8.  With so few input channels the layer is bound by writing its
 * output, the largest tensor of the network, not by arithmetic; cuDNN + a separate epilogue write it once
 * and then read and write it again.  y = act(a[k] * conv(x, weights)[k] + b[k]) with the folded coefficients
 * of pxe_fold_bn (NULL, NULL: no affine part).  Summation order differs from cuDNN's, so results agree with
 * the two-launch path to fp32 rounding (a few 1e-7 relative), not bit for bit.
 * ------------------------------------------------------------------------------------------ */
typedef struct pxe_stem_desc {
    const float* x;               /* [batch, in_channels, height, width], NCHW */
    long long x_batch_stride;     /* 0 = dense */
    const float* weights;         /* [out_channels, in_channels, 3, 3], the layer's weights_ */
    const float* a;               /* folded coefficients [out_channels], or NULL (with b) */
    const float* b;
    float* y;                     /* output, same height and width */
    int y_is_nhwc;                /* 0: [batch, out_channels, H, W]; 1: [batch, H, W, out_channels] */
    long long y_stride;           /* NCHW: batch stride; NHWC: pixel stride; 0 = dense */
    int batch, in_channels, out_channels, height, width;
    int act;                      /* pxe_activation */
} pxe_stem_desc;

PXE_API int pxe_conv_stem(pxe_stream_t stream, const pxe_stem_desc* desc);

/* Global average pooling (AvgPoolLayer::forward, include/AvgPoolLayer.h:66-87; cudnnPoolingForward with an
 * H x W average window on the CUDA path, include/cuda/AvgPoolLayer.h:66-75): y[b][c] = mean of plane (b, c).
 * x: [batch, channels, height, width] with batch stride (0 = dense); y: [batch, channels] likewise. */
PXE_API int pxe_avgpool(pxe_stream_t stream, const float* x, long long x_batch_stride, float* y,
                        long long y_batch_stride, int batch, int channels, int height, int width);

/* YOLOv1 detection head decode (DetectLayer::addDetects, include/DetectLayer.h:166-209; the CUDA layer copies
 * the whole head to the host first, include/cuda/DetectLayer.h).  `pred`: per image
 * [side*side*classes class scores][side*side*num object scales][side*side*num*coords boxes], the layer's
 * input as the connected layer before it leaves it.  A box is emitted when its scale is finite and positive
 * and scale * (best class score of its cell) >= threshold; its record carries that class and probability;
 * squared != 0 squares the predicted width / height (the layer's `sqrt` option; v*v here, powf(v, 2) on the
 * reference's host path, which can differ in the last bit).  Records are appended to
 * `dets` behind *count (device) in the reference's order (image, cell, box); *count advances past every
 * emitted box even when capacity is exceeded.  width / height: the scale of the boxes (1, 1 = normalised). */
PXE_API int pxe_detect_decode(pxe_stream_t stream, const float* pred, long long pred_batch_stride, int batch,
                              int side, int num, int classes, int coords, int squared, float width, float height,
                              float threshold, pxe_detection* dets, long long capacity, long long* count,
                              int batch_id_offset);

/* SoftmaxLayer::addDetects (include/SoftmaxLayer.h:182-196): one record per image whose largest class
 * probability (the first maximum, std::max_element) is >= threshold: box {0, 0, width, height}, that class and
 * probability.  probs: the output of pxe_softmax, [batch][classes] with batch stride (0 = classes).  Records
 * are appended behind *count (device), images in order. */
PXE_API int pxe_softmax_decode(pxe_stream_t stream, const float* probs, long long probs_batch_stride, int batch,
                               int classes, float width, float height, float threshold, pxe_detection* dets,
                               long long capacity, long long* count, int batch_id_offset);

/* RegionLayer::addDetects (include/RegionLayer.h:355-395, box from lightBox, src/DarkBox.cpp:191-202) on the
 * output of pxe_region_forward: for box (cell, n) with scale = its objectness entry, every class j with
 * scale * class_j >= threshold is one record {x - w/2, y - h/2, w, h} * image size, x = (col + logistic(tx)) / W,
 * w = exp(tw) * anchors[2n] / W.  anchors: 2*num floats on the HOST (the layer's `anchors`, at most 32 boxes per
 * cell).  Order: image, cell, box, class; records are appended behind *count (device) as in pxe_yolo_decode.
 * per_image = 0 reproduces the reference exactly: it indexes the predictions without the image's offset
 * (RegionLayer.h:363-369), so every image of a batch decodes image 0's boxes; per_image = 1 decodes each
 * image's own. */
PXE_API int pxe_region_decode(pxe_stream_t stream, const float* pred, int batch, int width, int height, int num,
                              int coords, int classes, const float* anchors, int per_image, float image_width,
                              float image_height, float threshold, pxe_detection* dets, long long capacity,
                              long long* count, int batch_id_offset);

/* ------------------------------------------------------------------------------------------
 * Post-processing on the host: px::nms (src/Box.cpp:56-145), same ordering, same 0.9 IoU
 * cross-class duplicate rule, same 1024-candidate cap per (image, class) group.
 * `out` must have room for n records; returns the number kept (or a negative pxe_status).
 * ------------------------------------------------------------------------------------------ */
PXE_API long long pxe_nms_host(const pxe_detection* dets, long long n, float threshold, pxe_detection* out);

/* The same post-processing on the device: `dets` and `out` are device buffers of n records (out has room for
 * n), *out_count (device) receives the number kept; the kept records are those pxe_nms_host keeps, in the
 * same order, bit for bit.  Nothing is copied to the host and nothing synchronises: the O(N^2) passes of
 * src/Box.cpp:68-139 run as one block per image / per (image, class) group.  n is the host's copy of the
 * record count (the decodes leave it on the device; the caller reads it to size its own buffers anyway).
 * `workspace`: pxe_nms_workspace_bytes(n) bytes, 256-byte aligned.  Records with NaN probabilities have no
 * defined order in the reference (its comparator is `a.prob > b.prob`); here they sort first. */
PXE_API size_t pxe_nms_workspace_bytes(long long n);
PXE_API int pxe_nms(pxe_stream_t stream, const pxe_detection* dets, long long n, float threshold,
                    pxe_detection* out, long long* out_count, void* workspace, size_t workspace_bytes);

/* ------------------------------------------------------------------------------------------
 * The other side of the same layers: what PixieNN's CUDA layers call on the way back through the
 * graph and when they set weights up.  Element-wise and reduction kernels; none synchronises.
 * ------------------------------------------------------------------------------------------ */
/* px::gradient (include/Activation.cuh:27, src/Activation.cu:84-92, 135-143): delta[i] *= f'(x[i]) with the
 * gradient() of the functor for `act` (include/Activation.h:54-228). */
PXE_API int pxe_activation_gradient(pxe_stream_t stream, int act, const float* x, size_t n, float* delta);
/* px::backwardBiasGpu (include/BiasKernels.cuh:22, src/BiasKernels.cu:39-111): bias_updates[f] += the sum of
 * delta[b, f, 0..size) over the images; size == 1 is the connected-layer form.  batch * size < 2^31.  The sum is
 * taken in a fixed order (the same bits on every call); it needs no scratch memory. */
PXE_API int pxe_backward_bias(pxe_stream_t stream, float* bias_updates, const float* delta, int batch, int n,
                              int size);
/* px::maxPoolBackwardGpu (include/MaxPoolKernels.cuh:7, src/MaxPoolKernels.cu:45-49, 61-65):
 * grad[indexes[i]] += delta[i] for every output i whose window had a tap. */
PXE_API int pxe_maxpool_backward(pxe_stream_t stream, const float* delta, const int* indexes, float* grad,
                                 size_t size);
/* px::upsampleGpu with forward == 0 (src/UpsampleKernels.cu:25-63): acc[b, c, y, x] += scale * the sum of the
 * stride x stride elements of `out` ([batch, channels, height*stride, width*stride]) above that input. */
PXE_API int pxe_upsample_backward(pxe_stream_t stream, float* acc, const float* out, int batch, int channels,
                                  int height, int width, int stride, float scale);
/* px::constrainGpu (src/CudaUtils.cu:122-138): x = min(alpha, max(-alpha, x)). */
PXE_API int pxe_constrain(pxe_stream_t stream, float* x, size_t n, float alpha);
/* px::mulGpu (src/CudaUtils.cu:140-146): y = x * y. */
PXE_API int pxe_mul(pxe_stream_t stream, const float* x, float* y, size_t n);
/* px::randomGpu / px::randomNormalGpu (src/CudaUtils.cu:77-120): element i is drawn from the minimal-standard
 * generator (seed 1) advanced i steps, mapped to U[a, b) or to N(mean, stddev) by inversion.  The uniform
 * values follow the reference's mapping; the normal values follow the same engine positions but this
 * library's own inversion, so they agree with the reference in distribution, not digit for digit. */
PXE_API int pxe_random_uniform(pxe_stream_t stream, float* out, size_t n, float a, float b);
PXE_API int pxe_random_normal(pxe_stream_t stream, float* out, size_t n, float mean, float stddev);

/* ------------------------------------------------------------------------------------------
 * Loss kernels of the detector heads.
 * ------------------------------------------------------------------------------------------ */
/* px::yoloLossGpu (include/YoloKernels.cuh:10-19, src/YoloKernels.cu:73-252) as one launch.  All pointers are
 * device memory.  `output` is the activated head [batch, mask_count*(5+classes), height, width]; `delta` has the
 * same shape and is updated in place (entries the loss does not decide keep their value, as in the reference,
 * which clears delta before the call); truths: [batch, max_truth, 5] = x, y, w, h, class; assigned_*: one entry
 * per box slot (image, mask slot, cell), assigned_classes < 0 where no truth is assigned; masks: anchor index
 * of every mask slot; anchors: [2 * anchors] floats.  stats (PXE_YOLO_STATS_SIZE floats) and cost (1 float) are
 * added to, not cleared. */
#define PXE_YOLO_STATS_SIZE 12
typedef struct pxe_yolo_loss_desc {
    const float* output;
    float* delta;
    const float* truths;
    const int* truth_counts;
    int max_truth;
    const int* assigned_classes;
    const int* assigned_anchors;
    const float* assigned_boxes;
    const int* masks;
    const float* anchors;
    float* stats;
    float* cost;
    int batch, mask_count, classes, width, height;
    int network_width, network_height;
    float ignore_threshold, truth_threshold, coord_scale, object_scale, no_object_scale, class_scale;
} pxe_yolo_loss_desc;

PXE_API int pxe_yolo_loss(pxe_stream_t stream, const pxe_yolo_loss_desc* desc);

/* px::centerNetLossGpu (include/CenterNetKernels.cuh:8-13, src/CenterNetKernels.cu:20-139): focal loss on the
 * heat map (costs[0]), L1 loss on size (costs[1]) and offset (costs[2]) at the cells target_mask marks; delta
 * [batch, classes+4, area] receives normalizer * the negative gradients.  costs is added to, not cleared. */
PXE_API int pxe_centernet_loss(pxe_stream_t stream, const float* output, float* delta, const float* target_heatmap,
                               const float* target_size, const float* target_offset, const float* target_mask,
                               float* costs, int batch, int classes, int area, float normalizer, float focal_alpha,
                               float focal_beta, float size_weight);

/* px::adamGpu (include/Adam.cuh:21, src/Adam.cu:26-47): x[i] += rate * mhat / (sqrt(vhat) + eps) with
 * mhat = m[i] / (1 - beta1^t), vhat = v[i] / (1 - beta2^t); t counts steps from 1. */
PXE_API int pxe_adam_update(pxe_stream_t stream, size_t n, float* x, const float* m, const float* v, float beta1,
                            float beta2, float rate, float eps, int t);
/* px::softmaxCrossEntropy (include/SoftmaxKernel.cuh:21, src/SoftmaxKernel.cu:25-48):
 * error[i] = truth[i] ? -log(pred[i] + 1e-9) : 0, delta[i] = truth[i] - pred[i]. */
PXE_API int pxe_softmax_cross_entropy(pxe_stream_t stream, size_t n, const float* pred, const float* truth, float* delta,
                                      float* error);

/* ------------------------------------------------------------------------------------------
 * Batch normalisation in training mode.  Replaces cudnnBatchNormalizationForwardTraining
 * (include/cuda/ConvLayer.h:285-292, include/cuda/BatchNormLayer.h:59-71, include/cuda/ConnLayer.h:198-203)
 * together with the copies around it (x_.copy(output_), preActivation_.copy(output_) and the in-place activation,
 * include/cuda/ConvLayer.h:286, 306-307), and cudnnBatchNormalizationBackward (include/cuda/ConvLayer.h:327-332,
 * include/cuda/BatchNormLayer.h:108-118, include/cuda/ConnLayer.h:233-238).  CPU twins: batchNormForward /
 * batchNormBackward, src/BatchNorm.cpp:24-98.  Tensors are dense NCHW; every sum is taken in a fixed order.
 * ------------------------------------------------------------------------------------------ */
typedef struct pxe_bn_train_desc {
    const float* x;          /* [batch, channels, height, width]: the convolution output (the reference's x_) */
    float* y;                /* gamma * xhat + beta (the reference's preActivation_); may be x itself */
    float* y_act;            /* NULL, or act(y): the layer output; must not alias x or y */
    int act;                 /* enum pxe_activation, evaluated with the precise math library */
    int batch, channels, height, width;
    const float* gamma;      /* [channels] scales */
    const float* beta;       /* [channels] biases */
    float* running_mean;     /* [channels] or NULL: (1 - f) * running + f * batch mean */
    float* running_var;      /* [channels] or NULL: fed the unbiased variance (PXE_BN_EPS_CUDNN, as cuDNN does) or
                                the population variance (PXE_BN_EPS_CPU, src/BatchNorm.cpp:55-56) */
    float exp_avg_factor;    /* f: 0.01 in the reference */
    float eps;               /* 1e-5 in the reference */
    int eps_mode;            /* enum pxe_bn_eps_mode */
    float* save_mean;        /* [channels] out: batch mean */
    float* save_scale;       /* [channels] out: 1 / sqrt(var + eps), cuDNN's saved inverse variance (PXE_BN_EPS_CUDNN),
                                or the population variance itself (PXE_BN_EPS_CPU: the reference's var) */
    void* workspace;         /* pxe_batchnorm_workspace_bytes(batch, channels, height, width), 16-byte aligned */
    size_t workspace_bytes;
} pxe_bn_train_desc;

typedef struct pxe_bn_backward_desc {
    const float* x;          /* the x the forward call saw */
    const float* dy;         /* gradient with respect to y (after px::gradient has been applied) */
    float* dx;               /* gradient with respect to x; may be dy itself, must not be x */
    int batch, channels, height, width;
    const float* gamma;
    float* dgamma;           /* [channels] or NULL: += sum of dy * xhat */
    float* dbeta;            /* [channels] or NULL: += sum of dy */
    const float* save_mean;  /* from the forward call, same eps_mode */
    const float* save_scale;
    float eps;
    int eps_mode;
    void* workspace;
    size_t workspace_bytes;
} pxe_bn_backward_desc;

PXE_API size_t pxe_batchnorm_workspace_bytes(int batch, int channels, int height, int width);
/* Three launches: per-channel sums, per-channel constants (and the running statistics), one pass that writes y and,
 * if asked, act(y). */
PXE_API int pxe_batchnorm_forward_training(pxe_stream_t stream, const pxe_bn_train_desc* desc);
/* Three launches: per-channel sums of dy and dy * (x - mean), per-channel constants (and the parameter gradients),
 * dx = k1 * dy + k2 * x + k3. */
PXE_API int pxe_batchnorm_backward(pxe_stream_t stream, const pxe_bn_backward_desc* desc);

#ifdef __cplusplus
}
#endif
#endif /* PXE_H */
