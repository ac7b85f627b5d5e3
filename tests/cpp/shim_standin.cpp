// Compiles the body fragments of include/shim/ inside member functions of minimal stand-ins for the reference's
// classes: the members the fragments touch, under the reference's names (include/Layer.h, ConvLayer.h, RouteLayer.h,
// YoloLayer.h, CenterNetLayer.h, Detection.h, Error.h).  Nothing runs on a GPU: main() builds a plan for a small graph,
// walks the conv fragment's host logic with null device pointers replaced by host arrays and checks which pointers
// and strides the descriptors end up with.  A misspelt field of pxe.h / pxe_plan.h, or a fragment that no longer
// matches the entry points, fails to compile here.
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <vector>

// ---- what the reference supplies -------------------------------------------------------------------------
#define PX_CHECK(cond, ...) do { if (!(cond)) { std::fprintf(stderr, __VA_ARGS__); std::fprintf(stderr, "\n"); std::exit(2); } } while (0)
#define PX_CUDA_CHECK_ERR(expr) do { if ((expr) != 0) std::exit(3); } while (0)
enum { cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2 };
static int cudaMemcpy(void*, const void*, std::size_t, int) { return 0; }          // never reached in this program
namespace cv { struct Rect2f { float x, y, width, height; Rect2f(float a, float b, float c, float d) : x(a), y(b), width(c), height(d) {} }; }

// ---- the entry points the fragments call, recorded instead of launched ------------------------------------
#include "pxe.h"
#include "pxe_plan.h"
static pxe_epilogue_desc g_last_epilogue;
static int g_epilogues = 0, g_concats = 0;
static pxe_bn_train_desc g_last_bn_train;
static pxe_bn_backward_desc g_last_bn_backward;
#define pxe_batchnorm_forward_training shim_test_bn_forward
#define pxe_batchnorm_backward shim_test_bn_backward
static int shim_test_bn_forward(pxe_stream_t, const pxe_bn_train_desc* d) { g_last_bn_train = *d; return PXE_OK; }
static int shim_test_bn_backward(pxe_stream_t, const pxe_bn_backward_desc* d) { g_last_bn_backward = *d; return PXE_OK; }
struct PoolCall { const float* x; float* y; long long ybs; int* indexes; int kernel, stride, padding; };
struct SppCall { const float* x; int n; int kernels[4]; float* ys[4]; long long strides[4]; };
struct UpCall { const float* x; float* y; long long ybs; int stride; };
struct ShortcutCall { const float* x; const float* from; float* y; long long ybs; float* y2; long long y2bs; int act; };
static std::vector<PoolCall> g_pools;
static std::vector<SppCall> g_spps;
static std::vector<UpCall> g_ups;
static std::vector<ShortcutCall> g_shortcuts;
static int g_general_shortcuts = 0, g_activations = 0;
static std::vector<float*> g_copy_dsts;
#define pxe_maxpool shim_test_maxpool
#define pxe_spp shim_test_spp
#define pxe_upsample shim_test_upsample
#define pxe_shortcut shim_test_shortcut
#define pxe_shortcut_general shim_test_shortcut_general
#define pxe_activate shim_test_activate
static int shim_test_maxpool(pxe_stream_t, const float* x, long long, float* y, long long ybs, int* idx, int, int, int, int, int k, int s, int p)
{ g_pools.push_back({x, y, ybs, idx, k, s, p}); return PXE_OK; }
static int shim_test_spp(pxe_stream_t, const float* x, long long, int, int, int, int, int n, const int* kernels, float* const* ys, const long long* strides)
{ SppCall c{}; c.x = x; c.n = n; for (int i = 0; i < n && i < 4; ++i) { c.kernels[i] = kernels[i]; c.ys[i] = ys[i]; c.strides[i] = strides[i]; } g_spps.push_back(c); return PXE_OK; }
static int shim_test_upsample(pxe_stream_t, const float* x, long long, float* y, long long ybs, int, int, int, int, int stride, float)
{ g_ups.push_back({x, y, ybs, stride}); return PXE_OK; }
static int shim_test_shortcut(pxe_stream_t, const float* x, long long, const float* from, long long, float* y, long long ybs, float* y2, long long y2bs,
                              int, int, int, int, float, float, int act)
{ g_shortcuts.push_back({x, from, y, ybs, y2, y2bs, act}); return PXE_OK; }
static int shim_test_shortcut_general(pxe_stream_t, int, int, int, int, const float*, int, int, int, float, float, float*) { ++g_general_shortcuts; return PXE_OK; }
static int shim_test_activate(pxe_stream_t, int, float*, size_t) { ++g_activations; return PXE_OK; }
struct RegionCall { const float* in; float* out; int num, coords, classes, softmax; };
struct RegionDecodeCall { const float* pred; const float* anchors; int per_image; float w, h, thr; long long capacity; };
struct SoftmaxCall { const float* in; float* out; int inputs, groups; float temp; };
struct AvgCall { const float* x; float* y; long long ybs; int c, h, w; };
static std::vector<RegionCall> g_regions;
static std::vector<RegionDecodeCall> g_region_decodes;
static std::vector<SoftmaxCall> g_softmaxes;
static std::vector<AvgCall> g_avgs;
struct DetectCall { const float* pred; long long pbs; int side, num, classes, coords, squared; float w, h; long long capacity; };
static std::vector<DetectCall> g_detects;
#define pxe_detect_decode shim_test_detect_decode
static int shim_test_detect_decode(pxe_stream_t, const float* pred, long long pbs, int, int side, int num, int classes, int coords, int squared,
                                   float w, float h, float, pxe_detection*, long long capacity, long long*, int)
{ g_detects.push_back({pred, pbs, side, num, classes, coords, squared, w, h, capacity}); return PXE_OK; }
#define pxe_region_forward shim_test_region_forward
#define pxe_region_decode shim_test_region_decode
#define pxe_softmax shim_test_softmax
#define pxe_avgpool shim_test_avgpool
static int shim_test_region_forward(pxe_stream_t, const float* in, float* out, int, int, int, int num, int coords, int classes, int softmax)
{ g_regions.push_back({in, out, num, coords, classes, softmax}); return PXE_OK; }
static int shim_test_region_decode(pxe_stream_t, const float* pred, int, int, int, int, int, int, const float* anchors, int per_image, float w, float h,
                                   float thr, pxe_detection*, long long capacity, long long*, int)
{ g_region_decodes.push_back({pred, anchors, per_image, w, h, thr, capacity}); return PXE_OK; }
static int shim_test_softmax(pxe_stream_t, const float* in, float* out, int, int inputs, int groups, float temp)
{ g_softmaxes.push_back({in, out, inputs, groups, temp}); return PXE_OK; }
static int shim_test_avgpool(pxe_stream_t, const float* x, long long, float* y, long long ybs, int, int c, int h, int w)
{ g_avgs.push_back({x, y, ybs, c, h, w}); return PXE_OK; }
#define pxe_conv_epilogue shim_test_conv_epilogue
#define pxe_concat shim_test_concat
#define pxe_yolo_decode shim_test_yolo_decode
#define pxe_centernet_decode shim_test_centernet_decode
static int shim_test_conv_epilogue(pxe_stream_t, const pxe_epilogue_desc* d) { g_last_epilogue = *d; ++g_epilogues; return PXE_OK; }
static int shim_test_concat(pxe_stream_t, int, const float* const*, const long long*, const int*, float* dst, long long, int, int, int) { ++g_concats; g_copy_dsts.push_back(dst); return PXE_OK; }
static int shim_test_yolo_decode(pxe_stream_t, const pxe_yolo_decode_desc*, pxe_detection*, long long, long long*, void*, size_t) { return PXE_OK; }
static int shim_test_centernet_decode(pxe_stream_t, const pxe_centernet_decode_desc*, pxe_detection*, int*, void*, size_t) { return PXE_OK; }

#include "shim/pxe_shim.h"

namespace px {

struct Detection { Detection(cv::Rect2f, int, int, float) {} };
using Detections = std::vector<Detection>;

template <typename T>
struct Vec {                                        // PxCudaVectorT: data() and size()
    std::vector<T> v;
    T* data() { return v.data(); }
    const T* data() const { return v.data(); }
    std::size_t size() const { return v.size(); }
    void copy(const Vec<T>& o) { v = o.v; }                // PxCudaVectorT::copy
};

struct Model;

struct Layer {
    Layer(Model& m, int index, int c, int h, int w, int batch) : model_(m), index_(index), c_(c), h_(h), w_(w), batch_(batch)
    {
        output_.v.resize((std::size_t)batch * c * h * w);
    }
    virtual ~Layer() = default;
    Model& model() { return model_; }
    int index() const { return index_; }
    int batch() const { return batch_; }
    int outChannels() const { return c_; }
    int outHeight() const { return h_; }
    int outWidth() const { return w_; }
    int outputs() const { return c_ * h_ * w_; }
    const Vec<float>& output() const { return output_; }
    float* pxeOutput() { return output_.data(); }      // the additive accessor
    float alpha() const { return 1.0f; }
    float beta() const { return 1.0f; }
    int pxeActivation() const { return pxeActivation_; }
    int padding() const { return 1; }
    int pxeKernel() const { return pxeKernel_; }
    bool training() const { return false; }
    // input geometry (the stand-in's layers keep their input's shape unless set otherwise)
    int channels() const { return in_c_ ? in_c_ : c_; }
    int height() const { return in_h_ ? in_h_ : h_; }
    int width() const { return in_w_ ? in_w_ : w_; }
    int in_c_ = 0, in_h_ = 0, in_w_ = 0, pxeKernel_ = 2;
    Model& model_;
    int index_, c_, h_, w_, batch_;
    Vec<float> output_;
    int pxeActivation_ = PXE_ACT_LINEAR;
};

struct Model {
    std::vector<std::unique_ptr<Layer>> layers_;
    pxe_shim::PlanView plan_;
    const pxe_shim::PlanView& pxePlan() const { return plan_; }
    Layer& layerAt(int i) { return *layers_[(std::size_t)i]; }
    int width() const { return 32; }
    int height() const { return 32; }
};

struct ConvLayer : Layer {
    ConvLayer(Model& m, int index, int filters, int h, int w, int batch, bool bn) : Layer(m, index, filters, h, w, batch), filters_(filters), batchNorm_(bn)
    {
        for (auto* p : {&scales_, &biases_, &rollingMean_, &rollingVar_}) p->v.resize((std::size_t)filters);
        pxeActivation_ = pxe_shim::activation_from_name("leaky");
    }
    void forwardEpilogue()
    {
#include "shim/conv_forward_epilogue.inl"
    }
    void forwardTraining()
    {
#include "shim/conv_forward_training.inl"
    }
    void backwardBatchNorm()
    {
#include "shim/conv_backward_batchnorm.inl"
    }
    int filters_;
    bool batchNorm_;
    Vec<float> scales_, biases_, rollingMean_, rollingVar_;
    Vec<float> x_, preActivation_, delta_, mean_, var_, scaleUpdates_, biasUpdates_;      // the training-side members
    Vec<char> pxeBnWorkspace_;
};

struct RouteLayer : Layer {
    using Layer::Layer;
    std::vector<Layer*> layers_;
    void forwardBody()
    {
#include "shim/route_forward.inl"
    }
};

struct MaxPoolLayer : Layer {
    using V = Vec<float>;
    MaxPoolLayer(Model& m, int index, int c, int h, int w, int batch, int kernel, int stride, int padding)
        : Layer(m, index, c, h, w, batch), kernel_(kernel), stride_(stride), padding_(padding) { pxeKernel_ = kernel; }
    int kernel_, stride_, padding_;
    Vec<int> indexes_;
    void forward(const V& input)
    {
#include "shim/maxpool_forward.inl"
    }
};

struct UpsampleLayer : Layer {
    using V = Vec<float>;
    UpsampleLayer(Model& m, int index, int c, int h, int w, int batch, int stride) : Layer(m, index, c, h * stride, w * stride, batch), stride_(stride)
    { in_c_ = c; in_h_ = h; in_w_ = w; }
    int stride_;
    float scale_ = 1.0f;
    void forward(const V& input)
    {
#include "shim/upsample_forward.inl"
    }
};

struct ShortcutLayer : Layer {
    using V = Vec<float>;
    ShortcutLayer(Model& m, int index, int c, int h, int w, int batch, Layer* from) : Layer(m, index, c, h, w, batch), from_(from) {}
    Layer* from_;
    float alpha_ = 1.0f, beta_ = 1.0f;
    void forward(const V& input)
    {
#include "shim/shortcut_forward.inl"
    }
};

struct RegionLayer : Layer {
    using V = Vec<float>;
    using Layer::Layer;
    int classes() const { return 3; }
    int num_ = 2, coords_ = 4;
    bool softmax_ = true;
    std::vector<float> anchors_{1.0f, 2.0f, 3.0f, 4.0f};
    Vec<char> pxeDets_;
    Vec<long long> pxeCount_;
    long long pxeCapacity_ = 64;
    void forward(const V& input)
    {
#include "shim/region_forward.inl"
    }
    void addDetects(Detections& detects, int width, int height, float threshold)
    {
#include "shim/region_add_detects.inl"
    }
};

struct SoftmaxLayer : Layer {
    using V = Vec<float>;
    using Layer::Layer;
    int inputs() const { return c_ * h_ * w_; }
    int groups_ = 2;
    float temperature_ = 0.5f;
    void forward(const V& input)
    {
#include "shim/softmax_forward.inl"
    }
};

struct AvgPoolLayer : Layer {
    using V = Vec<float>;
    AvgPoolLayer(Model& m, int index, int c, int h, int w, int batch) : Layer(m, index, c, 1, 1, batch) { in_c_ = c; in_h_ = h; in_w_ = w; }
    void forward(const V& input)
    {
#include "shim/avgpool_forward.inl"
    }
};

struct ConnLayer : Layer {
    ConnLayer(Model& m, int index, int outputs, int batch, bool bn) : Layer(m, index, outputs, 1, 1, batch), batchNorm_(bn)
    {
        for (auto* p : {&scales_, &biases_, &rollingMean_, &rollingVar_}) p->v.resize((std::size_t)outputs);
        pxeActivation_ = pxe_shim::activation_from_name("relu");
    }
    bool batchNorm_;
    Vec<float> scales_, biases_, rollingMean_, rollingVar_;
    void forwardEpilogue()
    {
#include "shim/conn_forward_epilogue.inl"
    }
};

struct DetectLayer : Layer {
    using Layer::Layer;
    int classes() const { return 20; }
    int coords_ = 4, num_ = 2, side_ = 7;
    bool sqrt_ = true;
    Vec<char> pxeDets_;
    Vec<long long> pxeCount_;
    long long pxeCapacity_ = 0;
    void addDetects(Detections& detects, int width, int height, float threshold)
    {
#include "shim/detect_add_detects.inl"
    }
};

struct YoloLayer : Layer {
    using Layer::Layer;
    int classes() const { return 2; }
    std::vector<int> mask_{0, 1, 2}, anchors_{10, 14, 23, 27, 37, 58};
    Vec<char> pxeDets_, pxeWorkspace_;
    Vec<long long> pxeCount_;
    long long pxeCapacity_ = 0;
    void addDetects(Detections& detects, int width, int height, float threshold)
    {
#include "shim/yolo_add_detects.inl"
    }
};

struct CenterNetLayer : Layer {
    using Layer::Layer;
    int classes_ = 3, maxDetections_ = 10;
    Vec<char> pxeDets_, pxeWorkspace_;
    Vec<int> pxeCounts_;
    void addDetects(Detections& detections, int width, int height, float threshold)
    {
#include "shim/centernet_add_detects.inl"
    }
};

}   // namespace px

static pxe_layer_desc desc(int type, int c, int h, int w, int src0, int src1 = -2)
{
    pxe_layer_desc d{};
    d.type = type; d.out_channels = c; d.out_height = h; d.out_width = w;
    d.kernel = type == PXE_LAYER_MAXPOOL ? 2 : 3; d.stride = type == PXE_LAYER_MAXPOOL ? 2 : 1; d.padding = 1;
    d.batch_norm = 1; d.activation = PXE_ACT_LEAKY;
    d.n_sources = 1; d.sources[0] = src0;
    if (src1 != -2) { d.n_sources = 2; d.sources[1] = src1; }
    return d;
}

int main()
{
    // 0 conv, 1 conv, 2 shortcut(1, from 0), 3 conv, 4 route(3, 2): conv 1 absorbs the shortcut; convs 3 and the shortcut's
    // value (layer 2) are stored into the route's buffer
    const int B = 2, C = 4, H = 8, W = 8;
    px::Model m;
    m.layers_.emplace_back(new px::ConvLayer(m, 0, C, H, W, B, true));
    m.layers_.emplace_back(new px::ConvLayer(m, 1, C, H, W, B, true));
    m.layers_.emplace_back(new px::Layer(m, 2, C, H, W, B));
    m.layers_.emplace_back(new px::ConvLayer(m, 3, C, H, W, B, false));
    auto* route = new px::RouteLayer(m, 4, 2 * C, H, W, B);
    route->layers_ = {m.layers_[3].get(), m.layers_[2].get()};
    m.layers_.emplace_back(route);
    std::vector<pxe_layer_desc> descs = {desc(PXE_LAYER_CONV, C, H, W, -1), desc(PXE_LAYER_CONV, C, H, W, 0),
                                         desc(PXE_LAYER_SHORTCUT, C, H, W, 1, 0), desc(PXE_LAYER_CONV, C, H, W, 2),
                                         desc(PXE_LAYER_ROUTE, 2 * C, H, W, 3, 2)};
    if (pxe_shim::build_plan(descs, true, &m.plan_) != PXE_OK) { std::printf("plan failed: %s\n", pxe_last_error_string()); return 1; }
    if (m.plan_.step(2) != m.plan_.step(1) || m.plan_.step(1)->fused_shortcut != 2) { std::printf("shortcut not folded\n"); return 1; }

    auto* c1 = static_cast<px::ConvLayer*>(m.layers_[1].get());
    c1->forwardEpilogue();
    const pxe_epilogue_desc& d = g_last_epilogue;
    // conv 1 + shortcut 2: residual = layer 0's output; the value of layer 2 goes to its own dense tensor (conv 3 reads it)
    // and to channel slot [C, 2C) of the route's buffer
    bool ok = g_epilogues == 1 && d.x == c1->output_.data() && d.residual == m.layers_[0]->output_.data() &&
              d.residual_batch_stride == C * H * W && d.gamma == c1->scales_.data() && d.act == PXE_ACT_LEAKY &&
              d.y == m.layers_[2]->output_.data() && d.y_batch_stride == C * H * W &&
              d.y2 == route->output_.data() + (long long)C * H * W && d.y2_batch_stride == 2 * C * H * W;
    auto* c3 = static_cast<px::ConvLayer*>(m.layers_[3].get());
    c3->forwardEpilogue();
    // conv 3 has one reader, the route: its only destination is slot [0, C)
    ok = ok && g_epilogues == 2 && g_last_epilogue.y == route->output_.data() && g_last_epilogue.y_batch_stride == 2 * C * H * W &&
         g_last_epilogue.y2 == nullptr && g_last_epilogue.bias == c3->biases_.data() && g_last_epilogue.gamma == nullptr;
    route->forwardBody();
    ok = ok && g_concats == 0;                         // every producer was redirected: the route runs nothing
    // training: the batch-norm fragments hand over the saved input, the two outputs and the statistics' homes
    c1->forwardTraining();
    c1->backwardBatchNorm();
    ok = ok && g_last_bn_train.x == c1->x_.data() && g_last_bn_train.y == c1->preActivation_.data() &&
         g_last_bn_train.y_act == c1->output_.data() && g_last_bn_train.channels == C && g_last_bn_train.save_scale == c1->var_.data() &&
         g_last_bn_backward.dx == c1->delta_.data() && g_last_bn_backward.dy == c1->delta_.data() &&
         g_last_bn_backward.dgamma == c1->scaleUpdates_.data() && g_last_bn_backward.save_mean == c1->mean_.data();
    std::printf("%s: epilogues=%d concats=%d\n", ok ? "ok" : "MISMATCH", g_epilogues, g_concats);
    pxe_plan_destroy(m.plan_.plan);
    if (!ok) return 1;

    // ---- pools, SPP block, upsample into a route slot, shortcuts that stand alone ------------------------------
    //  0 conv 16x16          1 maxpool 2/2 (folded into 0)   2 conv 8x8            3 maxpool 5/1 of 2
    //  4 route(2)            5 maxpool 9/1                   6 route(2)            7 maxpool 13/1
    //  8 route(7, 5, 3, 2)   9 conv 8x8                     10 upsample x2        11 route(10, 0)
    // 12 conv 16x16         13 maxpool 2/1                  14 shortcut(13, from 12)   15 conv 16x16
    // 16 shortcut(15, from 9): 16x16 with an 8x8 partner
    px::Model n;
    const int S = 16, Hh = 8;
    auto add = [&](px::Layer* l) { n.layers_.emplace_back(l); return l; };
    add(new px::ConvLayer(n, 0, C, S, S, B, true));
    auto* p1 = new px::MaxPoolLayer(n, 1, C, Hh, Hh, B, 2, 2, 1); p1->in_c_ = C; p1->in_h_ = S; p1->in_w_ = S; add(p1);
    add(new px::ConvLayer(n, 2, C, Hh, Hh, B, true));
    auto* p3 = static_cast<px::MaxPoolLayer*>(add(new px::MaxPoolLayer(n, 3, C, Hh, Hh, B, 5, 1, 4)));
    add(new px::RouteLayer(n, 4, C, Hh, Hh, B));
    auto* p5 = static_cast<px::MaxPoolLayer*>(add(new px::MaxPoolLayer(n, 5, C, Hh, Hh, B, 9, 1, 8)));
    add(new px::RouteLayer(n, 6, C, Hh, Hh, B));
    auto* p7 = static_cast<px::MaxPoolLayer*>(add(new px::MaxPoolLayer(n, 7, C, Hh, Hh, B, 13, 1, 12)));
    auto* r8 = add(new px::RouteLayer(n, 8, 4 * C, Hh, Hh, B));
    add(new px::ConvLayer(n, 9, C, Hh, Hh, B, true));
    auto* u10 = static_cast<px::UpsampleLayer*>(add(new px::UpsampleLayer(n, 10, C, Hh, Hh, B, 2)));
    auto* r11 = add(new px::RouteLayer(n, 11, 2 * C, S, S, B));
    add(new px::ConvLayer(n, 12, C, S, S, B, true));
    auto* p13 = static_cast<px::MaxPoolLayer*>(add(new px::MaxPoolLayer(n, 13, C, S, S, B, 2, 1, 1)));
    auto* s14 = static_cast<px::ShortcutLayer*>(add(new px::ShortcutLayer(n, 14, C, S, S, B, n.layers_[12].get())));
    add(new px::ConvLayer(n, 15, C, S, S, B, true));
    auto* s16 = static_cast<px::ShortcutLayer*>(add(new px::ShortcutLayer(n, 16, C, S, S, B, n.layers_[9].get())));
    auto pool = [](int c, int hw, int k, int st, int pad, int src) {
        pxe_layer_desc d = desc(PXE_LAYER_MAXPOOL, c, hw, hw, src);
        d.kernel = k; d.stride = st; d.padding = pad;
        return d;
    };
    auto route_of = [](int c, int hw, std::initializer_list<int> srcs) {
        pxe_layer_desc d = desc(PXE_LAYER_ROUTE, c, hw, hw, -1);
        d.n_sources = 0;
        for (int v : srcs) d.sources[d.n_sources++] = v;
        return d;
    };
    pxe_layer_desc up = desc(PXE_LAYER_UPSAMPLE, C, S, S, 9);
    up.stride = 2;
    std::vector<pxe_layer_desc> nd = {
        desc(PXE_LAYER_CONV, C, S, S, -1), pool(C, Hh, 2, 2, 1, 0), desc(PXE_LAYER_CONV, C, Hh, Hh, 1), pool(C, Hh, 5, 1, 4, 2),
        route_of(C, Hh, {2}), pool(C, Hh, 9, 1, 8, 4), route_of(C, Hh, {2}), pool(C, Hh, 13, 1, 12, 6), route_of(4 * C, Hh, {7, 5, 3, 2}),
        desc(PXE_LAYER_CONV, C, Hh, Hh, 8), up, route_of(2 * C, S, {10, 0}), desc(PXE_LAYER_CONV, C, S, S, 11), pool(C, S, 2, 1, 1, 12),
        desc(PXE_LAYER_SHORTCUT, C, S, S, 13, 12), desc(PXE_LAYER_CONV, C, S, S, 14), desc(PXE_LAYER_SHORTCUT, C, S, S, 15, 9)};
    if (pxe_shim::build_plan(nd, true, &n.plan_) != PXE_OK) { std::printf("plan 2 failed: %s\n", pxe_last_error_string()); return 1; }
    const long long small = (long long)Hh * Hh, big = (long long)S * S;
    // the folded pool and the later pools of the SPP block run nothing
    p1->forward(n.layers_[0]->output_);
    p5->forward(n.layers_[4]->output_);
    p7->forward(n.layers_[6]->output_);
    bool ok2 = g_pools.empty() && g_spps.empty();
    // the first pool of the block: one call, kernels 5 / 9 / 13, each into its slot of route 8 = (13, 9, 5, identity)
    p3->forward(n.layers_[2]->output_);
    ok2 = ok2 && g_spps.size() == 1 && g_spps[0].n == 3 && g_spps[0].x == n.layers_[2]->output_.data() &&
          g_spps[0].kernels[0] == 5 && g_spps[0].kernels[1] == 9 && g_spps[0].kernels[2] == 13 &&
          g_spps[0].ys[0] == r8->output_.data() + 2 * C * small && g_spps[0].ys[1] == r8->output_.data() + 1 * C * small &&
          g_spps[0].ys[2] == r8->output_.data() && g_spps[0].strides[0] == 4 * C * small && g_pools.empty();
    // the upsampled tensor goes straight into channels [0, C) of route 11
    u10->forward(n.layers_[9]->output_);
    ok2 = ok2 && g_ups.size() == 1 && g_ups[0].x == n.layers_[9]->output_.data() && g_ups[0].y == r11->output_.data() &&
          g_ups[0].ybs == 2 * C * big && g_ups[0].stride == 2;
    // conv 0: full-resolution output into channels [C, 2C) of route 11, pooled output into layer 1's own tensor
    static_cast<px::ConvLayer*>(n.layers_[0].get())->forwardEpilogue();
    ok2 = ok2 && g_last_epilogue.y == r11->output_.data() + C * big && g_last_epilogue.y_batch_stride == 2 * C * big &&
          g_last_epilogue.y_pool == p1->output_.data() && g_last_epilogue.pool_kernel == 2;
    // a pool that stands alone, with the layer's own kernel / stride / padding
    p13->forward(n.layers_[12]->output_);
    ok2 = ok2 && g_pools.size() == 1 && g_pools[0].x == n.layers_[12]->output_.data() && g_pools[0].y == p13->output_.data() &&
          g_pools[0].kernel == 2 && g_pools[0].stride == 1 && g_pools[0].padding == 1 && g_pools[0].indexes == nullptr;
    // a shortcut behind a pool cannot be folded into a convolution: one pass
    s14->pxeActivation_ = PXE_ACT_LEAKY;
    s14->forward(p13->output_);
    ok2 = ok2 && g_shortcuts.size() == 1 && g_shortcuts[0].x == p13->output_.data() && g_shortcuts[0].from == n.layers_[12]->output_.data() &&
          g_shortcuts[0].y == s14->output_.data() && g_shortcuts[0].y2 == nullptr && g_shortcuts[0].act == PXE_ACT_LEAKY;
    // partner of another shape: the reference's three steps (conv 15 keeps its epilogue: the plan does not fold this one)
    const pxe_step* st15 = n.plan_.step(15);
    ok2 = ok2 && st15 != nullptr && st15->fused_shortcut < 0;
    s16->forward(n.layers_[15]->output_);
    ok2 = ok2 && g_general_shortcuts == 1 && g_activations == 1 && g_shortcuts.size() == 1;
    std::printf("%s: pools=%zu spp=%zu upsamples=%zu shortcuts=%zu general=%d\n", ok2 ? "ok" : "MISMATCH", g_pools.size(), g_spps.size(),
                g_ups.size(), g_shortcuts.size(), g_general_shortcuts);
    pxe_plan_destroy(n.plan_.plan);
    if (!ok2) return 1;

    // ---- heads that need no plan: Region forward / addDetects, softmax, global average pool -----------------------
    px::Model h;
    px::RegionLayer region(h, 0, 2 * (4 + 1 + 3), 5, 5, B);
    px::Vec<float> head_in;
    head_in.v.resize(region.output_.size());
    region.pxeDets_.v.resize(64 * sizeof(pxe_detection));
    region.pxeCount_.v.resize(1);
    region.forward(head_in);
    px::Detections found;
    region.addDetects(found, 416, 320, 0.25f);
    px::SoftmaxLayer soft(h, 1, 10, 1, 1, B);
    px::Vec<float> soft_in;
    soft_in.v.resize(soft.output_.size());
    soft.forward(soft_in);
    px::AvgPoolLayer avg(h, 2, 6, 7, 7, B);
    px::Vec<float> avg_in;
    avg_in.v.resize((std::size_t)B * 6 * 7 * 7);
    avg.forward(avg_in);
    const bool ok3 = g_regions.size() == 1 && g_regions[0].in == head_in.data() && g_regions[0].out == region.output_.data() &&
                     g_regions[0].num == 2 && g_regions[0].coords == 4 && g_regions[0].classes == 3 && g_regions[0].softmax == 1 &&
                     g_region_decodes.size() == 1 && g_region_decodes[0].pred == region.output_.data() &&
                     g_region_decodes[0].anchors == region.anchors_.data() && g_region_decodes[0].per_image == 0 &&
                     g_region_decodes[0].w == 416.0f && g_region_decodes[0].h == 320.0f && g_region_decodes[0].capacity == 64 &&
                     found.empty() && g_softmaxes.size() == 1 && g_softmaxes[0].in == soft_in.data() && g_softmaxes[0].inputs == 10 &&
                     g_softmaxes[0].groups == 2 && g_softmaxes[0].temp == 0.5f && g_avgs.size() == 1 && g_avgs[0].x == avg_in.data() &&
                     g_avgs[0].y == avg.output_.data() && g_avgs[0].ybs == 6 && g_avgs[0].c == 6 && g_avgs[0].h == 7 && g_avgs[0].w == 7;
    std::printf("%s: region=%zu region_decode=%zu softmax=%zu avgpool=%zu\n", ok3 ? "ok" : "MISMATCH", g_regions.size(),
                g_region_decodes.size(), g_softmaxes.size(), g_avgs.size());
    if (!ok3) return 1;

    // connected layer: the conv epilogue on a 1x1 map, in place; YOLOv1 head decode
    const int before = g_epilogues;
    px::ConnLayer conn(h, 3, 1470, B, false);
    conn.forwardEpilogue();
    px::DetectLayer det(h, 4, 1470, 1, 1, B);
    det.pxeCapacity_ = (long long)B * 7 * 7 * 2;
    det.pxeDets_.v.resize((std::size_t)det.pxeCapacity_ * sizeof(pxe_detection));
    det.pxeCount_.v.resize(1);
    det.addDetects(found, 448, 448, 0.2f);
    const pxe_epilogue_desc& ce = g_last_epilogue;
    const bool ok4 = g_epilogues == before + 1 && ce.x == conn.output_.data() && ce.y == conn.output_.data() && ce.channels == 1470 &&
                     ce.height == 1 && ce.width == 1 && ce.bias == conn.biases_.data() && ce.gamma == nullptr && ce.act == PXE_ACT_RELU &&
                     g_detects.size() == 1 && g_detects[0].pred == det.output_.data() && g_detects[0].pbs == 1470 && g_detects[0].side == 7 &&
                     g_detects[0].num == 2 && g_detects[0].classes == 20 && g_detects[0].coords == 4 && g_detects[0].squared == 1 &&
                     g_detects[0].w == 448.0f && g_detects[0].capacity == (long long)B * 98;
    std::printf("%s: connected=%d detect=%zu\n", ok4 ? "ok" : "MISMATCH", g_epilogues - before, g_detects.size());
    return ok4 ? 0 : 1;
}
