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
#define pxe_conv_epilogue shim_test_conv_epilogue
#define pxe_concat shim_test_concat
#define pxe_yolo_decode shim_test_yolo_decode
#define pxe_centernet_decode shim_test_centernet_decode
static int shim_test_conv_epilogue(pxe_stream_t, const pxe_epilogue_desc* d) { g_last_epilogue = *d; ++g_epilogues; return PXE_OK; }
static int shim_test_concat(pxe_stream_t, int, const float* const*, const long long*, const int*, float*, long long, int, int, int) { ++g_concats; return PXE_OK; }
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
    return ok ? 0 : 1;
}
