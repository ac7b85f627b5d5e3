// A C++ client of libpxe.so the way a PixieNN build would be one: includes the C headers and the
// px:: declarations, links the shared library, and drives the host-only entry points (no GPU needed):
// the planner on a five-layer graph and the host NMS.  Prints what it found; exit code 0 = all as expected.
#include <cstdio>
#include <vector>

#include "pxe.h"
#include "pxe_compat.hpp"
#include "pxe_plan.h"

static pxe_layer_desc layer(int type, int c, int h, int w, int src, int kernel = 1, int stride = 1, int pad = 0,
                            int bn = 0, int act = PXE_ACT_LINEAR)
{
    pxe_layer_desc d{};
    d.type = type; d.out_channels = c; d.out_height = h; d.out_width = w;
    d.kernel = kernel; d.stride = stride; d.padding = pad; d.batch_norm = bn; d.activation = act;
    d.n_sources = 1; d.sources[0] = src;
    return d;
}

int main()
{
    if (pxe_version() < 100) return 1;
    // conv -> maxpool 2/2 -> conv -> shortcut(from 1) -> conv(linear) -> yolo
    std::vector<pxe_layer_desc> L;
    L.push_back(layer(PXE_LAYER_CONV, 16, 32, 32, -1, 3, 1, 1, 1, PXE_ACT_LEAKY));
    L.push_back(layer(PXE_LAYER_MAXPOOL, 16, 16, 16, 0, 2, 2, 1));
    L.push_back(layer(PXE_LAYER_CONV, 16, 16, 16, 1, 3, 1, 1, 1, PXE_ACT_LEAKY));
    pxe_layer_desc sc = layer(PXE_LAYER_SHORTCUT, 16, 16, 16, 2);
    sc.n_sources = 2; sc.sources[1] = 1;
    L.push_back(sc);
    L.push_back(layer(PXE_LAYER_CONV, 24, 16, 16, 3, 1, 1, 0, 0, PXE_ACT_LINEAR));
    L.push_back(layer(PXE_LAYER_YOLO, 24, 16, 16, 4));
    pxe_plan* plan = nullptr;
    if (pxe_plan_build(L.data(), (int)L.size(), 1, 1, &plan) != PXE_OK) {
        std::printf("plan failed: %s\n", pxe_last_error_string());
        return 2;
    }
    pxe_plan_stats st{};
    pxe_plan_get_stats(plan, &st);
    const int steps = pxe_plan_step_count(plan);
    std::printf("steps=%d fused_pool=%d fused_shortcut=%d raw_heads=%d\n", steps, st.fused_pool, st.fused_shortcut, st.raw_heads);
    const pxe_step* first = pxe_plan_step(plan, 0);
    const bool ok = steps == 4 && st.fused_pool == 1 && st.fused_shortcut == 1 && st.raw_heads == 1
                    && first && first->op == PXE_STEP_CONV && first->fused_pool == 1 && first->keep_full == 0
                    && pxe_plan_alias(plan, 2) == 3;
    pxe_plan_destroy(plan);
    if (!ok) return 3;

    // two overlapping boxes of one class, one box elsewhere
    pxe_detection d[3] = {{0.10f, 0.10f, 0.30f, 0.30f, 0.9f, 1, 0, 0}, {0.12f, 0.11f, 0.30f, 0.30f, 0.8f, 1, 0, 1},
                          {0.60f, 0.60f, 0.20f, 0.20f, 0.7f, 1, 0, 2}};
    pxe_detection out[3];
    const long long kept = pxe_nms_host(d, 3, 0.4f, out);
    std::printf("nms kept=%lld\n", kept);
    if (kept != 2 || out[0].source != 0 || out[1].source != 2) return 4;

    // the link-compatible tier resolves: taking the addresses is enough to make the linker look them up
    auto f1 = static_cast<void (*)(float*, const float*, int, int, int)>(&px::addBiasGpu);
    auto f2 = static_cast<void (*)(const float*, float*, int, int, int, int)>(&px::yoloActivateGpu);
    std::printf("px:: symbols %s\n", (f1 && f2) ? "resolved" : "missing");
    return (f1 && f2) ? 0 : 5;
}
