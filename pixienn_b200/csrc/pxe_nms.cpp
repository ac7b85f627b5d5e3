// Host-side non-maximum suppression with the behaviour of px::nms (src/Box.cpp:56-145):
// stable sort by probability, a cross-class pass that drops near-identical boxes (IoU > 0.9)
// of the same image, then greedy suppression inside each (image, class) group, looking only at
// the first 1024 members of a group.  cv::Rect2f intersection / area follow OpenCV >= 4.5.4
// (core/types.hpp operator&=), the version the reference's CMakeLists.txt:86 requires.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <unordered_map>
#include <vector>

#include "pxe.h"

namespace {

struct Rect { float x, y, w, h; };

inline bool empty(const Rect& r) { return r.w <= 0 || r.h <= 0; }

Rect intersect(const Rect& a, const Rect& b)
{
    if (empty(a) || empty(b)) return {0, 0, 0, 0};
    const Rect& rx_min = (a.x < b.x) ? a : b;
    const Rect& rx_max = (a.x < b.x) ? b : a;
    const Rect& ry_min = (a.y < b.y) ? a : b;
    const Rect& ry_max = (a.y < b.y) ? b : a;
    if ((rx_min.x < 0 && rx_min.x + rx_min.w < rx_max.x) || (ry_min.y < 0 && ry_min.y + ry_min.h < ry_max.y))
        return {0, 0, 0, 0};
    Rect r;
    r.w = std::min(rx_min.w - (rx_max.x - rx_min.x), rx_max.w);
    r.h = std::min(ry_min.h - (ry_max.y - ry_min.y), ry_max.h);
    r.x = rx_max.x;
    r.y = ry_max.y;
    if (empty(r)) return {0, 0, 0, 0};
    return r;
}

inline float area(const Rect& r) { return r.w * r.h; }

float iou(const Rect& a, const Rect& b)
{
    const float inter = area(intersect(a, b));
    const float uni = std::max(0.0f, area(a) + area(b) - inter);
    const float r = inter / uni;
    return (std::isnan(r) || std::isinf(r)) ? 0.0f : r;
}

Rect normalized(const pxe_detection& d)
{
    const float x1 = std::min(d.x, d.x + d.w), y1 = std::min(d.y, d.y + d.h);
    const float x2 = std::max(d.x, d.x + d.w), y2 = std::max(d.y, d.y + d.h);
    return {x1, y1, std::max(0.0f, x2 - x1), std::max(0.0f, y2 - y1)};
}

}  // namespace

extern "C" long long pxe_nms_host(const pxe_detection* dets, long long n, float threshold, pxe_detection* out)
{
    if (n < 0 || (n > 0 && (!dets || !out))) return -PXE_ERR_BAD_ARG;
    if (n == 0) return 0;
    try {
        std::vector<pxe_detection> v(dets, dets + n);
        std::stable_sort(v.begin(), v.end(),
                         [](const pxe_detection& a, const pxe_detection& b) { return a.prob > b.prob; });
        std::vector<Rect> rects(v.size());
        for (size_t i = 0; i < v.size(); ++i) rects[i] = normalized(v[i]);
        std::vector<char> discard(v.size(), 0);

        for (size_t i = 0; i < v.size(); ++i) {
            for (size_t j = 0; j < i; ++j) {
                if (discard[j] || v[i].batch_id != v[j].batch_id || v[i].class_id == v[j].class_id) continue;
                if (iou(rects[i], rects[j]) > 0.9f) { discard[i] = 1; break; }
            }
        }

        std::unordered_map<uint64_t, std::vector<size_t>> groups;
        groups.reserve(v.size());
        for (size_t i = 0; i < v.size(); ++i) {
            const uint64_t key = (static_cast<uint64_t>(static_cast<uint32_t>(v[i].batch_id)) << 32)
                                 | static_cast<uint32_t>(v[i].class_id);
            groups[key].push_back(i);
        }
        std::vector<size_t> kept;
        for (const auto& g : groups) {
            kept.clear();
            const size_t count = std::min<size_t>(g.second.size(), 1024);
            for (size_t pos = 0; pos < count; ++pos) {
                const size_t i = g.second[pos];
                if (discard[i]) continue;
                bool suppressed = false;
                for (size_t j : kept)
                    if (iou(rects[i], rects[j]) > threshold) { suppressed = true; break; }
                if (suppressed) discard[i] = 1; else kept.push_back(i);
            }
        }
        long long m = 0;
        for (size_t i = 0; i < v.size(); ++i)
            if (!discard[i]) out[m++] = v[i];
        return m;
    } catch (...) {
        return -PXE_ERR_UNSUPPORTED;
    }
}
