// The fusion planner behind pxe_plan.h: one walk over the layer list decides what the reference
// leaves to run time, layer by layer (Model<D>::forward, include/Model.h:1748-1756):
//   * a route with one source is an alias of that source (include/RouteLayer.h:40-80);
//   * every source of a wider route gets a channel range of the route's concat buffer and is stored
//     there by its producer, so the route itself runs nothing (include/cuda/RouteLayer.h:21-44);
//   * a conv whose only reader is the shortcut that follows takes the residual add into its epilogue
//     (include/cuda/ShortcutLayer.h:23-34); a conv followed by a 2x2 stride-2 max pool takes the pool
//     (include/cuda/MaxPoolLayer.h:36-42);
//   * consecutive stride-1 "same" pools of one tensor (SPP) read it once;
//   * a linear, bias-only conv that feeds a YOLO layer keeps its raw output: bias and logistic are
//     applied where the decode reads it (include/cuda/YoloLayer.h:70-96).
// Host code only.
#include <cstdarg>
#include <cstdio>
#include <map>
#include <set>
#include <vector>

#include "pxe.h"
#include "pxe_plan.h"

namespace pxe {
int set_error(int status, const char* fmt, ...);
}

struct pxe_plan {
    std::vector<pxe_step> steps;
    std::vector<int> alias;            // per layer, -1 = none
    std::vector<int> concat_channels;  // per layer, 0 = owns no concat buffer
    std::vector<int> last_use;         // per layer, -1 = never read
    int last_use_input = -1;           // the network input (layer -1)
    pxe_plan_stats stats{};
};

namespace {

struct Slot { int route, offset; };

bool reads_dense_only(int type)
{
    // cuDNN convolutions and the heads read dense tensors; everything on the epilogue path takes a
    // batch stride and can read a channel slot of a wider buffer
    switch (type) {
    case PXE_LAYER_CONV: case PXE_LAYER_CONNECTED: case PXE_LAYER_YOLO: case PXE_LAYER_CENTERNET:
    case PXE_LAYER_REGION: case PXE_LAYER_SOFTMAX: case PXE_LAYER_AVGPOOL: case PXE_LAYER_DROPOUT:
    case PXE_LAYER_DETECTION:
        return true;
    default:
        return false;
    }
}

struct Builder {
    const pxe_layer_desc* L;
    int n;
    bool fuse, raw_heads;
    std::vector<std::vector<int>> cons;          // index t + 1 -> layers reading tensor t
    std::map<int, int> alias;
    std::map<int, std::vector<Slot>> slots;      // tensor -> concat slots it is stored into
    std::set<int> absorbed;
    pxe_plan* plan;

    int resolve(int i) const
    {
        for (auto it = alias.find(i); it != alias.end(); it = alias.find(i)) i = it->second;
        return i;
    }
    // who really reads tensor t, looking through alias routes
    void real_consumers(int t, std::vector<int>& out) const
    {
        for (int c : cons[t + 1]) {
            auto it = alias.find(c);
            if (it != alias.end() && it->second == t) real_consumers(c, out);
            else out.push_back(c);
        }
    }
    std::vector<int> real_consumers(int t) const
    {
        std::vector<int> out;
        real_consumers(t, out);
        return out;
    }
    bool needs_dense(int t, const std::vector<int>& readers) const
    {
        if (!slots.count(t)) return true;
        for (int r : readers)
            if (reads_dense_only(L[r].type)) return true;
        return false;
    }
    int dests_for(int t, const std::vector<int>& readers, pxe_dest* out) const
    {
        int k = 0;
        if (needs_dense(t, readers)) out[k++] = pxe_dest{0, -1, 0};
        auto it = slots.find(t);
        if (it != slots.end())
            for (const Slot& s : it->second) {
                if (k == PXE_PLAN_MAX_DESTS) return -1;
                out[k++] = pxe_dest{1, s.route, s.offset};
            }
        return k;
    }
    static pxe_step blank(int op, int layer)
    {
        pxe_step st{};
        st.op = op; st.layer = layer;
        st.fused_shortcut = -1; st.fused_pool = -1; st.keep_full = 1;
        return st;
    }
    static bool same_shape(const pxe_layer_desc& a, const pxe_layer_desc& b)
    {
        return a.out_channels == b.out_channels && a.out_height == b.out_height && a.out_width == b.out_width;
    }
    static bool spp_pool(const pxe_layer_desc& l) { return l.type == PXE_LAYER_MAXPOOL && l.stride == 1 && l.padding == l.kernel - 1; }

    int run()
    {
        cons.assign(n + 1, {});
        for (int i = 0; i < n; ++i)
            for (int s = 0; s < L[i].n_sources; ++s) cons[L[i].sources[s] + 1].push_back(i);

        // 1. fan-in-1 routes are pure aliases
        if (fuse)
            for (int i = 0; i < n; ++i)
                if (L[i].type == PXE_LAYER_ROUTE && L[i].n_sources == 1) alias[i] = L[i].sources[0];
        // 2. every source of a wider route gets a channel range of that route's buffer
        if (fuse)
            for (int i = 0; i < n; ++i)
                if (L[i].type == PXE_LAYER_ROUTE && L[i].n_sources > 1) {
                    int off = 0;
                    for (int s = 0; s < L[i].n_sources; ++s) {
                        const int src = L[i].sources[s];
                        slots[resolve(src)].push_back(Slot{i, off});
                        off += L[src].out_channels;
                    }
                    plan->concat_channels[i] = off;
                }

        pxe_plan_stats& stats = plan->stats;
        for (int i = 0; i < n; ++i) {
            const pxe_layer_desc& l = L[i];
            if (absorbed.count(i)) continue;
            if (alias.count(i)) {
                pxe_step st = blank(PXE_STEP_ALIAS, i);
                st.n_inputs = 1; st.inputs[0] = alias[i];
                plan->steps.push_back(st);
                ++stats.routes_aliased;
                continue;
            }
            switch (l.type) {
            case PXE_LAYER_CONV: {
                pxe_step st = blank(PXE_STEP_CONV, i);
                st.n_inputs = 1; st.inputs[0] = resolve(l.sources[0]);
                int out_t = i;
                std::vector<int> readers = real_consumers(i);
                const pxe_layer_desc* nxt = i + 1 < n ? &L[i + 1] : nullptr;
                if (fuse && nxt && readers.size() == 1 && readers[0] == i + 1) {
                    if (nxt->type == PXE_LAYER_SHORTCUT && nxt->sources[0] == i && nxt->sources[1] >= 0
                        && same_shape(L[nxt->sources[1]], l)) {
                        st.fused_shortcut = i + 1;
                        st.inputs[st.n_inputs++] = resolve(nxt->sources[1]);
                        absorbed.insert(i + 1);
                        alias[i] = i + 1;            // the conv's own value is never materialised
                        out_t = i + 1;
                        ++stats.fused_shortcut;
                    } else if (raw_heads && nxt->type == PXE_LAYER_YOLO && !l.batch_norm && l.activation == PXE_ACT_LINEAR) {
                        st.head_raw = 1;
                        ++stats.raw_heads;
                    }
                }
                bool next_reads = false;
                for (int r : readers) next_reads = next_reads || r == i + 1;
                if (fuse && st.fused_shortcut < 0 && nxt && nxt->type == PXE_LAYER_MAXPOOL && nxt->kernel == 2
                    && nxt->stride == 2 && (nxt->padding == 0 || nxt->padding == 1) && next_reads) {
                    std::vector<int> others;
                    for (int r : readers)
                        if (r != i + 1) others.push_back(r);
                    const bool covered = 2 * nxt->out_height >= l.out_height && 2 * nxt->out_width >= l.out_width;
                    if (covered || others.empty()) {
                        st.fused_pool = i + 1;
                        st.keep_full = (!others.empty() || slots.count(i)) ? 1 : 0;
                        st.n_pool_dests = dests_for(i + 1, real_consumers(i + 1), st.pool_dests);
                        if (st.n_pool_dests < 0) return too_many(i + 1);
                        absorbed.insert(i + 1);
                        ++stats.fused_pool;
                        readers = others;
                    }
                }
                st.n_dests = dests_for(out_t, out_t != i ? real_consumers(out_t) : readers, st.dests);
                if (st.n_dests < 0) return too_many(out_t);
                if (st.fused_pool >= 0 && !st.keep_full) st.n_dests = 0;
                plan->steps.push_back(st);
                break;
            }
            case PXE_LAYER_MAXPOOL: {
                const int src = resolve(l.sources[0]);
                std::vector<int> group{i};
                if (fuse && spp_pool(l)) {
                    // later stride-1 pools of the same tensor, separated only by alias routes
                    for (int j = i + 1; j < n;) {
                        if (alias.count(j)) { ++j; continue; }
                        if (spp_pool(L[j]) && resolve(L[j].sources[0]) == src && (int)group.size() < PXE_PLAN_MAX_SPP) {
                            group.push_back(j++);
                            continue;
                        }
                        break;
                    }
                }
                if (group.size() > 1) {
                    pxe_step st = blank(PXE_STEP_SPP, i);
                    st.n_inputs = 1; st.inputs[0] = src;
                    st.n_spp = (int)group.size();
                    for (int g = 0; g < st.n_spp; ++g) {
                        st.spp_layers[g] = group[g];
                        st.n_spp_dests[g] = dests_for(group[g], real_consumers(group[g]), st.spp_dests[g]);
                        if (st.n_spp_dests[g] < 0) return too_many(group[g]);
                        if (g > 0) absorbed.insert(group[g]);
                    }
                    plan->steps.push_back(st);
                    ++stats.spp_blocks;
                } else {
                    pxe_step st = blank(PXE_STEP_MAXPOOL, i);
                    st.n_inputs = 1; st.inputs[0] = src;
                    st.n_dests = dests_for(i, real_consumers(i), st.dests);
                    if (st.n_dests < 0) return too_many(i);
                    plan->steps.push_back(st);
                }
                break;
            }
            case PXE_LAYER_UPSAMPLE:
            case PXE_LAYER_SHORTCUT: {
                pxe_step st = blank(l.type == PXE_LAYER_UPSAMPLE ? PXE_STEP_UPSAMPLE : PXE_STEP_SHORTCUT, i);
                st.n_inputs = l.type == PXE_LAYER_UPSAMPLE ? 1 : 2;
                for (int k = 0; k < st.n_inputs; ++k) st.inputs[k] = resolve(l.sources[k]);
                st.n_dests = dests_for(i, real_consumers(i), st.dests);
                if (st.n_dests < 0) return too_many(i);
                plan->steps.push_back(st);
                break;
            }
            case PXE_LAYER_ROUTE: {
                if (fuse) {
                    // every source already stored into this route's buffer; when the route is itself a
                    // source of a later route, its buffer is copied into that slot
                    pxe_step st = blank(PXE_STEP_ALIAS, i);
                    auto it = slots.find(i);
                    if (it != slots.end())
                        for (const Slot& s : it->second) {
                            if (st.n_dests == PXE_PLAN_MAX_DESTS) return too_many(i);
                            st.dests[st.n_dests++] = pxe_dest{1, s.route, s.offset};
                        }
                    plan->steps.push_back(st);
                    ++stats.routes_eliminated;
                } else {
                    pxe_step st = blank(PXE_STEP_CONCAT, i);
                    if (l.n_sources > 2) {
                        // the step record lists two inputs; the caller reads the full source list from its layer
                        st.n_inputs = 2;
                    } else {
                        st.n_inputs = l.n_sources;
                    }
                    for (int k = 0; k < st.n_inputs; ++k) st.inputs[k] = l.sources[k];
                    st.n_dests = 1; st.dests[0] = pxe_dest{0, -1, 0};
                    plan->steps.push_back(st);
                    ++stats.concat_copies;
                }
                break;
            }
            case PXE_LAYER_YOLO: case PXE_LAYER_CENTERNET: case PXE_LAYER_REGION: case PXE_LAYER_SOFTMAX:
            case PXE_LAYER_AVGPOOL: case PXE_LAYER_DROPOUT: case PXE_LAYER_CONNECTED: case PXE_LAYER_DETECTION: {
                pxe_step st = blank(PXE_STEP_HEAD, i);
                st.n_inputs = 1; st.inputs[0] = resolve(l.sources[0]);
                // a dense tensor of its own, plus a copy into every route buffer that concatenates it
                st.n_dests = 1; st.dests[0] = pxe_dest{0, -1, 0};
                {
                    auto it = slots.find(i);
                    if (it != slots.end())
                        for (const Slot& sl : it->second) {
                            if (st.n_dests == PXE_PLAN_MAX_DESTS) return too_many(i);
                            st.dests[st.n_dests++] = pxe_dest{1, sl.route, sl.offset};
                        }
                }
                if (l.type == PXE_LAYER_YOLO && !plan->steps.empty() && plan->steps.back().op == PXE_STEP_CONV
                    && plan->steps.back().head_raw)
                    st.head_raw = 1;
                plan->steps.push_back(st);
                break;
            }
            default:
                return pxe::set_error(PXE_ERR_BAD_ARG, "plan: layer %d has unknown type %d", i, l.type);
            }
        }
        for (const auto& a : alias) plan->alias[a.first] = a.second;
        for (size_t si = 0; si < plan->steps.size(); ++si) {
            const pxe_step& st = plan->steps[si];
            // a route step that really copies reads every source of its layer
            if (st.op == PXE_STEP_CONCAT)
                for (int k = 0; k < L[st.layer].n_sources; ++k) touch(L[st.layer].sources[k], (int)si);
            for (int k = 0; k < st.n_inputs; ++k) touch(st.inputs[k], (int)si);
        }
        return PXE_OK;
    }
    void touch(int t, int si)
    {
        if (t < 0) plan->last_use_input = si;
        else plan->last_use[t] = si;
    }
    int too_many(int t) const
    {
        return pxe::set_error(PXE_ERR_UNSUPPORTED, "plan: tensor %d is stored into more than %d places", t, PXE_PLAN_MAX_DESTS);
    }
};

int validate(const pxe_layer_desc* L, int n)
{
    for (int i = 0; i < n; ++i) {
        const pxe_layer_desc& l = L[i];
        if (l.n_sources < 1 || l.n_sources > PXE_PLAN_MAX_SOURCES)
            return pxe::set_error(PXE_ERR_BAD_ARG, "plan: layer %d has %d sources (1..%d)", i, l.n_sources, PXE_PLAN_MAX_SOURCES);
        for (int s = 0; s < l.n_sources; ++s)
            if (l.sources[s] < -1 || l.sources[s] >= i)
                return pxe::set_error(PXE_ERR_BAD_ARG, "plan: layer %d reads layer %d, which does not precede it", i, l.sources[s]);
        if (l.type == PXE_LAYER_SHORTCUT && l.n_sources != 2)
            return pxe::set_error(PXE_ERR_BAD_ARG, "plan: shortcut layer %d needs two sources (previous, from)", i);
        if (l.type == PXE_LAYER_ROUTE)
            for (int s = 0; s < l.n_sources; ++s)
                if (l.sources[s] < 0)
                    return pxe::set_error(PXE_ERR_BAD_ARG, "plan: route layer %d reads the network input", i);
        if (l.out_channels <= 0 || l.out_height <= 0 || l.out_width <= 0)
            return pxe::set_error(PXE_ERR_BAD_ARG, "plan: layer %d has an empty output shape", i);
    }
    return PXE_OK;
}

}  // namespace

extern "C" int pxe_plan_build(const pxe_layer_desc* layers, int n_layers, int fuse, int raw_heads, pxe_plan** out)
{
    if (!out) return pxe::set_error(PXE_ERR_BAD_ARG, "plan: out is null");
    *out = nullptr;
    if (!layers || n_layers <= 0) return pxe::set_error(PXE_ERR_BAD_ARG, "plan: no layers");
    int rc = validate(layers, n_layers);
    if (rc != PXE_OK) return rc;
    pxe_plan* plan = new pxe_plan;
    plan->alias.assign(n_layers, -1);
    plan->concat_channels.assign(n_layers, 0);
    plan->last_use.assign(n_layers, -1);
    Builder b{layers, n_layers, fuse != 0, raw_heads != 0, {}, {}, {}, {}, plan};
    rc = b.run();
    if (rc != PXE_OK) {
        delete plan;
        return rc;
    }
    *out = plan;
    return PXE_OK;
}

extern "C" void pxe_plan_destroy(pxe_plan* plan) { delete plan; }

extern "C" int pxe_plan_step_count(const pxe_plan* plan) { return plan ? (int)plan->steps.size() : 0; }

extern "C" const pxe_step* pxe_plan_step(const pxe_plan* plan, int i)
{
    if (!plan || i < 0 || i >= (int)plan->steps.size()) return nullptr;
    return &plan->steps[i];
}

extern "C" int pxe_plan_alias(const pxe_plan* plan, int layer)
{
    if (!plan || layer < 0 || layer >= (int)plan->alias.size()) return -1;
    return plan->alias[layer];
}

extern "C" int pxe_plan_concat_channels(const pxe_plan* plan, int route)
{
    if (!plan || route < 0 || route >= (int)plan->concat_channels.size()) return 0;
    return plan->concat_channels[route];
}

extern "C" int pxe_plan_last_use(const pxe_plan* plan, int layer)
{
    if (!plan) return -1;
    if (layer == -1) return plan->last_use_input;
    if (layer < 0 || layer >= (int)plan->last_use.size()) return -1;
    return plan->last_use[layer];
}

extern "C" void pxe_plan_get_stats(const pxe_plan* plan, pxe_plan_stats* stats)
{
    if (plan && stats) *stats = plan->stats;
}
