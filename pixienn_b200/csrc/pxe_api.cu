// Library-wide pieces of the C ABI: version, per-thread error text, cached device properties.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "pxe_common.cuh"
#include "pxe_debug.h"

namespace pxe {

namespace {
thread_local char g_error[512] = "";
constexpr int kMaxDevices = 64;
std::mutex g_info_mutex;
bool g_info_valid[kMaxDevices];
DeviceInfo g_info[kMaxDevices];
}  // namespace

int set_error(int status, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

int device_info(DeviceInfo* out)
{
    int dev = 0;
    PXE_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return set_error(PXE_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_info_mutex);
    if (!g_info_valid[dev]) {
        DeviceInfo di{};
        PXE_CUDA_OK(cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev));
        PXE_CUDA_OK(cudaDeviceGetAttribute(&di.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        g_info[dev] = di;
        g_info_valid[dev] = true;
    }
    *out = g_info[dev];
    return PXE_OK;
}

}  // namespace pxe

// ---------------------------------------------------------------- the bounds-checked build (include/pxe_debug.h)
#ifdef PXE_BOUNDS_CHECK
namespace pxe {
namespace {
struct BoundsState {
    std::vector<void (*)(BoundsTable*)> units;                              // one attach function per translation unit
    std::vector<std::pair<unsigned long long, unsigned long long>> user, internal;
    BoundsTable* device_table = nullptr;
    bool armed = false;
};
BoundsState& bounds_state() { static BoundsState s; return s; }

int bounds_upload()
{
    BoundsState& st = bounds_state();
    PXE_CUDA_OK(cudaDeviceSynchronize());
    if (st.device_table == nullptr) {
        PXE_CUDA_OK(cudaMalloc(&st.device_table, sizeof(BoundsTable)));
        PXE_CUDA_OK(cudaMemset(st.device_table, 0, sizeof(BoundsTable)));
        for (auto attach : st.units) attach(st.device_table);
        PXE_CUDA_OK(cudaGetLastError());
    }
    std::vector<std::pair<unsigned long long, unsigned long long>> spans;
    if (st.armed) {
        spans = st.user;
        spans.insert(spans.end(), st.internal.begin(), st.internal.end());
        std::sort(spans.begin(), spans.end());
    }
    PXE_REQUIRE((int)spans.size() <= kBoundsMaxSpans, "pxe_debug_set_allocations: %zu ranges, at most %d", spans.size(), kBoundsMaxSpans);
    std::vector<unsigned long long> start(spans.size()), end(spans.size());
    for (size_t i = 0; i < spans.size(); ++i) { start[i] = spans[i].first; end[i] = spans[i].second; }
    const int n = (int)spans.size();
    if (n > 0) {
        PXE_CUDA_OK(cudaMemcpy(st.device_table->start, start.data(), n * sizeof(unsigned long long), cudaMemcpyHostToDevice));
        PXE_CUDA_OK(cudaMemcpy(st.device_table->end, end.data(), n * sizeof(unsigned long long), cudaMemcpyHostToDevice));
    }
    PXE_CUDA_OK(cudaMemcpy(&st.device_table->n, &n, sizeof(int), cudaMemcpyHostToDevice));
    return PXE_OK;
}
}  // namespace

void bounds_register_unit(void (*attach)(BoundsTable*)) { bounds_state().units.push_back(attach); }

// Memory the library owns and its kernels reach through a pointer.
int bounds_add_internal(const void* p, size_t bytes)
{
    BoundsState& st = bounds_state();
    const unsigned long long a = (unsigned long long)reinterpret_cast<uintptr_t>(p);
    for (const auto& s : st.internal) if (s.first == a) return PXE_OK;
    st.internal.emplace_back(a, a + bytes);
    return st.armed ? bounds_upload() : PXE_OK;
}
}  // namespace pxe

extern "C" int pxe_debug_bounds_checked(void) { return 1; }

extern "C" int pxe_debug_set_allocations(const void* const* starts, const size_t* bytes, int count)
{
    using namespace pxe;
    PXE_REQUIRE(count >= 0 && (count == 0 || (starts && bytes)), "pxe_debug_set_allocations: null array or negative count");
    BoundsState& st = bounds_state();
    st.user.clear();
    for (int i = 0; i < count; ++i) {
        const unsigned long long a = (unsigned long long)reinterpret_cast<uintptr_t>(starts[i]);
        if (bytes[i] > 0) st.user.emplace_back(a, a + bytes[i]);
    }
    st.armed = count > 0;
    return bounds_upload();
}

extern "C" int pxe_debug_read_report(pxe_bounds_report* out, int reset)
{
    using namespace pxe;
    PXE_REQUIRE(out != nullptr, "pxe_debug_read_report: null report");
    BoundsState& st = bounds_state();
    std::memset(out, 0, sizeof(*out));
    PXE_CUDA_OK(cudaDeviceSynchronize());
    if (st.device_table == nullptr) return PXE_OK;
    static BoundsTable host;                                                // 64 KB: not on the stack
    PXE_CUDA_OK(cudaMemcpy(&host, st.device_table, sizeof(BoundsTable), cudaMemcpyDeviceToHost));
    out->violations = host.violations;
    out->bytes = host.bad_bytes;
    out->address = host.bad_address;
    out->line = host.bad_line;
    out->is_store = host.bad_store;
    out->misaligned = host.bad_misaligned;
    std::memcpy(out->file, host.bad_file, sizeof(out->file));
    out->file[sizeof(out->file) - 1] = 0;
    if (reset) {
        const size_t off = offsetof(BoundsTable, violations);
        PXE_CUDA_OK(cudaMemset(reinterpret_cast<char*>(st.device_table) + off, 0, sizeof(BoundsTable) - off));
    }
    return PXE_OK;
}
#else
extern "C" int pxe_debug_bounds_checked(void) { return 0; }

extern "C" int pxe_debug_set_allocations(const void* const*, const size_t*, int)
{
    return pxe::set_error(PXE_ERR_UNSUPPORTED, "pxe_debug_set_allocations: this library was built without PXE_BOUNDS_CHECK");
}

extern "C" int pxe_debug_read_report(pxe_bounds_report*, int)
{
    return pxe::set_error(PXE_ERR_UNSUPPORTED, "pxe_debug_read_report: this library was built without PXE_BOUNDS_CHECK");
}
#endif

extern "C" int pxe_version(void) { return 100; }

extern "C" const char* pxe_last_error_string(void) { return pxe::g_error; }

extern "C" const char* pxe_status_string(int status)
{
    switch (status) {
    case PXE_OK: return "ok";
    case PXE_ERR_BAD_ARG: return "bad argument";
    case PXE_ERR_UNSUPPORTED: return "unsupported";
    case PXE_ERR_CUDA: return "CUDA error";
    case PXE_ERR_WORKSPACE: return "workspace too small";
    default: return "unknown status";
    }
}
