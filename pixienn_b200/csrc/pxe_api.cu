// Library-wide pieces of the C ABI: version, per-thread error text, cached device properties.
#include <mutex>

#include "pxe_common.cuh"

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
