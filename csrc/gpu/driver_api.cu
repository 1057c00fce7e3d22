#include "driver_api.hpp"
#include <cuda_runtime_api.h>
#include <mutex>

namespace dccl {

static DriverApi g_api;
static bool g_tried = false, g_have = false;
static std::string g_err;
static std::mutex g_mu;

template <typename F>
static bool resolve(const char* name, F* out) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) { cudaGetLastError(); *out = nullptr; return false; }
    *out = reinterpret_cast<F>(fn);
    return true;
}

static const DriverApi* g_override = nullptr;

void set_driver_api_override(const DriverApi* api) {
    std::lock_guard<std::mutex> g(g_mu);
    g_override = api;
}

const DriverApi* driver_api(std::string* err) {
    std::lock_guard<std::mutex> g(g_mu);
    if (g_override) return g_override;
    if (!g_tried) {
        g_tried = true;
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
            cudaGetLastError();
            g_err = "no CUDA device or driver";
        } else {
            bool vmm = true, mc = true;
            vmm &= resolve("cuMemCreate", &g_api.MemCreate);
            vmm &= resolve("cuMemRelease", &g_api.MemRelease);
            vmm &= resolve("cuMemAddressReserve", &g_api.MemAddressReserve);
            vmm &= resolve("cuMemAddressFree", &g_api.MemAddressFree);
            vmm &= resolve("cuMemMap", &g_api.MemMap);
            vmm &= resolve("cuMemUnmap", &g_api.MemUnmap);
            vmm &= resolve("cuMemSetAccess", &g_api.MemSetAccess);
            vmm &= resolve("cuMemExportToShareableHandle", &g_api.MemExportToShareableHandle);
            vmm &= resolve("cuMemImportFromShareableHandle", &g_api.MemImportFromShareableHandle);
            vmm &= resolve("cuMemGetAllocationGranularity", &g_api.MemGetAllocationGranularity);
            vmm &= resolve("cuMemGetAddressRange", &g_api.MemGetAddressRange);
            vmm &= resolve("cuDeviceGet", &g_api.DeviceGet);
            vmm &= resolve("cuDeviceGetAttribute", &g_api.DeviceGetAttribute);
            resolve("cuGetErrorString", &g_api.GetErrorString);
            resolve("cuPointerGetAttribute", &g_api.PointerGetAttribute);
            mc &= resolve("cuMulticastCreate", &g_api.MulticastCreate);
            mc &= resolve("cuMulticastAddDevice", &g_api.MulticastAddDevice);
            mc &= resolve("cuMulticastBindMem", &g_api.MulticastBindMem);
            mc &= resolve("cuMulticastUnbind", &g_api.MulticastUnbind);
            mc &= resolve("cuMulticastGetGranularity", &g_api.MulticastGetGranularity);
            g_api.vmm_ok = vmm;
            g_api.multicast_ok = vmm && mc;
            g_have = true;
        }
    }
    if (!g_have && err) *err = g_err;
    return g_have ? &g_api : nullptr;
}

std::string cu_error(const DriverApi* d, CUresult r) {
    const char* s = nullptr;
    if (d && d->GetErrorString && d->GetErrorString(r, &s) == CUDA_SUCCESS && s) return std::string(s) + " (" + std::to_string((int)r) + ")";
    return "CUDA driver error " + std::to_string((int)r);
}

} // namespace dccl
