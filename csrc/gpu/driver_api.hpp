/**
 * The handful of CUDA driver entry points the library needs (virtual memory
 * management and multicast objects), resolved at run time through the runtime's
 * cudaGetDriverEntryPoint. The library therefore has no link-time dependency
 * on libcuda and still loads on a machine without a GPU driver, where only the
 * host backend is used.
 */
#pragma once
#include <cuda.h>
#include <string>

namespace dccl {

struct DriverApi {
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
    CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
    CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
    CUresult (*DeviceGet)(CUdevice*, int);
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*GetErrorString)(CUresult, const char**);
    CUresult (*PointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr);   // optional (lazy registration)
    bool vmm_ok = false;         // all memory-management entry points resolved
    bool multicast_ok = false;   // all multicast entry points resolved
};

/** Resolved once per process; null when the CUDA runtime cannot reach a driver. */
const DriverApi* driver_api(std::string* err);
/** Tests only: make driver_api() hand out `api` (a stand-in for the driver) until called again with nullptr. */
void set_driver_api_override(const DriverApi* api);
std::string cu_error(const DriverApi* d, CUresult r);

} // namespace dccl
