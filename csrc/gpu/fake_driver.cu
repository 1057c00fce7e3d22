/**
 * A stand-in for the CUDA driver's memory-management and multicast entry points, built on memfd + mmap, so that the
 * collective plumbing of the symmetric allocator (descriptor export and import over the unix sockets, agreement
 * between the ranks, mapping of every peer's segment, teardown, the failure paths) runs on a machine without a GPU,
 * between real processes and through really shared memory. Only the self test below installs it.
 */
#include "symmem.hpp"
#include "../api/comm.hpp"
#include <sys/mman.h>
#include <unistd.h>
#include <cstring>

namespace dccl {
namespace {

int g_fail_create = 0;     // this rank's cuMemCreate reports out of memory

inline int fd_of(CUmemGenericAllocationHandle h) { return (int)h - 1; }

CUresult f_MemCreate(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp*, unsigned long long) {
    if (g_fail_create) return CUDA_ERROR_OUT_OF_MEMORY;
    const int fd = memfd_create("dccl-fake-segment", 0);
    if (fd < 0 || ftruncate(fd, (off_t)size) != 0) { if (fd >= 0) close(fd); return CUDA_ERROR_OUT_OF_MEMORY; }
    *h = (CUmemGenericAllocationHandle)(fd + 1);
    return CUDA_SUCCESS;
}
CUresult f_MemRelease(CUmemGenericAllocationHandle h) { close(fd_of(h)); return CUDA_SUCCESS; }
CUresult f_MemAddressReserve(CUdeviceptr* p, size_t size, size_t, CUdeviceptr, unsigned long long) {
    void* m = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (m == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
    *p = (CUdeviceptr)m;
    return CUDA_SUCCESS;
}
CUresult f_MemAddressFree(CUdeviceptr p, size_t size) { munmap((void*)p, size); return CUDA_SUCCESS; }
CUresult f_MemMap(CUdeviceptr p, size_t size, size_t, CUmemGenericAllocationHandle h, unsigned long long) {
    return mmap((void*)p, size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd_of(h), 0) == MAP_FAILED ? CUDA_ERROR_INVALID_VALUE : CUDA_SUCCESS;
}
CUresult f_MemUnmap(CUdeviceptr p, size_t size) {
    return mmap((void*)p, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0) == MAP_FAILED ? CUDA_ERROR_INVALID_VALUE : CUDA_SUCCESS;
}
CUresult f_MemSetAccess(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) { return CUDA_SUCCESS; }
CUresult f_Export(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType, unsigned long long) {
    const int d = dup(fd_of(h));
    if (d < 0) return CUDA_ERROR_INVALID_VALUE;
    *(int*)out = d;
    return CUDA_SUCCESS;
}
CUresult f_Import(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType) {
    const int d = dup((int)(uintptr_t)os_handle);
    if (d < 0) return CUDA_ERROR_INVALID_VALUE;
    *h = (CUmemGenericAllocationHandle)(d + 1);
    return CUDA_SUCCESS;
}
CUresult f_Granularity(size_t* g, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) { *g = 2u << 20; return CUDA_SUCCESS; }
CUresult f_AddressRange(CUdeviceptr*, size_t*, CUdeviceptr) { return CUDA_ERROR_INVALID_VALUE; }
CUresult f_McCreate(CUmemGenericAllocationHandle* h, const CUmulticastObjectProp* p) { return f_MemCreate(h, p->size, nullptr, 0); }
CUresult f_McAddDevice(CUmemGenericAllocationHandle, CUdevice) { return CUDA_SUCCESS; }
CUresult f_McBind(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) { return CUDA_SUCCESS; }
CUresult f_McUnbind(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) { return CUDA_SUCCESS; }
CUresult f_McGranularity(size_t* g, const CUmulticastObjectProp*, CUmulticastGranularity_flags) { *g = 2u << 20; return CUDA_SUCCESS; }
CUresult f_DeviceGet(CUdevice* d, int ordinal) { *d = ordinal; return CUDA_SUCCESS; }
CUresult f_DeviceGetAttribute(int* v, CUdevice_attribute, CUdevice) { *v = 1; return CUDA_SUCCESS; }   // everything asked for is supported
CUresult f_ErrorString(CUresult, const char** s) { *s = "stand-in driver error"; return CUDA_SUCCESS; }

const DriverApi* fake_api() {
    static DriverApi a;
    a.MemCreate = f_MemCreate; a.MemRelease = f_MemRelease; a.MemAddressReserve = f_MemAddressReserve;
    a.MemAddressFree = f_MemAddressFree; a.MemMap = f_MemMap; a.MemUnmap = f_MemUnmap; a.MemSetAccess = f_MemSetAccess;
    a.MemExportToShareableHandle = f_Export; a.MemImportFromShareableHandle = f_Import;
    a.MemGetAllocationGranularity = f_Granularity; a.MemGetAddressRange = f_AddressRange;
    a.MulticastCreate = f_McCreate; a.MulticastAddDevice = f_McAddDevice; a.MulticastBindMem = f_McBind;
    a.MulticastUnbind = f_McUnbind; a.MulticastGetGranularity = f_McGranularity;
    a.DeviceGet = f_DeviceGet; a.DeviceGetAttribute = f_DeviceGetAttribute; a.GetErrorString = f_ErrorString;
    a.vmm_ok = true; a.multicast_ok = true;
    return &a;
}

} // namespace
} // namespace dccl

extern "C" {

/**
 * Self test of the symmetric allocator over the stand-in driver (no GPU): every rank allocates a segment, fills its
 * own copy with a pattern and reads every peer's copy through its own mapping of it. With `fail_rank` >= 0 that
 * rank's cuMemCreate fails: every rank must then come back with a failure (the cudaIpc fall-back cannot work
 * without a GPU either) and nobody may hang. Returns 0 when things went as they should.
 */
int dccl_selftest_symmem(void* comm, int fail_rank) {
    using namespace dccl;
    dcclComm* c = (dcclComm*)comm;
    if (!c) return -1;
    Bootstrap& bs = c->bs;
    const int n = bs.world(), r = bs.rank();
    if (n > kMaxPeers) return -1;
    set_driver_api_override(fake_api());
    g_fail_create = fail_rank == r ? 1 : 0;
    int rc = 0;
    {
        SymAllocator sa(&bs, 0);
        SymSegment seg;
        std::string err;
        if (!sa.uses_vmm()) rc = -2;
        else {
            const bool ok = sa.alloc(3u << 20, true, &seg, &err);
            if (fail_rank >= 0 && fail_rank < n) rc = ok ? -3 : 0;
            else if (!ok) rc = -4;
            else {
                if (seg.size < (3u << 20) || (n > 1 && !seg.mc_base)) rc = -5;
                memset(seg.base[r], 0x10 + r, seg.size);
                if (!bs.barrier()) rc = -6;
                for (int p = 0; p < n && rc == 0; p++)
                    if ((unsigned char)seg.base[p][0] != 0x10 + p || (unsigned char)seg.base[p][seg.size - 1] != 0x10 + p) rc = 100 + p;
                if (!bs.barrier() && rc == 0) rc = -6;
                sa.free(&seg);
            }
        }
    }
    g_fail_create = 0;
    set_driver_api_override(nullptr);
    return rc;
}

} // extern "C"
