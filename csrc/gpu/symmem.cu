#include "symmem.hpp"
#include "../core/config.hpp"
#include "../core/log.hpp"
#include <cuda_runtime_api.h>
#include <cstring>
#include <unistd.h>
#include <vector>

namespace dccl {

static const CUmemAllocationHandleType kFd = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;

bool SymAllocator::agree(bool ok) {
    std::vector<unsigned char> all(n_);
    unsigned char mine = ok ? 1 : 0;
    if (!bs_->allgather(&mine, 1, all.data())) return false;
    for (unsigned char v : all) if (!v) return false;
    return true;
}

SymAllocator::SymAllocator(Bootstrap* bs, int device) : bs_(bs), dev_(device), rank_(bs->rank()), n_(bs->world()) {
    std::string err;
    d_ = driver_api(&err);
    bool vmm = false, mc = false;
    const std::string mode = Config::global().get_str("DCCL/pool_mode", "auto");
    if (d_ && d_->vmm_ok && mode != "ipc") {
        CUdevice cu;
        int a = 0, b = 0, m = 0;
        if (d_->DeviceGet(&cu, device) == CUDA_SUCCESS) {
            d_->DeviceGetAttribute(&a, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cu);
            d_->DeviceGetAttribute(&b, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cu);
            if (d_->multicast_ok) d_->DeviceGetAttribute(&m, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cu);
            vmm = a && b;
            mc = vmm && m && Config::global().get_bool("DCCL/nvls", true) && n_ > 1;
        }
    }
    vmm_ = agree(vmm);
    mc_ = vmm_ && agree(mc);
    dccl_info("symmetric memory: %s handles, multicast %s", vmm_ ? "cuMem file-descriptor" : "cudaIpc", mc_ ? "available" : "not used");
}

bool SymAllocator::alloc(size_t bytes, bool want_mc, SymSegment* seg, std::string* err) {
    *seg = SymSegment();
    seg->requested = bytes;
    if (vmm_) {
        std::string e;
        bool ok = alloc_vmm(bytes, want_mc, seg, &e);
        if (ok) return true;
        // every rank saw the same verdict (alloc_vmm agrees before returning): fall back together
        dccl_warn("cuMem allocation of %zu bytes failed (%s); falling back to cudaIpc", bytes, e.c_str());
        vmm_ = false;
        mc_ = false;
    }
    return alloc_ipc(bytes, seg, err);
}

bool SymAllocator::alloc_vmm(size_t bytes, bool want_mc, SymSegment* seg, std::string* err) {
    const uint32_t tag = next_tag_;
    next_tag_ += 2;
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev_;
    prop.requestedHandleTypes = kFd;
    size_t gran = 2u << 20;
    bool ok = d_->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS;
    if (ok && mc_ && want_mc) {
        CUmulticastObjectProp mp;
        memset(&mp, 0, sizeof(mp));
        mp.numDevices = (unsigned)n_;
        mp.size = bytes;
        mp.handleTypes = kFd;
        size_t mg = 0;
        if (d_->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    }
    const size_t size = (bytes + gran - 1) / gran * gran;
    seg->size = size;
    seg->vmm = true;
    std::string why;
    CUresult r;
    int fd = -1;
    if (ok && (r = d_->MemCreate(&seg->handles[rank_], size, &prop, 0)) != CUDA_SUCCESS) { ok = false; why = "cuMemCreate: " + cu_error(d_, r); }
    if (ok && (r = d_->MemExportToShareableHandle(&fd, seg->handles[rank_], kFd, 0)) != CUDA_SUCCESS) { ok = false; why = "export: " + cu_error(d_, r); }
    // hand my descriptor to every peer, then collect theirs
    if (ok) for (int k = 1; k < n_ && ok; k++) if (!bs_->send_fd((rank_ + k) % n_, fd, tag)) { ok = false; why = "send_fd: " + bs_->last_error(); }
    if (!agree(ok)) {   // nobody waits for a descriptor that will not come
        bs_->discard_fds(tag);   // ... and the descriptors that did come are not left lying around for a later exchange
        if (fd >= 0) ::close(fd);
        if (seg->handles[rank_]) { d_->MemRelease(seg->handles[rank_]); seg->handles[rank_] = 0; }
        if (err) *err = why.empty() ? "a peer could not create or export its segment" : why;
        return false;
    }
    if (fd >= 0) ::close(fd);
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (int p = 0; p < n_ && ok; p++) {
        if (p != rank_) {
            int pfd = -1;
            if (!bs_->recv_fd(p, tag, &pfd, 30000)) { ok = false; why = "recv_fd: " + bs_->last_error(); break; }
            r = d_->MemImportFromShareableHandle(&seg->handles[p], (void*)(uintptr_t)pfd, kFd);
            ::close(pfd);
            if (r != CUDA_SUCCESS) { ok = false; why = "import: " + cu_error(d_, r); break; }
        }
        CUdeviceptr va = 0;
        if ((r = d_->MemAddressReserve(&va, size, gran, 0, 0)) != CUDA_SUCCESS) { ok = false; why = "reserve: " + cu_error(d_, r); break; }
        seg->base[p] = (char*)va;
        if ((r = d_->MemMap(va, size, 0, seg->handles[p], 0)) != CUDA_SUCCESS) { ok = false; why = "map: " + cu_error(d_, r); break; }
        if ((r = d_->MemSetAccess(va, size, &acc, 1)) != CUDA_SUCCESS) { ok = false; why = "set access (peer " + std::to_string(p) + "): " + cu_error(d_, r); break; }
    }
    if (!agree(ok)) {
        bs_->discard_fds(tag);
        SymSegment tmp = *seg;
        tmp.mc_handle = 0;
        // local teardown only: free() would run a barrier the failing path must not depend on
        for (int p = 0; p < n_; p++) {
            if (tmp.base[p]) { d_->MemUnmap((CUdeviceptr)tmp.base[p], size); d_->MemAddressFree((CUdeviceptr)tmp.base[p], size); }
            if (tmp.handles[p]) d_->MemRelease(tmp.handles[p]);
        }
        *seg = SymSegment();
        if (err) *err = why.empty() ? "a peer could not map the segments" : why;
        return false;
    }
    if (mc_ && want_mc) {
        std::string me;
        if (!bind_multicast(seg, &me)) dccl_warn("multicast binding failed (%s); this segment uses peer loads/stores only", me.c_str());
    }
    return true;
}

bool SymAllocator::bind_multicast(SymSegment* seg, std::string* err) {
    const uint32_t tag = next_tag_ - 1;
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)n_;
    mp.size = seg->size;
    mp.handleTypes = kFd;
    bool ok = true;
    std::string why;
    CUresult r;
    CUdevice cu = 0;
    d_->DeviceGet(&cu, dev_);
    if (rank_ == 0) {
        int fd = -1;
        if ((r = d_->MulticastCreate(&seg->mc_handle, &mp)) != CUDA_SUCCESS) { ok = false; why = "cuMulticastCreate: " + cu_error(d_, r); }
        if (ok && (r = d_->MemExportToShareableHandle(&fd, seg->mc_handle, kFd, 0)) != CUDA_SUCCESS) { ok = false; why = "export multicast: " + cu_error(d_, r); }
        if (ok) for (int p = 1; p < n_ && ok; p++) if (!bs_->send_fd(p, fd, tag)) { ok = false; why = "send_fd: " + bs_->last_error(); }
        if (fd >= 0) ::close(fd);
    }
    // learn whether rank 0 managed before anybody blocks on a descriptor
    unsigned char root_ok = ok ? 1 : 0;
    if (!bs_->broadcast(&root_ok, 1, 0) || !root_ok) {
        bs_->discard_fds(tag);
        if (seg->mc_handle) { d_->MemRelease(seg->mc_handle); seg->mc_handle = 0; }
        if (err) *err = why.empty() ? "rank 0 could not create the multicast object" : why;
        return false;
    }
    if (rank_ != 0) {
        int fd = -1;
        if (!bs_->recv_fd(0, tag, &fd, 30000)) { ok = false; why = "recv_fd: " + bs_->last_error(); }
        else {
            r = d_->MemImportFromShareableHandle(&seg->mc_handle, (void*)(uintptr_t)fd, kFd);
            ::close(fd);
            if (r != CUDA_SUCCESS) { ok = false; why = "import multicast: " + cu_error(d_, r); }
        }
    }
    if (ok && (r = d_->MulticastAddDevice(seg->mc_handle, cu)) != CUDA_SUCCESS) { ok = false; why = "cuMulticastAddDevice: " + cu_error(d_, r); }
    // binding blocks until every device was added, so agree first
    if (!agree(ok)) { bs_->discard_fds(tag); drop_multicast(seg); if (err) *err = why.empty() ? "a peer could not join the multicast object" : why; return false; }
    if ((r = d_->MulticastBindMem(seg->mc_handle, 0, seg->handles[rank_], 0, seg->size, 0)) != CUDA_SUCCESS) { ok = false; why = "cuMulticastBindMem: " + cu_error(d_, r); }
    else seg->mc_bound = true;
    if (ok) {
        CUdeviceptr va = 0;
        CUmemAccessDesc acc;
        memset(&acc, 0, sizeof(acc));
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = dev_;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        if ((r = d_->MemAddressReserve(&va, seg->size, 2u << 20, 0, 0)) != CUDA_SUCCESS) { ok = false; why = "reserve multicast: " + cu_error(d_, r); }
        else {
            seg->mc_base = (char*)va;
            if ((r = d_->MemMap(va, seg->size, 0, seg->mc_handle, 0)) != CUDA_SUCCESS) { ok = false; why = "map multicast: " + cu_error(d_, r); }
            else if ((r = d_->MemSetAccess(va, seg->size, &acc, 1)) != CUDA_SUCCESS) { ok = false; why = "set access multicast: " + cu_error(d_, r); }
        }
    }
    if (!agree(ok)) { drop_multicast(seg); if (err) *err = why.empty() ? "a peer could not bind or map the multicast object" : why; return false; }
    return true;
}

void SymAllocator::drop_multicast(SymSegment* seg) {
    CUdevice cu = 0;
    d_->DeviceGet(&cu, dev_);
    if (seg->mc_base) {
        d_->MemUnmap((CUdeviceptr)seg->mc_base, seg->size);
        d_->MemAddressFree((CUdeviceptr)seg->mc_base, seg->size);
        seg->mc_base = nullptr;
    }
    if (seg->mc_bound) { d_->MulticastUnbind(seg->mc_handle, cu, 0, seg->size); seg->mc_bound = false; }
    if (seg->mc_handle) { d_->MemRelease(seg->mc_handle); seg->mc_handle = 0; }
}

bool SymAllocator::alloc_ipc(size_t bytes, SymSegment* seg, std::string* err) {
    const size_t size = (bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
    seg->size = size;
    seg->vmm = false;
    void* p = nullptr;
    bool ok = cudaMalloc(&p, size) == cudaSuccess;
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof(mine));
    if (ok) ok = cudaIpcGetMemHandle(&mine, p) == cudaSuccess;
    if (!ok) cudaGetLastError();
    std::vector<cudaIpcMemHandle_t> all(n_);
    if (!bs_->allgather(&mine, sizeof(mine), all.data())) ok = false;
    if (!agree(ok)) { if (p) cudaFree(p); if (err) *err = "cudaMalloc / cudaIpcGetMemHandle failed on some rank"; *seg = SymSegment(); return false; }
    seg->base[rank_] = (char*)p;
    for (int q = 0; q < n_ && ok; q++) {
        if (q == rank_) continue;
        void* m = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&m, all[q], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { ok = false; if (err) *err = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e); cudaGetLastError(); break; }
        seg->base[q] = (char*)m;
    }
    if (!agree(ok)) {
        for (int q = 0; q < n_; q++) if (q != rank_ && seg->base[q]) cudaIpcCloseMemHandle(seg->base[q]);
        cudaFree(p);
        *seg = SymSegment();
        if (err && err->empty()) *err = "a peer could not open the cudaIpc handles";
        return false;
    }
    return true;
}

void SymAllocator::free(SymSegment* seg) {
    if (!seg->size) return;
    if (seg->vmm) {
        drop_multicast(seg);
        for (int p = 0; p < n_; p++) {
            if (seg->base[p]) { d_->MemUnmap((CUdeviceptr)seg->base[p], seg->size); d_->MemAddressFree((CUdeviceptr)seg->base[p], seg->size); }
            if (seg->handles[p]) d_->MemRelease(seg->handles[p]);
        }
    } else {
        for (int q = 0; q < n_; q++) if (q != rank_ && seg->base[q]) cudaIpcCloseMemHandle(seg->base[q]);
        if (seg->base[rank_]) cudaFree(seg->base[rank_]);
    }
    *seg = SymSegment();
}

} // namespace dccl
