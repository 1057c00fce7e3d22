/**
 * Symmetric device memory: every rank allocates a segment of the same size and
 * maps every peer's segment into its own address space, so a kernel can load
 * from and store to any rank's copy; where the NVSwitch supports it the
 * segments are also bound to one multicast object whose mapping gives
 * multimem.ld_reduce / multimem.st access to all copies at once.
 *
 * This is what memory registration with the NIC is in the original
 * (register_oob_memory_ex, reference src/core/dccl.cpp:516-540). Two
 * mechanisms: CUDA virtual memory management with POSIX file-descriptor
 * handles passed over a unix socket (needed for multicast), or, where that is
 * not available, cudaMalloc + cudaIpc handles exchanged over the control plane.
 */
#pragma once
#include "driver_api.hpp"
#include "../bootstrap/bootstrap.hpp"
#include "../device/prims.cuh"

namespace dccl {

struct SymSegment {
    size_t size = 0;                    // bytes mapped on every rank
    size_t requested = 0;
    bool vmm = false;
    char* base[kMaxPeers] = {nullptr};  // base[my rank] is the local mapping
    char* mc_base = nullptr;            // multicast mapping, or nullptr
    CUmemGenericAllocationHandle handles[kMaxPeers] = {0};
    CUmemGenericAllocationHandle mc_handle = 0;
    bool mc_bound = false;
};

class SymAllocator {
public:
    /** Collective: ranks agree on the mechanism every later allocation uses. */
    SymAllocator(Bootstrap* bs, int device);
    /** Collective. want_mc asks for a multicast binding; absence of one is not an error. */
    bool alloc(size_t bytes, bool want_mc, SymSegment* seg, std::string* err);
    /** Collective. The caller makes sure no kernel still uses the segment. */
    void free(SymSegment* seg);
    bool uses_vmm() const { return vmm_; }
    bool multicast_usable() const { return mc_; }

private:
    bool alloc_vmm(size_t bytes, bool want_mc, SymSegment* seg, std::string* err);
    bool alloc_ipc(size_t bytes, SymSegment* seg, std::string* err);
    bool bind_multicast(SymSegment* seg, std::string* err);
    void drop_multicast(SymSegment* seg);
    bool agree(bool ok);   // logical AND over all ranks
    Bootstrap* bs_;
    const DriverApi* d_;
    int dev_, rank_, n_;
    bool vmm_ = false, mc_ = false;
    uint32_t next_tag_ = 1;
};

} // namespace dccl
