/**
 * Lazy registration of ordinary device buffers.
 *
 * The original asks the application to register every buffer before use
 * (reference src/core/dccl.cpp:503-542, src/application/cli.cpp:455-466) and
 * then moves data zero-copy between the registered regions. Here a large call
 * on buffers that were never registered does it by itself: inside the call the
 * ranks tell each other, over the shared-memory exchange board of the bootstrap
 * (a few microseconds, no system call), which allocation each buffer lies in;
 * an allocation the peers have not seen yet is exported with cudaIpc and opened
 * by every peer once, and from then on the zero-copy peer kernels (direct.cu)
 * read and write the user's memory directly.
 *
 * Every rank takes part in every exchange, in the order of the calls, so all
 * ranks see the same messages and come to the same answer. An allocation is
 * known by its driver buffer id, which changes when memory is freed and
 * allocated again at the same address: the stale mapping is then closed and the
 * new one opened. What cannot be exported (memory of a stream-ordered pool or of
 * the virtual-memory API, or more allocations than the table holds) is reported
 * as such and the call takes the staged path, on every rank alike.
 *
 * Only peer loads and stores ever touch these mappings: they are never handed to
 * a library kernel and never read with a multicast load.
 */
#include "gpu_impl.hpp"
#include "driver_api.hpp"
#include "../core/log.hpp"
#include <cstring>

namespace dccl {

namespace {
struct AutoBuf {                  // what a rank tells the others about one of its buffers
    unsigned long long id;        // driver buffer id of the allocation; 0: cannot be exported
    unsigned long long base;      // of the allocation, in the owner's address space
    unsigned long long offset;    // of the buffer inside the allocation
    unsigned long long size;      // of the allocation
    unsigned int fresh;           // the peers have not opened this allocation yet
    unsigned int symmetric;       // 1: symmetric memory, mapped everywhere already; `base` is the number of the segment
    cudaIpcMemHandle_t handle;
};
struct AutoMsg { AutoBuf b[2]; };
static_assert(sizeof(AutoMsg) <= kBoardBytes, "the exchange board is too small for two buffer descriptions");
constexpr size_t kAutoMaxExports = 64;   // allocations of one rank that its peers keep open
}

/** Describe `buf` for the peers: find its allocation, export it if it is new. */
static void describe(const DriverApi* d, const void* buf, std::map<unsigned long long, AutoExport>& mine, AutoBuf* out) {
    memset(out, 0, sizeof(*out));
    if (!d || !d->PointerGetAttribute || !d->MemGetAddressRange) return;
    unsigned long long id = 0;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (d->PointerGetAttribute(&id, CU_POINTER_ATTRIBUTE_BUFFER_ID, (CUdeviceptr)buf) != CUDA_SUCCESS || id == 0) return;
    if (d->MemGetAddressRange(&base, &size, (CUdeviceptr)buf) != CUDA_SUCCESS) return;
    auto it = mine.find((unsigned long long)base);
    if (it != mine.end() && it->second.id == id) {
        if (it->second.refused) return;
        out->fresh = it->second.announced ? 0u : 1u;
    } else {
        AutoExport e;
        e.id = id;
        e.size = size;
        // a new allocation (perhaps at an address seen before: the old one is gone, the peers drop it when they see the new id)
        const bool room = it != mine.end() || mine.size() < kAutoMaxExports;
        if (!room || cudaIpcGetMemHandle(&e.handle, (void*)base) != cudaSuccess) {
            cudaGetLastError();
            e.refused = true;
        }
        if (it != mine.end()) it->second = e;
        else if (room) it = mine.emplace((unsigned long long)base, e).first;
        if (e.refused) return;
        out->fresh = 1u;
    }
    out->id = id;
    out->base = (unsigned long long)base;
    out->offset = (unsigned long long)((const char*)buf - (const char*)base);
    out->size = (unsigned long long)it->second.size;
    out->handle = it->second.handle;
}

bool GpuCommImpl::auto_view(const void* send, const void* recv, const char** send_peers, const char** recv_peers) {
    std::string err;
    const DriverApi* d = driver_api(&err);
    AutoMsg mine;
    auto describe_any = [&](const void* buf, AutoBuf* out) {
        // symmetric memory was allocated collectively: segment i is segment i on every rank, and every rank maps all of it
        const char* c = (const char*)buf;
        for (size_t i = 0; i < user_segs_.size(); i++) {
            const SymSegment& s = user_segs_[i];
            if (c < s.base[rank_] || c >= s.base[rank_] + s.size) continue;
            memset(out, 0, sizeof(*out));
            out->id = ~0ull; out->base = i; out->offset = (unsigned long long)(c - s.base[rank_]); out->size = s.size; out->symmetric = 1;
            return;
        }
        describe(d, buf, auto_exports_, out);
    };
    describe_any(send, &mine.b[0]);
    if (recv == send) mine.b[1] = mine.b[0];
    else describe_any(recv, &mine.b[1]);
    std::vector<AutoMsg> all((size_t)n_);
    if (!bs_->fast_allgather(&mine, sizeof(mine), all.data())) { dccl_warn("lazy registration: %s", bs_->last_error().c_str()); return false; }
    for (int k = 0; k < 2; k++)
        if (mine.b[k].id && !mine.b[k].symmetric) auto_exports_[mine.b[k].base].announced = true;

    bool usable = true, any_fresh = false;
    unsigned char failed[2] = {0, 0};     // bit q: this rank could not open rank q's send / receive allocation
    for (int q = 0; q < n_; q++) {
        for (int k = 0; k < 2; k++) {
            const AutoBuf& b = all[q].b[k];
            if (!b.id) { usable = false; continue; }
            if (b.symmetric) { if (b.base >= user_segs_.size()) usable = false; continue; }
            if (b.fresh) any_fresh = true;
            if (q == rank_) continue;
            if (!import_allocation(q, b.base, b.id, (size_t)b.size, b.handle)) failed[k] |= (unsigned char)(1u << q);
        }
    }
    if (any_fresh) {
        // something was opened in this call: learn whether every rank managed (all ranks see the flag, all take this branch)
        std::vector<unsigned char> oks((size_t)n_ * 2);
        if (!bs_->fast_allgather(failed, 2, oks.data())) { dccl_warn("lazy registration: %s", bs_->last_error().c_str()); return false; }
        for (int k = 0; k < 2; k++) {
            unsigned char bad = 0;
            for (int p = 0; p < n_; p++) bad |= oks[(size_t)p * 2 + k];
            for (int q = 0; q < n_ && bad; q++) {
                if (!(bad >> q & 1)) continue;
                usable = false;
                const AutoBuf& b = all[q].b[k];
                if (q == rank_) {
                    auto it = auto_exports_.find(b.base);
                    if (it != auto_exports_.end()) it->second.refused = true;     // not offered again
                    dccl_debug("lazy registration: a peer cannot open the allocation at %#llx; calls on it use the staged path", b.base);
                } else {
                    auto it = auto_imports_.find(std::make_pair(q, b.base));
                    if (it != auto_imports_.end()) { close_import(it->second); auto_imports_.erase(it); }
                }
            }
        }
    }
    if (!usable) return false;
    for (int q = 0; q < n_; q++) {
        if (q == rank_) { send_peers[q] = (const char*)send; recv_peers[q] = (const char*)recv; continue; }
        const char** out[2] = {&send_peers[q], &recv_peers[q]};
        for (int k = 0; k < 2; k++) {
            const AutoBuf& b = all[q].b[k];
            *out[k] = b.symmetric ? user_segs_[(size_t)b.base].base[q] + b.offset
                                  : (const char*)auto_imports_[std::make_pair(q, b.base)].mapped + b.offset;
        }
    }
    return true;
}

AutoImport* GpuCommImpl::import_allocation(int owner, unsigned long long base, unsigned long long id, size_t size, const cudaIpcMemHandle_t& handle) {
    const std::pair<int, unsigned long long> key(owner, base);
    auto it = auto_imports_.find(key);
    if (it != auto_imports_.end() && it->second.id != id) {
        // the owner freed that allocation and got the address again: drop the stale mapping
        close_import(it->second);
        auto_imports_.erase(it);
        it = auto_imports_.end();
    }
    if (it != auto_imports_.end()) return &it->second;
    AutoImport im;
    im.id = id;
    im.size = size;
    im.stamp = ++import_stamp_;
    im.hkey.assign((const char*)&handle, sizeof(cudaIpcMemHandle_t));
    im.hkey += (char)owner;
    auto op = ipc_opened_.find(im.hkey);      // one open per allocation and process, shared with explicit registration
    if (op != ipc_opened_.end()) im.mapped = op->second;
    else if (cudaIpcOpenMemHandle(&im.mapped, handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess) ipc_opened_[im.hkey] = im.mapped;
    else { cudaGetLastError(); return nullptr; }
    return &(auto_imports_[key] = im);
}

/* ---- send / recv: the receiver's exports reach the sender through the bulletin, nobody waits ---- */

namespace {
struct ExportNote {               // one exported allocation, as posted on the owner's bulletin
    unsigned long long id, base, size;
    cudaIpcMemHandle_t handle;
};
static_assert(sizeof(ExportNote) <= kBulletinBytes, "an export note must fit a bulletin entry");
}

void GpuCommImpl::describe_receive_buffer(const void* buf, size_t bytes, P2pOp* op) {
    op->dst_kind = P2P_DST_NONE;
    const char* c = (const char*)buf;
    for (size_t i = 0; i < user_segs_.size(); i++) {      // symmetric memory: allocated collectively, so segment i is segment i everywhere
        const SymSegment& s = user_segs_[i];
        if (c < s.base[rank_] || c + bytes > s.base[rank_] + s.size) continue;
        op->dst_kind = P2P_DST_SYM; op->dst_a = i; op->dst_id = 0; op->dst_off = (unsigned long long)(c - s.base[rank_]);
        return;
    }
    std::string err;
    AutoBuf d;
    describe(driver_api(&err), buf, auto_exports_, &d);
    if (!d.id) return;
    AutoExport& e = auto_exports_[d.base];
    if (!e.posted) {
        ExportNote note;
        memset(&note, 0, sizeof(note));
        note.id = d.id; note.base = d.base; note.size = d.size; note.handle = d.handle;
        if (!bs_->bulletin_post(&note, sizeof(note))) return;
        e.posted = true;
    }
    op->dst_kind = P2P_DST_IPC; op->dst_a = d.base; op->dst_id = d.id; op->dst_off = d.offset;
}

void GpuCommImpl::poll_exports(int peer) {
    ExportNote note;
    for (;;) {
        const int got = bs_->bulletin_read(peer, bulletin_seen_[peer], &note, sizeof(note));
        if (got == 0) return;
        bulletin_seen_[peer]++;
        if (got < 0) continue;                      // overwritten before this rank looked: that buffer keeps using the FIFO
        import_allocation(peer, note.base, note.id, (size_t)note.size, note.handle);
    }
}

void GpuCommImpl::close_import(const AutoImport& im) {
    auto op = ipc_opened_.find(im.hkey);
    if (op == ipc_opened_.end()) return;
    cudaIpcCloseMemHandle(op->second);
    ipc_opened_.erase(op);
}

} // namespace dccl
