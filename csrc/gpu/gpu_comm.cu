/**
 * Life cycle and memory management of the device side of a communicator:
 * the symmetric pool (flags, packet region, send/recv FIFOs, two staging
 * halves), its peer and multicast mappings, the pinned status block the
 * kernels report through, symmetric user allocations and buffer registration.
 * Takes the place of the scratchpad management and NIC registration of the
 * original (reference src/core/dccl.cpp:57-237, 503-549): the pool is created
 * once per communicator, so no call allocates or registers anything.
 */
#include "gpu_impl.hpp"
#include "canary.hpp"
#include "../core/config.hpp"
#include "../core/log.hpp"
#include <cstring>

namespace dccl {

bool is_device_pointer(const void* p, int* device) {
    if (device) *device = -1;
    if (!p) return false;
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) { cudaGetLastError(); return false; }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
        if (device) *device = attr.device;
        return true;
    }
    return false;
}

int cuda_device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

GpuComm* GpuComm::create(Bootstrap* bs, int device, std::string* err) {
    if (bs->world() > kMaxPeers) { if (err) *err = "device collectives support at most 8 ranks (one NVSwitch domain)"; return nullptr; }
    GpuCommImpl* g = new GpuCommImpl(bs, device);
    if (!g->init(err)) { delete g; return nullptr; }
    return g;
}

GpuCommImpl::GpuCommImpl(Bootstrap* bs, int device) : bs_(bs), dev_(device), rank_(bs->rank()), n_(bs->world()) {
    memset(&dc_, 0, sizeof(dc_));
    for (int i = 0; i < COLL_COUNT; i++) last_[i] = ALGO_AUTO;
    for (int i = 0; i < kMaxPeers; i++) sent_chunks_[i] = recv_chunks_[i] = 0;
}

bool GpuCommImpl::init(std::string* err) {
    Config& cfg = Config::global();
    bool ok = cudaSetDevice(dev_) == cudaSuccess;
    if (!ok) { cudaGetLastError(); if (err) *err = "cudaSetDevice(" + std::to_string(dev_) + ") failed"; }
    if (ok) { int sms = 0; if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_) == cudaSuccess && sms > 0) sm_count_ = sms; }
    ctas_override_ = (int)cfg.get_int("DCCL/ctas", 0);
    p2p_ctas_ = (int)cfg.get_int("DCCL/p2p_ctas", 32);
    set_param("threads", (int)cfg.get_int("DCCL/threads", 512));
    set_param("unroll", (int)cfg.get_int("DCCL/unroll", 8));
    pipe_min_bytes_ = (size_t)cfg.get_int("DCCL/nvls_pipe_min_bytes", 16ll << 20);
    auto_min_bytes_ = (size_t)cfg.get_int("DCCL/auto_register_min_bytes", 4ll << 20);
    direct_rs_ = cfg.get_bool("DCCL/direct_reduce_scatter", true);
    direct_rs_min_bytes_ = (size_t)cfg.get_int("DCCL/direct_reduce_scatter_min_bytes", 32ll << 20);
    p2p_rdv_ = cfg.get_bool("DCCL/p2p_rendezvous", true);
    pipe_ctas_ = (int)cfg.get_int("DCCL/nvls_pipe_ctas", 112);
    pipe_nv_ctas_ = (int)cfg.get_int("DCCL/nvls_pipe_nv_ctas", 16);
    pipe_teams_ = (int)cfg.get_int("DCCL/nvls_pipe_teams", 2);
    if (pipe_teams_ < 1 || pipe_teams_ > 4) pipe_teams_ = 2;
    device_stamps_ = cfg.get_bool("DCCL/device_stamps", false);
    rooted_pipe_ = cfg.get_bool("DCCL/nvls_rooted_pipe", false);
    direct_rooted_ = cfg.get_bool("DCCL/direct_rooted", true);
    direct_rooted_ctas_ = (int)cfg.get_int("DCCL/direct_rooted_ctas", 64);
    direct_bcast_min_bytes_ = (size_t)cfg.get_int("DCCL/direct_broadcast_min_bytes", 32ll << 20);
    if (direct_rooted_ctas_ < 1 || direct_rooted_ctas_ > kMaxCtas) direct_rooted_ctas_ = 64;
    direct_bcast_ctas_ = (int)cfg.get_int("DCCL/direct_broadcast_ctas", 128);
    if (direct_bcast_ctas_ < 1 || direct_bcast_ctas_ > kMaxCtas) direct_bcast_ctas_ = 128;
    nvls_pipe_set_chunk_bytes((size_t)cfg.get_int("DCCL/nvls_pipe_chunk_bytes", 16ll << 20));
    rooted_pipe_min_bytes_ = (size_t)cfg.get_int("DCCL/nvls_rooted_pipe_min_bytes", 16ll << 20);
    if (p2p_ctas_ < 1) p2p_ctas_ = 1;
    if (p2p_ctas_ > kP2pCtas) p2p_ctas_ = kP2pCtas;
    stage_bytes_ = (size_t)cfg.get_int("DCCL/staging_bytes", 256ll << 20);
    stage_bytes_ = (stage_bytes_ + (2u << 20) - 1) / (2u << 20) * (2u << 20);

    // status block in pinned host memory: the kernels write it, the host reads it without a sync
    if (ok) {
        void* h = nullptr;
        ok = cudaHostAlloc(&h, (ST_WORDS + 8) * sizeof(uint32_t), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess;
        if (ok) {
            status_host_ = (uint32_t*)h;
            memset(status_host_, 0, (ST_WORDS + 8) * sizeof(uint32_t));
            void* d = nullptr;
            ok = cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess;
            status_dev_ = (uint32_t*)d;
        }
        if (!ok) { cudaGetLastError(); if (err) *err = "cannot allocate the pinned status block"; }
    }
    dc_.rank = rank_;
    dc_.nranks = n_;
    dc_.status = status_dev_;
    dc_.abort_word = status_dev_ + ST_WORDS;
    dc_.timeout_ns = (unsigned long long)cfg.get_int("DCCL/timeout_ms", 5000) * 1000000ull;
    dc_.stage_bytes = stage_bytes_;

    if (cfg.get_bool("DCCL/topology", true)) {
        // collective (every rank reads the same key): also a rank whose set-up failed above takes part, or its peers
        // would wait for it. The table is a report; nothing else depends on it, so a failure here is only logged.
        std::string terr;
        if (!discover_topology(&terr)) dccl_warn("topology discovery incomplete: %s", terr.c_str());
    }
    if (n_ == 1) return ok;   // a world of one needs no pool: every collective is a local copy

    // sequence counter on the device (used when DCCL/device_seq is on): {next sequence number, CTAs done}
    if (ok) {
        void* d = nullptr;
        ok = cudaMalloc(&d, 256) == cudaSuccess && cudaMemset(d, 0, 256) == cudaSuccess;
        seq_dev_ = (uint32_t*)d;
        if (!ok) { cudaGetLastError(); if (err) *err = "cannot allocate the sequence counter"; }
    }

    // every rank reports whether it got this far, so nobody blocks in the exchange below
    {
        std::vector<unsigned char> all(n_);
        unsigned char mine = ok ? 1 : 0;
        if (!bs_->allgather(&mine, 1, all.data())) { if (err) *err = "control plane failed: " + bs_->last_error(); return false; }
        for (unsigned char v : all) if (!v) { if (err && err->empty()) *err = "device setup failed on a peer"; return false; }
    }
    sym_ = new SymAllocator(bs_, dev_);
    const size_t pool_bytes = kStageOff + 2 * stage_bytes_;
    if (!sym_->alloc(pool_bytes, true, &pool_, err)) return false;
    // flags and packet tags must start from zero
    cudaError_t e = cudaMemset(pool_.base[rank_], 0, kStageOff);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    bool zero_ok = e == cudaSuccess;
    if (!zero_ok) cudaGetLastError();
    // debug aid: guard words in the unused parts of the pool, checked at finalize and by dcclDebugCheck
    guard_ = cfg.get_bool("DCCL/debug_bounds", false);
    if (guard_ && zero_ok && !canary_fill(pool_.base[rank_], canary_copy_cuda)) { zero_ok = false; cudaGetLastError(); }
    for (int p = 0; p < n_; p++) dc_.pool[p] = pool_.base[p];
    dc_.mc_pool = pool_.mc_base;
    // nobody signals into a pool that is not cleared yet
    if (!bs_->barrier()) { if (err) *err = "control plane failed: " + bs_->last_error(); return false; }
    if (!zero_ok) { if (err) *err = "clearing the pool failed"; return false; }
    if (cfg.get_bool("DCCL/device_seq", false) && !set_device_seq(true)) { if (err) *err = "cannot switch to the device-side sequence counter"; return false; }
    dccl_info("device %d: pool of %zu MB per rank (%s), multicast %s", dev_, pool_.size >> 20,
              pool_.vmm ? "cuMem" : "cudaIpc", pool_.mc_base ? "bound" : "off");
    return true;
}

GpuCommImpl::~GpuCommImpl() {
    DeviceGuard g(dev_);
    // kernels of this communicator may still be queued on user streams
    cudaDeviceSynchronize();
    cudaGetLastError();
    if (guard_) {
        char msg[160];
        if (debug_check(msg, sizeof(msg)) != ncclSuccess) dccl_error("%s", msg);
    }
    for (auto& r : regs_)
        for (int p = 0; p < n_; p++) r.peer[p] = nullptr;
    for (auto& kv : ipc_opened_) cudaIpcCloseMemHandle(kv.second);
    ipc_opened_.clear();
    if (sym_) {
        for (auto& s : user_segs_) sym_->free(&s);
        user_segs_.clear();
        sym_->free(&pool_);
        delete sym_;
        sym_ = nullptr;
    }
    if (status_host_) cudaFreeHost(status_host_);
    if (seq_dev_) cudaFree(seq_dev_);
    cudaGetLastError();
}

/* ---------------- topology ---------------- */

bool GpuCommImpl::discover_topology(std::string* err) {
    topo_ = Topology();
    topo_.nranks = n_;
    GpuInfo mine;
    const bool have = discover_gpu(dev_, &mine, err);
    if (n_ == 1) {
        topo_.gpu[0] = mine;
        topo_.access[0][0] = 2;
        topo_.atomics[0][0] = 1;
        if (have) dccl_info("topology: %s", topology_summary(topo_).c_str());
        return have;
    }
    // the control plane carries both exchanges; a rank whose discovery failed still takes part (with an empty record)
    if (!bs_->allgather(&mine, sizeof(mine), topo_.gpu)) { if (err) *err = "control plane failed: " + bs_->last_error(); return false; }
    unsigned char row[2][kMaxPeers];
    memset(row, 0, sizeof(row));
    discover_peer_row(dev_, topo_.gpu, n_, row[0], row[1]);
    unsigned char all[kMaxPeers][2][kMaxPeers];
    if (!bs_->allgather(row, sizeof(row), all)) { if (err) *err = "control plane failed: " + bs_->last_error(); return false; }
    bool blocked = false;
    for (int a = 0; a < n_; a++)
        for (int b = 0; b < n_; b++) {
            topo_.access[a][b] = all[a][0][b];
            topo_.atomics[a][b] = all[a][1][b];
            if (a != b && all[a][0][b] == 0) blocked = true;
        }
    if (rank_ == 0) dccl_info("topology: %s", topology_summary(topo_).c_str());
    if (blocked) dccl_warn("some GPU pairs report no peer access; mapping the pools will show whether they can be reached");
    for (int a = 0; a < n_; a++) if (topo_.gpu[a].device < 0) { if (err) *err = "rank " + std::to_string(a) + " could not describe its GPU"; return false; }
    return true;   // (the caller only logs a failure: the table is a report)
}

/* ---------------- where the sequence number lives ---------------- */

bool GpuCommImpl::set_device_seq(bool on) {
    if (on == device_seq_) return true;
    if (n_ == 1) { device_seq_ = on; return true; }
    if (!seq_dev_) return false;
    DeviceGuard g(dev_);
    // calls in flight still count with the old owner of the number
    if (cudaDeviceSynchronize() != cudaSuccess) { cudaGetLastError(); return false; }
    if (on) {
        const uint32_t words[2] = {next_seq(seq_), 0u};
        if (cudaMemcpy(seq_dev_, words, sizeof(words), cudaMemcpyHostToDevice) != cudaSuccess) { cudaGetLastError(); return false; }
        dc_.seq_word = seq_dev_;
        dc_.done_word = seq_dev_ + 1;
    } else {
        uint32_t next = 0;
        if (cudaMemcpy(&next, seq_dev_, sizeof(next), cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return false; }
        seq_ = next - 1u;   // next_seq(seq_) is `next` again, also across the wrap
        dc_.seq_word = nullptr;
        dc_.done_word = nullptr;
    }
    device_seq_ = on;
    return true;
}

ncclResult_t GpuCommImpl::capture_check(cudaStream_t stream, bool p2p) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) { cudaGetLastError(); return ncclSuccess; }
    if (st == cudaStreamCaptureStatusNone) return ncclSuccess;
    if (p2p) {
        dccl_error("send / recv cannot be captured into a CUDA graph: their chunk numbers are counted on the host");
        return ncclInvalidUsage;
    }
    if (!device_seq_ && n_ > 1) {
        dccl_error("a collective on a capturing stream needs the device-side sequence counter: set DCCL_DEVICE_SEQ=1 "
                   "(or the parameter device_seq) on every rank before capturing");
        return ncclInvalidUsage;
    }
    return ncclSuccess;
}

/* ---------------- stream-time stamps ---------------- */

struct StampMsg { uint64_t tag, rank, extra; };

static void CUDART_CB stamp_callback(void* p) {
    StampMsg* m = (StampMsg*)p;
    Timestamp::log(m->tag, m->rank, m->extra);
    delete m;
}

void GpuCommImpl::stamp(cudaStream_t stream, uint64_t tag, uint64_t extra) {
    if (!device_stamps_) return;
    // a host function in the stream runs when the work before it has finished: TT_DEVICE_KERNEL_BEGIN right
    // before the collective's kernel may start, TT_DEVICE_KERNEL_END right after it has completed
    StampMsg* m = new StampMsg{tag, (uint64_t)rank_, extra};
    if (cudaLaunchHostFunc(stream, stamp_callback, m) != cudaSuccess) { cudaGetLastError(); delete m; }
}

/* ---------------- errors ---------------- */

ncclResult_t GpuCommImpl::cuda_result(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return ncclSuccess;
    dccl_error("%s: %s", what, cudaGetErrorString(e));
    cudaGetLastError();
    return ncclUnhandledCudaError;
}

ncclResult_t GpuCommImpl::debug_check(char* msg, size_t len) {
    if (msg && len) msg[0] = 0;
    if (!guard_ || !pool_.base[rank_]) return ncclSuccess;
    DeviceGuard g(dev_);
    size_t bad = 0;
    const int rc = canary_check(pool_.base[rank_], canary_copy_cuda, &bad);
    if (rc == 0) return ncclSuccess;
    if (rc < 0) { cudaGetLastError(); if (msg && len) snprintf(msg, len, "the pool of rank %d could not be read", rank_); return ncclUnhandledCudaError; }
    const PoolGap* gaps = nullptr;
    pool_gaps(&gaps);
    if (msg && len)
        snprintf(msg, len, "rank %d: the pool was written outside its regions, first at offset %zu (the gap after %s, %zu..%zu)",
                 rank_, bad, gaps[rc - 1].after, gaps[rc - 1].lo, gaps[rc - 1].hi);
    return ncclInternalError;
}

ncclResult_t GpuCommImpl::async_error(char* msg, size_t len) {
    if (!status_host_) return ncclSuccess;
    volatile uint32_t* st = status_host_;
    const uint32_t code = st[ST_CODE];
    if (code == DEV_OK) return ncclSuccess;
    sticky_error_ = true;
    if (msg && len && code == DEV_BOUNDS)
        snprintf(msg, len, "a range check failed in a kernel of rank %u (site %u, value %u)", st[ST_PEER], st[ST_SITE], st[ST_SEQ]);
    else if (msg && len && code == DEV_MISMATCH)
        snprintf(msg, len, "send / recv with rank %u: the sender used %u CTAs per operation, this rank another number "
                           "(p2p_ctas, or the operations of a group, differ between the ranks)", st[ST_PEER], st[ST_SEQ]);
    else if (msg && len) {
        const char* what = code == DEV_TIMEOUT ? "timed out waiting for" : code == DEV_ABORTED ? "gave up (abort) waiting for" : "failed on";
        snprintf(msg, len, "a kernel %s rank %u (site %u, call %u)", what, st[ST_PEER], st[ST_SITE], st[ST_SEQ]);
    }
    return code == DEV_BOUNDS ? ncclInternalError : code == DEV_MISMATCH ? ncclInvalidUsage : ncclRemoteError;
}

void GpuCommImpl::abort(int failed_rank) {
    (void)failed_rank;
    if (status_host_) {
        volatile uint32_t* st = status_host_;
        st[ST_WORDS] = 1;   // the abort word the kernels poll
    }
}

ncclResult_t GpuCommImpl::precheck() {
    if (status_host_) {
        volatile uint32_t* st = status_host_;
        if (st[ST_CODE] != DEV_OK || st[ST_WORDS] != 0) {
            if (!sticky_error_) {
                char msg[160] = "aborted";
                async_error(msg, sizeof(msg));
                dccl_error("communicator is in error state: %s", msg);
                sticky_error_ = true;
            }
            return ncclRemoteError;
        }
    }
    return ncclSuccess;
}

/* ---------------- symmetric user memory ---------------- */

ncclResult_t GpuCommImpl::mem_alloc(void** ptr, size_t size) {
    DeviceGuard g(dev_);
    if (n_ == 1) return cuda_result(cudaMalloc(ptr, size), "cudaMalloc");
    SymSegment seg;
    std::string err;
    if (!sym_->alloc(size, true, &seg, &err)) { dccl_error("dcclMemAlloc(%zu): %s", size, err.c_str()); return ncclSystemError; }
    *ptr = seg.base[rank_];
    user_segs_.push_back(seg);
    return ncclSuccess;
}

ncclResult_t GpuCommImpl::mem_free(void* ptr) {
    DeviceGuard g(dev_);
    if (n_ == 1) return cuda_result(cudaFree(ptr), "cudaFree");
    for (size_t i = 0; i < user_segs_.size(); i++) {
        if (user_segs_[i].base[rank_] != (char*)ptr) continue;
        // no kernel here or on a peer may still touch the segment
        cudaDeviceSynchronize();
        if (!bs_->barrier()) dccl_warn("dcclMemFree: barrier failed (%s); freeing anyway", bs_->last_error().c_str());
        sym_->free(&user_segs_[i]);
        user_segs_.erase(user_segs_.begin() + (long)i);
        return ncclSuccess;
    }
    return ncclInvalidArgument;
}

bool GpuCommImpl::sym_view(const void* p, size_t bytes, const char** peers, const char** mc) const {
    const char* c = (const char*)p;
    for (const auto& s : user_segs_) {
        const char* b = s.base[rank_];
        if (c < b || c + bytes > b + s.size) continue;
        const size_t off = (size_t)(c - b);
        for (int q = 0; q < n_; q++) peers[q] = s.base[q] + off;
        *mc = s.mc_base ? s.mc_base + off : nullptr;
        return true;
    }
    for (const auto& r : regs_) {
        if (c < r.base || c + bytes > r.base + r.size) continue;
        const size_t off = (size_t)(c - r.base);
        for (int q = 0; q < n_; q++) peers[q] = r.peer[q] + off;
        *mc = nullptr;
        return true;
    }
    return false;
}

/* ---------------- registration of ordinary device buffers ---------------- */

struct RegMsg {
    cudaIpcMemHandle_t handle;
    unsigned long long offset;   // of the buffer inside its allocation
    unsigned long long size;
    int ok;
    int pad;
};

ncclResult_t GpuCommImpl::register_buffer(void* buf, size_t size) {
    DeviceGuard g(dev_);
    if (n_ == 1) return ncclSuccess;
    for (const auto& s : user_segs_)   // symmetric memory is mapped everywhere already
        if ((char*)buf >= s.base[rank_] && (char*)buf + size <= s.base[rank_] + s.size) return ncclSuccess;
    for (const auto& r : regs_) if (r.base == (char*)buf && r.size >= size) return ncclSuccess;
    RegMsg mine;
    memset(&mine, 0, sizeof(mine));
    mine.size = size;
    std::string err;
    const DriverApi* d = driver_api(&err);
    CUdeviceptr abase = 0;
    size_t asize = 0;
    if (d && d->MemGetAddressRange && d->MemGetAddressRange(&abase, &asize, (CUdeviceptr)buf) == CUDA_SUCCESS &&
        cudaIpcGetMemHandle(&mine.handle, (void*)abase) == cudaSuccess) {
        mine.offset = (unsigned long long)((char*)buf - (char*)abase);
        mine.ok = 1;
    } else cudaGetLastError();   // e.g. memory from a pool allocator cannot be exported: not fatal
    std::vector<RegMsg> all(n_);
    if (!bs_->allgather(&mine, sizeof(mine), all.data())) return ncclSystemError;
    bool everyone = true;
    for (auto& m : all) if (!m.ok || m.size != size) everyone = false;
    if (!everyone) {
        dccl_debug("buffer %p is not exportable on every rank; calls on it use the staged path", buf);
        return ncclSuccess;
    }
    RegisteredBuffer r;
    r.base = (char*)buf;
    r.size = size;
    bool ok = true;
    for (int q = 0; q < n_; q++) {
        if (q == rank_) { r.peer[q] = (char*)buf; continue; }
        std::string key((const char*)&all[q].handle, sizeof(cudaIpcMemHandle_t));
        key += (char)q;
        void* m = nullptr;
        auto it = ipc_opened_.find(key);
        if (it != ipc_opened_.end()) m = it->second;
        else {
            cudaError_t e = cudaIpcOpenMemHandle(&m, all[q].handle, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) { cudaGetLastError(); ok = false; m = nullptr; }
            else ipc_opened_[key] = m;
        }
        r.peer[q] = m ? (char*)m + all[q].offset : nullptr;
    }
    std::vector<unsigned char> oks(n_);
    unsigned char mo = ok ? 1 : 0;
    if (!bs_->allgather(&mo, 1, oks.data())) return ncclSystemError;
    for (unsigned char v : oks) if (!v) ok = false;
    if (ok) regs_.push_back(r);
    else dccl_debug("buffer %p could not be opened on every rank; calls on it use the staged path", buf);
    return ncclSuccess;
}

ncclResult_t GpuCommImpl::deregister_buffer(void* buf) {
    for (size_t i = 0; i < regs_.size(); i++)
        if (regs_[i].base == (char*)buf) { regs_.erase(regs_.begin() + (long)i); break; }   // mappings stay cached until finalize
    return ncclSuccess;
}

} // namespace dccl
