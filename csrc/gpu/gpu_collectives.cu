/**
 * Device collectives: choose the variant for a call, cut messages larger than
 * the staging capacity into several launches, fill the kernel arguments and
 * launch on the caller's stream. Counterpart of the algorithm switch in the
 * original (reference src/core/dccl.cpp:412-496), with the choice coming from
 * the tuner table unless the caller forces a variant.
 *
 * Every launch takes the next sequence number; its parity selects the staging
 * half and the packet generation. All ranks issue the same calls in the same
 * order, so they agree on sequence numbers without talking to each other.
 */
#include "gpu_impl.hpp"
#include "../core/config.hpp"
#include "../core/log.hpp"
#include "../core/types.hpp"
#include <nvtx3/nvToolsExt.h>
#include <algorithm>

namespace dccl {

int GpuCommImpl::ctas_for(int tuned) const {
    int c = ctas_override_ > 0 ? ctas_override_ : tuned;
    if (c < 1) c = 1;
    if (c > kMaxCtas) c = kMaxCtas;
    if (c > sm_count_) c = sm_count_;   // CTAs of one call wait on each other's peers: keep them all resident
    return c;
}

bool GpuCommImpl::set_param(const char* name, int value) {
    const std::string k(name ? name : "");
    if (k == "ctas" && value >= 0 && value <= kMaxCtas) { ctas_override_ = value; return true; }
    if (k == "threads" && value >= 64 && value <= 512 && value % 32 == 0) { threads_ = value; return true; }
    if (k == "unroll" && (value == 2 || value == 4 || value == 8)) { unroll_ = value; return true; }
    if (k == "p2p_ctas" && value >= 1 && value <= kP2pCtas) { p2p_ctas_ = value; return true; }
    if (k == "pipe_min_mb" && value >= 0) { pipe_min_bytes_ = (size_t)value << 20; return true; }
    if (k == "pipe_ctas" && value >= 3 && value <= kMaxCtas) { pipe_ctas_ = value; return true; }
    if (k == "pipe_nv_ctas" && value >= 1 && value <= kMaxCtas / 2) { pipe_nv_ctas_ = value; return true; }
    if (k == "pipe_teams" && value >= 1 && value <= 4) { pipe_teams_ = value; return true; }
    if (k == "pipe_unroll" && (value == 2 || value == 4 || value == 8)) { pipe_unroll_ = value; return true; }
    if (k == "auto_register_min_kb" && value >= 0) { auto_min_bytes_ = (size_t)value << 10; return true; }
    if (k == "direct_rs" && (value == 0 || value == 1)) { direct_rs_ = value == 1; return true; }
    if (k == "direct_rs_min_mb" && value >= 0) { direct_rs_min_bytes_ = (size_t)value << 20; return true; }
    if (k == "p2p_rendezvous" && (value == 0 || value == 1)) { p2p_rdv_ = value == 1; return true; }
    if (k == "device_seq" && (value == 0 || value == 1)) return set_device_seq(value == 1);
    if (k == "rooted_pipe" && (value == 0 || value == 1)) { rooted_pipe_ = value == 1; return true; }
    if (k == "direct_rooted" && (value == 0 || value == 1)) { direct_rooted_ = value == 1; return true; }
    if (k == "direct_rooted_ctas" && value >= 1 && value <= kMaxCtas) { direct_rooted_ctas_ = value; return true; }
    if (k == "direct_bcast_min_kb" && value >= 0) { direct_bcast_min_bytes_ = (size_t)value << 10; return true; }
    if (k == "direct_bcast_ctas" && value >= 1 && value <= kMaxCtas) { direct_bcast_ctas_ = value; return true; }
    if (k == "direct_reduce_small_worlds" && (value == 0 || value == 1)) { direct_reduce_small_ = value == 1; return true; }
    if (k == "pipe_chunk_kb" && value >= 256) { nvls_pipe_set_chunk_bytes((size_t)value << 10); return true; }
    return false;
}

uint64_t GpuCommImpl::stat(const char* name) const {
    const std::string k(name ? name : "");
    if (k == "launches") return launches_;
    if (k == "zero_copy_calls") return zero_copy_calls_;
    if (k == "symmetric_calls") return symmetric_calls_;
    return 0;
}

CollArgs GpuCommImpl::base_args(const void* send, void* recv, ncclRedOp_t op, int root) {
    CollArgs a;
    memset(&a, 0, sizeof(a));
    a.comm = dc_;
    a.io.send = send;
    a.io.recv = recv;
    a.op = (int)op;
    a.root = root;
    a.unroll = unroll_;
    return a;
}

/** Stamps the device time line around one API call when DCCL/device_stamps is on, and opens an NVTX range. */
struct CallScope {
    GpuCommImpl* g; cudaStream_t s; uint64_t coll;
    CallScope(GpuCommImpl* g_, cudaStream_t s_, uint64_t coll_, const char* name) : g(g_), s(s_), coll(coll_) { nvtxRangePushA(name); g->stamp_begin(s, coll); }
    ~CallScope() { g->stamp_end(s, coll); nvtxRangePop(); }
};

#define NEXT_SEQ(a)                                   \
    do {                                              \
        seq_ = next_seq(seq_);                        \
        (a).seq = seq_;                               \
        (a).parity = (int)(seq_ & 1u);                \
    } while (0)

ncclResult_t GpuCommImpl::all_reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op,
                                     GpuAlgo algo, cudaStream_t stream) {
    DeviceGuard g(dev_);
    const size_t es = size_of_type(dt), bytes = count * es;
    if (n_ == 1) {
        last_[COLL_ALLREDUCE] = ALGO_LOCAL;
        if (send != recv && bytes) { launches_++; return cuda_result(launch_local_copy(recv, send, bytes, stream), "local copy"); }
        return ncclSuccess;
    }
    ncclResult_t pre = precheck();
    if (pre == ncclSuccess) pre = capture_check(stream, false);
    if (pre != ncclSuccess) return pre;
    if (!count) return ncclSuccess;
    CallScope scope(this, stream, COLL_ALLREDUCE, "dccl:allreduce");

    const bool nvls_ok = pool_.mc_base != nullptr && nvls_supports(dt, op);
    // both buffers in multicast-bound symmetric memory: the switch variant can run without copies
    const char* sp[kMaxPeers];
    const char* rp[kMaxPeers];
    const char *smc = nullptr, *rmc = nullptr;
    // every rank can address both buffers of every rank (symmetric memory, or registered buffers)
    bool peer_addr = sym_view(send, bytes, sp, &smc) && sym_view(recv, bytes, rp, &rmc);
    // all ranks must come to the same answer: look at every rank's alignment, not only the local one
    for (int p = 0; peer_addr && p < n_; p++) peer_addr = (uintptr_t)sp[p] % 16 == 0 && (uintptr_t)rp[p] % 16 == 0;
    const bool sym = peer_addr && nvls_ok && bytes % 16 == 0 && smc && rmc && ((uintptr_t)smc % 16 == 0) && ((uintptr_t)rmc % 16 == 0);
    TuneChoice ch = tuner_.choose(sym ? TUNE_ALLREDUCE_SYM : COLL_ALLREDUCE, n_, bytes, nvls_ok, (int)es);
    if (algo != ALGO_AUTO) ch.algo = algo;
    // a forced variant that cannot serve this call falls back to the closest one that can
    if (ch.algo == ALGO_NVLS && !nvls_ok) ch.algo = ALGO_TWOSHOT;
    if (ch.algo == ALGO_ONESHOT && bytes > oneshot_ll_capacity_bytes()) ch.algo = ALGO_TWOSHOT;
    if (ch.algo == ALGO_TWOSHOT_LL && bytes > ll_twoshot_capacity_bytes(n_)) ch.algo = ALGO_TWOSHOT;
    if (ch.algo == ALGO_LOCAL || ch.algo == ALGO_AUTO) ch.algo = ALGO_TWOSHOT;
    last_[COLL_ALLREDUCE] = ch.algo;

    LaunchCfg cfg;
    cfg.ctas = ctas_for(ch.ctas);
    cfg.stream = stream;
    cfg.threads = threads_;
    CollArgs a = base_args(send, recv, op, 0);

    if (ch.algo == ALGO_ONESHOT) {
        a.count = count;
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_oneshot_ll(a, dt, cfg), "one-shot all-reduce");
    }

    if (ch.algo == ALGO_TWOSHOT_LL) {
        a.mode = LL2_ALLREDUCE;
        a.count = count;
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_ll_twoshot(a, dt, cfg), "two-shot packet all-reduce");
    }

    // ordinary buffers that were never registered: the ranks exchange where they lie and map what is new (collective;
    // entered on facts every rank shares), after which the call runs zero-copy like one on registered buffers
    if (ch.algo == ALGO_TWOSHOT && !peer_addr && auto_min_bytes_ > 0 && bytes >= auto_min_bytes_ && auto_view(send, recv, sp, rp)) {
        peer_addr = true;
        for (int p = 0; peer_addr && p < n_; p++) peer_addr = (uintptr_t)sp[p] % 16 == 0 && (uintptr_t)rp[p] % 16 == 0;
    }
    // The table asked for the peer form because zero-copy beats the switch at this world size, but these buffers cannot
    // be mapped (pool or virtual-memory allocations): large messages then do better through the switch's pipeline than
    // through peer staging. (The answer of the exchange is the same on every rank.)
    if (ch.algo == ALGO_TWOSHOT && !peer_addr && algo == ALGO_AUTO && n_ > 2 && nvls_ok && pipe_min_bytes_ > 0 && bytes >= pipe_min_bytes_) {
        ch.algo = ALGO_NVLS;
        last_[COLL_ALLREDUCE] = ch.algo;
    }
    // two-shot on buffers the peers can address: fold straight out of / into the user buffers, no staging
    if (ch.algo == ALGO_TWOSHOT && peer_addr) {
        zero_copy_calls_++;
        a.symmetric = 1;
        for (int p = 0; p < n_; p++) { a.io.send_peer[p] = sp[p]; a.io.recv_peer[p] = (char*)rp[p]; }
        a.mode = DIRECT_ALLREDUCE;
        a.count = count;
        if (ch.ctas < 64 && ctas_override_ == 0) cfg.ctas = ctas_for(64);   // a row meant for the switch variant
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_direct(a, dt, cfg), "zero-copy two-shot all-reduce");
    }

    if (ch.algo == ALGO_NVLS && sym) {
        a.symmetric = 1;
        a.io.send_mc = smc;
        a.io.recv_mc = (char*)rmc;
        a.mode = NV_ALLREDUCE;
        a.count = count;
        NEXT_SEQ(a);
        launches_++;
        symmetric_calls_++;
        return cuda_result(launch_nvls(a, dt, cfg), "nvls all-reduce (symmetric)");
    }

    // large ordinary buffers through the switch: copy-in, switch pass and copy-out overlap chunk by chunk
    const bool pipe = ch.algo == ALGO_NVLS && pipe_min_bytes_ > 0 && bytes >= pipe_min_bytes_;
    if (pipe) cfg.ctas = pipe_ctas_ < sm_count_ ? pipe_ctas_ : sm_count_;
    size_t cap;
    switch (ch.algo) {
    case ALGO_NVLS: cap = !pipe ? nvls_capacity(NV_ALLREDUCE, n_, es, stage_bytes_) : device_seq_ ? nvls_pipe_capacity(es, stage_bytes_, n_, false) : count; break;
    case ALGO_RING: cap = ring_capacity(RING_ALLREDUCE, n_, es, stage_bytes_); break;
    case ALGO_RABENSEIFNER: cap = hd_capacity(n_, es, stage_bytes_); break;
    default: cap = twoshot_capacity(TS_ALLREDUCE, n_, es, stage_bytes_); break;
    }
    for (size_t off = 0; off < count; off += cap) {
        const size_t c = count - off < cap ? count - off : cap;
        a.io.send = (const char*)send + off * es;
        a.io.recv = (char*)recv + off * es;
        a.count = c;
        NEXT_SEQ(a);
        cudaError_t e;
        switch (ch.algo) {
        case ALGO_NVLS:
            if (pipe) {
                a.unroll = pipe_unroll_;
                e = launch_nvls_pipe(a, dt, cfg, false, stage_bytes_, pipe_nv_ctas_, pipe_teams_, device_seq_);
                // chunk numbers beyond one call's flag values live in the following call numbers of the same parity
                for (int k = nvls_pipe_extra_seqs(c, es, stage_bytes_, n_, false, device_seq_); k > 0; k--) seq_ = next_seq(seq_);
            }
            else { a.mode = NV_ALLREDUCE; e = launch_nvls(a, dt, cfg); }
            break;
        case ALGO_RING: a.mode = RING_ALLREDUCE; e = launch_ring(a, dt, cfg); break;
        case ALGO_RABENSEIFNER: e = launch_hd(a, dt, cfg); break;
        default: a.mode = TS_ALLREDUCE; e = launch_twoshot(a, dt, cfg); break;
        }
        launches_++;
        if (e != cudaSuccess) return cuda_result(e, "all-reduce launch");
    }
    return ncclSuccess;
}

ncclResult_t GpuCommImpl::reduce_scatter(const void* send, void* recv, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op,
                                         GpuAlgo algo, cudaStream_t stream) {
    DeviceGuard g(dev_);
    const size_t es = size_of_type(dt);
    if (n_ == 1) {
        last_[COLL_REDUCESCATTER] = ALGO_LOCAL;
        if (send != recv && recvcount) { launches_++; return cuda_result(launch_local_copy(recv, send, recvcount * es, stream), "local copy"); }
        return ncclSuccess;
    }
    ncclResult_t pre = precheck();
    if (pre == ncclSuccess) pre = capture_check(stream, false);
    if (pre != ncclSuccess) return pre;
    if (!recvcount) return ncclSuccess;
    CallScope scope(this, stream, COLL_REDUCESCATTER, "dccl:reducescatter");
    const size_t bytes = recvcount * es * (size_t)n_;
    const bool nvls_ok = pool_.mc_base != nullptr && nvls_supports(dt, op);
    // a send buffer in multicast-bound symmetric memory can be reduced by the switch where it lies
    const char* sym_peers[kMaxPeers];
    const char* sym_mc = nullptr;
    const bool sym = nvls_ok && (recvcount * es) % 16 == 0 && sym_view(send, bytes, sym_peers, &sym_mc) && sym_mc && (uintptr_t)sym_mc % 16 == 0;
    TuneChoice ch = tuner_.choose(sym ? TUNE_REDUCESCATTER_SYM : COLL_REDUCESCATTER, n_, bytes, nvls_ok, (int)es);
    if (algo != ALGO_AUTO) ch.algo = algo;
    if (ch.algo == ALGO_NVLS && !nvls_ok) ch.algo = ALGO_TWOSHOT;
    if (ch.algo == ALGO_ONESHOT && recvcount * es > oneshot_ll_capacity_bytes()) ch.algo = ALGO_TWOSHOT;
    if (ch.algo != ALGO_NVLS && ch.algo != ALGO_RING && ch.algo != ALGO_ONESHOT) ch.algo = ALGO_TWOSHOT;
    last_[COLL_REDUCESCATTER] = ch.algo;

    LaunchCfg cfg;
    cfg.ctas = ctas_for(ch.ctas);
    cfg.stream = stream;
    cfg.threads = threads_;
    CollArgs a = base_args(send, recv, op, 0);
    a.stride = recvcount;

    if (ch.algo == ALGO_ONESHOT) {
        a.mode = LL_REDUCESCATTER;
        a.count = recvcount;
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_ll_collective(a, dt, cfg), "packet reduce-scatter");
    }
    // two-shot on buffers the peers can address: every rank folds its slot straight out of the peers' send buffers.
    // Chosen by itself only at world size 2, where this form is measured (all-reduce: 1.5 x the staged form);
    // elsewhere the caller asks for it with dcclSetAlgorithm(twoshot).
    if (ch.algo == ALGO_TWOSHOT && (n_ == 2 || (direct_rs_ && bytes >= direct_rs_min_bytes_) || algo == ALGO_TWOSHOT) && (recvcount * es) % 16 == 0) {
        // the kernel moves whole 16-byte vectors, so every rank's send and receive pointer must be aligned; the ranks
        // know each other's through the symmetric layout or through the exchange
        const char* rp[kMaxPeers];
        const char* rmc = nullptr;
        bool peer_addr = sym_view(send, bytes, sym_peers, &sym_mc) && sym_view(recv, recvcount * es, rp, &rmc);
        if (!peer_addr && auto_min_bytes_ > 0 && bytes >= auto_min_bytes_) peer_addr = auto_view(send, recv, sym_peers, rp);
        // every rank must come to the same answer, so every rank's alignment counts
        for (int p = 0; peer_addr && p < n_; p++) peer_addr = (uintptr_t)sym_peers[p] % 16 == 0 && (uintptr_t)rp[p] % 16 == 0;
        if (peer_addr) {
            zero_copy_calls_++;
            a.symmetric = 1;
            for (int p = 0; p < n_; p++) a.io.send_peer[p] = sym_peers[p];
            a.mode = DIRECT_REDUCESCATTER;
            a.count = recvcount;
            NEXT_SEQ(a);
            launches_++;
            return cuda_result(launch_direct(a, dt, cfg), "zero-copy two-shot reduce-scatter");
        }
    }
    if (ch.algo == ALGO_NVLS) {
        if (sym) {
            a.symmetric = 1;
            a.io.send_mc = sym_mc;
            a.mode = NV_REDUCESCATTER;
            a.count = recvcount;
            NEXT_SEQ(a);
            launches_++;
        symmetric_calls_++;
            return cuda_result(launch_nvls(a, dt, cfg), "nvls reduce-scatter (symmetric)");
        }
    }
    // large ordinary buffers through the switch: copy-in and switch pass overlap chunk by chunk
    // (only facts that are the same on every rank may pick the kernel; an unaligned receive buffer is handled inside it)
    const bool pipe = ch.algo == ALGO_NVLS && pipe_min_bytes_ > 0 && bytes >= pipe_min_bytes_;
    if (pipe) {
        // the switch group as in the all-reduce, one copy group instead of two
        const int total = pipe_ctas_ < sm_count_ ? pipe_ctas_ : sm_count_;
        const int nv = pipe_nv_ctas_ < total ? pipe_nv_ctas_ : total / 3;
        cfg.ctas = nv + (total - nv) / 2;
    }
    size_t cap = pipe ? (device_seq_ ? nvls_pipe_capacity(es, stage_bytes_, n_, true) : recvcount)
                 : ch.algo == ALGO_NVLS ? nvls_capacity(NV_REDUCESCATTER, n_, es, stage_bytes_)
                 : ch.algo == ALGO_RING ? ring_capacity(RING_REDUCESCATTER, n_, es, stage_bytes_)
                                        : twoshot_capacity(TS_REDUCESCATTER, n_, es, stage_bytes_);
    for (size_t off = 0; off < recvcount; off += cap) {
        const size_t c = recvcount - off < cap ? recvcount - off : cap;
        a.io.send = (const char*)send + off * es;   // slot j of this piece starts at send + j*stride + off
        a.io.recv = (char*)recv + off * es;
        a.count = c;
        NEXT_SEQ(a);
        cudaError_t e;
        if (pipe) {
            a.unroll = pipe_unroll_;
            e = launch_nvls_pipe(a, dt, cfg, true, stage_bytes_, pipe_nv_ctas_, pipe_teams_, device_seq_);
            for (int k = nvls_pipe_extra_seqs(c, es, stage_bytes_, n_, true, device_seq_); k > 0; k--) seq_ = next_seq(seq_);
        }
        else if (ch.algo == ALGO_NVLS) { a.mode = NV_REDUCESCATTER; e = launch_nvls(a, dt, cfg); }
        else if (ch.algo == ALGO_RING) { a.mode = RING_REDUCESCATTER; e = launch_ring(a, dt, cfg); }
        else { a.mode = TS_REDUCESCATTER; e = launch_twoshot(a, dt, cfg); }
        launches_++;
        if (e != cudaSuccess) return cuda_result(e, "reduce-scatter launch");
    }
    return ncclSuccess;
}

ncclResult_t GpuCommImpl::all_gather(const void* send, void* recv, size_t sendcount, ncclDataType_t dt,
                                     GpuAlgo algo, cudaStream_t stream) {
    DeviceGuard g(dev_);
    const size_t es = size_of_type(dt);
    if (n_ == 1) {
        last_[COLL_ALLGATHER] = ALGO_LOCAL;
        if (send != recv && sendcount) { launches_++; return cuda_result(launch_local_copy(recv, send, sendcount * es, stream), "local copy"); }
        return ncclSuccess;
    }
    ncclResult_t pre = precheck();
    if (pre == ncclSuccess) pre = capture_check(stream, false);
    if (pre != ncclSuccess) return pre;
    if (!sendcount) return ncclSuccess;
    CallScope scope(this, stream, COLL_ALLGATHER, "dccl:allgather");
    const size_t bytes = sendcount * es * (size_t)n_;
    const bool nvls_ok = pool_.mc_base != nullptr;
    TuneChoice ch = tuner_.choose(COLL_ALLGATHER, n_, bytes, nvls_ok, (int)es);
    if (algo != ALGO_AUTO) ch.algo = algo;
    if (ch.algo == ALGO_NVLS && !nvls_ok) ch.algo = ALGO_TWOSHOT;
    if (ch.algo == ALGO_ONESHOT && sendcount * es > oneshot_ll_capacity_bytes()) ch.algo = ALGO_TWOSHOT;
    if (ch.algo != ALGO_NVLS && ch.algo != ALGO_RING && ch.algo != ALGO_ONESHOT) ch.algo = ALGO_TWOSHOT;
    last_[COLL_ALLGATHER] = ch.algo;

    LaunchCfg cfg;
    cfg.ctas = ctas_for(ch.ctas);
    cfg.stream = stream;
    cfg.threads = threads_;
    CollArgs a = base_args(send, recv, ncclSum, 0);
    a.stride = sendcount;

    if (ch.algo == ALGO_ONESHOT) {
        a.mode = LL_ALLGATHER;
        a.count = sendcount;
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_ll_collective(a, dt, cfg), "packet all-gather");
    }
    if (ch.algo == ALGO_NVLS) {
        const char* rp[kMaxPeers];
        const char* rmc = nullptr;
        // only facts that every rank shares decide; a source that is not 16-byte aligned is handled inside the kernel
        if ((sendcount * es) % 16 == 0 && sym_view(recv, bytes, rp, &rmc) && rmc && (uintptr_t)rmc % 16 == 0) {
            a.symmetric = 1;
            a.io.recv_mc = (char*)rmc;
            a.mode = NV_ALLGATHER;
            a.count = sendcount;
            NEXT_SEQ(a);
            launches_++;
        symmetric_calls_++;
            return cuda_result(launch_nvls(a, dt, cfg), "nvls all-gather (symmetric)");
        }
    }
    size_t cap = ch.algo == ALGO_NVLS ? nvls_capacity(NV_ALLGATHER, n_, es, stage_bytes_)
                 : ch.algo == ALGO_RING ? ring_capacity(RING_ALLGATHER, n_, es, stage_bytes_)
                                        : twoshot_capacity(TS_ALLGATHER, n_, es, stage_bytes_);
    for (size_t off = 0; off < sendcount; off += cap) {
        const size_t c = sendcount - off < cap ? sendcount - off : cap;
        a.io.send = (const char*)send + off * es;
        a.io.recv = (char*)recv + off * es;
        a.count = c;
        NEXT_SEQ(a);
        cudaError_t e;
        if (ch.algo == ALGO_NVLS) { a.mode = NV_ALLGATHER; e = launch_nvls(a, dt, cfg); }
        else if (ch.algo == ALGO_RING) { a.mode = RING_ALLGATHER; e = launch_ring(a, dt, cfg); }
        else { a.mode = TS_ALLGATHER; e = launch_twoshot(a, dt, cfg); }
        launches_++;
        if (e != cudaSuccess) return cuda_result(e, "all-gather launch");
    }
    return ncclSuccess;
}

ncclResult_t GpuCommImpl::broadcast(const void* send, void* recv, size_t count, ncclDataType_t dt, int root,
                                    GpuAlgo algo, cudaStream_t stream) {
    DeviceGuard g(dev_);
    const size_t es = size_of_type(dt), bytes = count * es;
    if (n_ == 1) {
        last_[COLL_BROADCAST] = ALGO_LOCAL;
        if (send != recv && bytes) { launches_++; return cuda_result(launch_local_copy(recv, send, bytes, stream), "local copy"); }
        return ncclSuccess;
    }
    ncclResult_t pre = precheck();
    if (pre == ncclSuccess) pre = capture_check(stream, false);
    if (pre != ncclSuccess) return pre;
    if (!count) return ncclSuccess;
    CallScope scope(this, stream, COLL_BROADCAST, "dccl:broadcast");
    const bool nvls_ok = pool_.mc_base != nullptr;
    TuneChoice ch = tuner_.choose(COLL_BROADCAST, n_, bytes, nvls_ok, (int)es);
    if (algo != ALGO_AUTO) ch.algo = algo;
    if (ch.algo == ALGO_NVLS && !nvls_ok) ch.algo = ALGO_TWOSHOT;
    if (ch.algo != ALGO_NVLS && ch.algo != ALGO_ONESHOT) ch.algo = ALGO_TWOSHOT;
    last_[COLL_BROADCAST] = ch.algo;

    LaunchCfg cfg;
    cfg.ctas = ctas_for(ch.ctas);
    cfg.stream = stream;
    cfg.threads = threads_;
    if (rank_ != root) send = recv;   // only the root's source is read
    CollArgs a = base_args(send, recv, ncclSum, root);

    if (ch.algo == ALGO_ONESHOT && bytes <= oneshot_ll_capacity_bytes()) {
        a.mode = LL_BROADCAST;
        a.count = count;
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_ll_collective(a, dt, cfg), "packet broadcast");
    }
    if (ch.algo == ALGO_NVLS) {
        const char* rp[kMaxPeers];
        const char* rmc = nullptr;
        // every rank must take the same branch, so only properties that all ranks share may decide
        if (bytes % 16 == 0 && sym_view(recv, bytes, rp, &rmc) && rmc && (uintptr_t)rmc % 16 == 0 &&
            Config::global().get_bool("DCCL/symmetric_broadcast", false)) {
            a.symmetric = 1;
            a.io.recv_mc = (char*)rmc;
            a.mode = NV_BROADCAST;
            a.count = count;
            NEXT_SEQ(a);
            launches_++;
        symmetric_calls_++;
            return cuda_result(launch_nvls(a, dt, cfg), "nvls broadcast (symmetric)");
        }
    }
    // Large messages on buffers the peers can address (symmetric, registered, or ordinary ones mapped on first use): the
    // receivers load the message out of the root's buffer and out of each other's, no staging. The exchange is collective
    // and entered on facts every rank shares; the root describes its source, the others only their destination.
    // (two ranks: one hop, nothing to forward; it beats the staged form from 16 MB on)
    const size_t direct_min = n_ == 2 && direct_bcast_min_bytes_ > (16u << 20) ? (size_t)(16u << 20) : direct_bcast_min_bytes_;
    if (algo == ALGO_AUTO && direct_rooted_ && auto_min_bytes_ > 0 && bytes >= auto_min_bytes_ && bytes >= direct_min &&
        (ch.algo == ALGO_NVLS || ch.algo == ALGO_TWOSHOT)) {
        const char* sp[kMaxPeers];
        const char* rp[kMaxPeers];
        bool ok = auto_view(send, recv, sp, rp);
        ok = ok && (uintptr_t)sp[root] % 16 == 0;
        for (int p = 0; ok && p < n_; p++) ok = (uintptr_t)rp[p] % 16 == 0;
        if (ok) {
            zero_copy_calls_++;
            a.symmetric = 1;
            for (int p = 0; p < n_; p++) { a.io.send_peer[p] = sp[p]; a.io.recv_peer[p] = (char*)rp[p]; }
            if (ctas_override_ == 0) cfg.ctas = ctas_for(direct_bcast_ctas_);
            NEXT_SEQ(a);
            launches_++;
            last_[COLL_BROADCAST] = ALGO_TWOSHOT;
            return cuda_result(launch_direct_bcast(a, bytes, n_, cfg), "zero-copy broadcast");
        }
    }
    const int ts_mode = ch.algo == ALGO_ONESHOT ? TS_BROADCAST_DIRECT : TS_BROADCAST;
    // large messages through the switch: the receivers' copy-out overlaps the root's push chunk by chunk
    const bool rooted = ch.algo == ALGO_NVLS && rooted_pipe_ && bytes >= rooted_pipe_min_bytes_;
    size_t cap = rooted ? nvls_pipe_capacity(es, stage_bytes_, n_, false)
                 : ch.algo == ALGO_NVLS ? nvls_capacity(NV_BROADCAST, n_, es, stage_bytes_) : twoshot_capacity(ts_mode, n_, es, stage_bytes_);
    for (size_t off = 0; off < count; off += cap) {
        const size_t c = count - off < cap ? count - off : cap;
        a.io.send = (const char*)send + off * es;
        a.io.recv = (char*)recv + off * es;
        a.count = c;
        NEXT_SEQ(a);
        cudaError_t e;
        if (rooted) { a.mode = ROOTED_BROADCAST; e = launch_nvls_rooted(a, dt, cfg); }
        else if (ch.algo == ALGO_NVLS) { a.mode = NV_BROADCAST; e = launch_nvls(a, dt, cfg); }
        else { a.mode = ts_mode; e = launch_twoshot(a, dt, cfg); }
        launches_++;
        if (e != cudaSuccess) return cuda_result(e, "broadcast launch");
    }
    return ncclSuccess;
}

ncclResult_t GpuCommImpl::reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root,
                                 GpuAlgo algo, cudaStream_t stream) {
    DeviceGuard g(dev_);
    const size_t es = size_of_type(dt), bytes = count * es;
    if (n_ == 1) {
        last_[COLL_REDUCE] = ALGO_LOCAL;
        if (send != recv && bytes) { launches_++; return cuda_result(launch_local_copy(recv, send, bytes, stream), "local copy"); }
        return ncclSuccess;
    }
    ncclResult_t pre = precheck();
    if (pre == ncclSuccess) pre = capture_check(stream, false);
    if (pre != ncclSuccess) return pre;
    if (!count) return ncclSuccess;
    CallScope scope(this, stream, COLL_REDUCE, "dccl:reduce");
    const bool nvls_ok = pool_.mc_base != nullptr && nvls_supports(dt, op);
    TuneChoice ch = tuner_.choose(COLL_REDUCE, n_, bytes, nvls_ok, (int)es);
    if (algo != ALGO_AUTO) ch.algo = algo;
    if (ch.algo == ALGO_NVLS && !nvls_ok) ch.algo = ALGO_TWOSHOT;
    if (ch.algo == ALGO_ONESHOT && bytes > oneshot_ll_capacity_bytes()) ch.algo = ALGO_TWOSHOT;
    if (ch.algo == ALGO_TWOSHOT_LL && bytes > ll_twoshot_capacity_bytes(n_)) ch.algo = ALGO_TWOSHOT;
    if (ch.algo != ALGO_NVLS && ch.algo != ALGO_ONESHOT && ch.algo != ALGO_TWOSHOT_LL) ch.algo = ALGO_TWOSHOT;
    last_[COLL_REDUCE] = ch.algo;

    LaunchCfg cfg;
    cfg.ctas = ctas_for(ch.ctas);
    cfg.stream = stream;
    cfg.threads = threads_;
    CollArgs a = base_args(send, recv, op, root);
    if (ch.algo == ALGO_ONESHOT) {
        a.mode = LL_REDUCE;
        a.count = count;
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_ll_collective(a, dt, cfg), "packet reduce");
    }
    if (ch.algo == ALGO_TWOSHOT_LL) {
        a.mode = LL2_REDUCE;
        a.count = count;
        NEXT_SEQ(a);
        launches_++;
        return cuda_result(launch_ll_twoshot(a, dt, cfg), "two-shot packet reduce");
    }
    // Large messages on buffers the peers can address: the ranks other than the root fold one shard each straight out of
    // every rank's send buffer into the root's receive buffer. Only the root's receive buffer matters.
    // (measured: at 8 ranks it beats the staged form from 4 MB on; at 2 ranks the staged form is still ahead at 16 MB, 43.7 against
    // 47.9 us, and behind at 256 MB, 669 against 562 us; small worlds therefore start at 32 MB)
    const size_t reduce_min = n_ > 4 || direct_reduce_small_ ? auto_min_bytes_ : (auto_min_bytes_ > (32u << 20) ? auto_min_bytes_ : (size_t)(32u << 20));
    if (algo == ALGO_AUTO && direct_rooted_ && auto_min_bytes_ > 0 && bytes >= reduce_min && (ch.algo == ALGO_NVLS || ch.algo == ALGO_TWOSHOT)) {
        const char* sp[kMaxPeers];
        const char* rp[kMaxPeers];
        bool ok = auto_view(send, rank_ == root ? recv : send, sp, rp);
        ok = ok && (uintptr_t)rp[root] % 16 == 0;
        for (int p = 0; ok && p < n_; p++) ok = (uintptr_t)sp[p] % 16 == 0;
        if (ok) {
            zero_copy_calls_++;
            a.symmetric = 1;
            for (int p = 0; p < n_; p++) { a.io.send_peer[p] = sp[p]; a.io.recv_peer[p] = (char*)rp[p]; }
            a.mode = DIRECT_REDUCE;
            a.count = count;
            if (ctas_override_ == 0) cfg.ctas = ctas_for(direct_rooted_ctas_);
            NEXT_SEQ(a);
            launches_++;
            last_[COLL_REDUCE] = ALGO_TWOSHOT;
            return cuda_result(launch_direct(a, dt, cfg), "zero-copy reduce");
        }
    }
    // large messages through the switch: every rank's copy-in overlaps the root's switch pass chunk by chunk
    const bool rooted = ch.algo == ALGO_NVLS && rooted_pipe_ && bytes >= rooted_pipe_min_bytes_;
    size_t cap = rooted ? nvls_pipe_capacity(es, stage_bytes_, n_, false)
                 : ch.algo == ALGO_NVLS ? nvls_capacity(NV_REDUCE, n_, es, stage_bytes_) : twoshot_capacity(TS_REDUCE, n_, es, stage_bytes_);
    for (size_t off = 0; off < count; off += cap) {
        const size_t c = count - off < cap ? count - off : cap;
        a.io.send = (const char*)send + off * es;
        a.io.recv = recv ? (char*)recv + off * es : nullptr;
        a.count = c;
        NEXT_SEQ(a);
        cudaError_t e;
        if (rooted) { a.mode = ROOTED_REDUCE; e = launch_nvls_rooted(a, dt, cfg); }
        else if (ch.algo == ALGO_NVLS) { a.mode = NV_REDUCE; e = launch_nvls(a, dt, cfg); }
        else { a.mode = TS_REDUCE; e = launch_twoshot(a, dt, cfg); }
        launches_++;
        if (e != cudaSuccess) return cuda_result(e, "reduce launch");
    }
    return ncclSuccess;
}

/* ---------------- point to point ---------------- */

ncclResult_t GpuCommImpl::p2p_launch(std::vector<P2pOp>& ops, cudaStream_t stream, int ctas_per_op) {
    if (ctas_per_op <= 0) ctas_per_op = p2p_ctas_;
    DeviceGuard g(dev_);
    for (size_t first = 0; first < ops.size(); first += kMaxP2pOps) {
        P2pArgs a;
        memset(&a, 0, sizeof(a));
        a.comm = dc_;
        a.ctas_per_op = ctas_per_op;
        a.nops = (int)(ops.size() - first < (size_t)kMaxP2pOps ? ops.size() - first : (size_t)kMaxP2pOps);
        // Within one launch the receivers get the lower block numbers: they never wait for anything but data, so once
        // they are resident every sender that waits for FIFO credit waits for a CTA that runs, however many CTAs the
        // launch has. Batches keep the recording order, so that both ends of a transfer land in the same batch when
        // the ranks record their operations in matching order.
        std::stable_partition(ops.begin() + (long)first, ops.begin() + (long)first + a.nops, [](const P2pOp& o) { return o.is_send == 0; });
        for (int i = 0; i < a.nops; i++) a.ops[i] = ops[first + i];
        // what this rank has mapped of the peers it sends large messages to in this launch: their symmetric segments and
        // their exported allocations, newest first; the receiver's kernel says which buffer it is, the sender's kernel looks here
        a.nmaps = 0;
        bool listed[kMaxPeers] = {false};
        for (int i = 0; i < a.nops; i++) {
            const P2pOp& o = a.ops[i];
            if (!o.is_send || !o.rdv || listed[o.peer]) continue;
            listed[o.peer] = true;
            for (size_t k = 0; k < user_segs_.size() && a.nmaps < kMaxP2pMaps; k++) {
                P2pMap& m = a.maps[a.nmaps++];
                m.peer = o.peer; m.kind = P2P_DST_SYM; m.a = k; m.id = 0; m.size = user_segs_[k].size; m.mapped = user_segs_[k].base[o.peer];
            }
            std::vector<const std::pair<const std::pair<int, unsigned long long>, AutoImport>*> mine;
            for (const auto& kv : auto_imports_) if (kv.first.first == o.peer) mine.push_back(&kv);
            std::sort(mine.begin(), mine.end(), [](auto* x, auto* y) { return x->second.stamp > y->second.stamp; });
            for (const auto* kv : mine) {
                if (a.nmaps >= kMaxP2pMaps) break;
                P2pMap& m = a.maps[a.nmaps++];
                m.peer = o.peer; m.kind = P2P_DST_IPC; m.a = kv->first.second; m.id = kv->second.id; m.size = kv->second.size; m.mapped = (char*)kv->second.mapped;
            }
        }
        LaunchCfg cfg;
        cfg.ctas = a.nops * ctas_per_op;
        cfg.stream = stream;
        cfg.threads = threads_;
        a.ctas_per_rank = cfg.ctas;
        launches_++;
        cudaError_t e = launch_p2p(a, cfg);
        if (e != cudaSuccess) return cuda_result(e, "send/recv launch");
    }
    return ncclSuccess;
}

ncclResult_t GpuCommImpl::send(const void* buf, size_t bytes, int peer, cudaStream_t stream) {
    ncclResult_t pre = precheck();
    if (pre == ncclSuccess) pre = capture_check(stream, true);
    if (pre != ncclSuccess) return pre;
    last_[COLL_SENDRECV] = ALGO_ONESHOT;
    if (!bytes) return ncclSuccess;
    P2pOp op;
    memset(&op, 0, sizeof(op));
    op.is_send = 1; op.peer = peer; op.buf = (char*)buf; op.bytes = bytes; op.chunk_base = sent_chunks_[peer];
    sent_chunks_[peer] += p2p_chunks(bytes);
    if (p2p_rdv_ && bytes >= kP2pRdvMinBytes) {     // a large message: meet the receiver first, zero-copy where its buffer is mapped here
        DeviceGuard g(dev_);
        op.rdv = 1;
        op.rdv_index = sent_rdv_[peer]++;
        poll_exports(peer);
    }
    if (in_group_) { if (group_ops_.empty()) group_stream_ = stream; group_ops_.push_back(op); return ncclSuccess; }
    std::vector<P2pOp> ops{op};
    return p2p_launch(ops, stream);
}

ncclResult_t GpuCommImpl::recv(void* buf, size_t bytes, int peer, cudaStream_t stream) {
    ncclResult_t pre = precheck();
    if (pre == ncclSuccess) pre = capture_check(stream, true);
    if (pre != ncclSuccess) return pre;
    last_[COLL_SENDRECV] = ALGO_ONESHOT;
    if (!bytes) return ncclSuccess;
    P2pOp op;
    memset(&op, 0, sizeof(op));
    op.is_send = 0; op.peer = peer; op.buf = (char*)buf; op.bytes = bytes; op.chunk_base = recv_chunks_[peer];
    recv_chunks_[peer] += p2p_chunks(bytes);
    if (p2p_rdv_ && bytes >= kP2pRdvMinBytes) {
        DeviceGuard g(dev_);
        op.rdv = 1;
        op.rdv_index = recv_rdv_[peer]++;
        describe_receive_buffer(buf, bytes, &op);
    }
    if (in_group_) { if (group_ops_.empty()) group_stream_ = stream; group_ops_.push_back(op); return ncclSuccess; }
    std::vector<P2pOp> ops{op};
    return p2p_launch(ops, stream);
}

ncclResult_t GpuCommImpl::group_end() {
    in_group_ = false;
    const int per_op = group_ctas_;
    group_ctas_ = 0;
    if (group_ops_.empty()) return ncclSuccess;
    std::vector<P2pOp> ops;
    ops.swap(group_ops_);
    return p2p_launch(ops, group_stream_, per_op);
}

} // namespace dccl
