#include "cpu_backend.hpp"
#include "host_reduce.hpp"
#include "../core/config.hpp"
#include "../core/log.hpp"
#include <chrono>
#include <cstring>
#include <sched.h>

namespace dccl {

static inline int64_t mono_ms() {
    using namespace std::chrono;
    return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}

CpuBackend::CpuBackend(Bootstrap* bs) : bs_(bs), rank_(bs->rank()), world_(bs->world()) {
    timeout_ms_ = (int)Config::global().get_int("DCCL/timeout_ms", 5000);
}

char* CpuBackend::scratch(size_t bytes, int which) {
    // grows on demand and is kept for the life of the communicator (no per-call allocation)
    if (scratch_[which].size() < bytes) scratch_[which].resize(bytes);
    return scratch_[which].data();
}

static inline size_t round16(size_t b) { return (b + 15) & ~(size_t)15; }

CpuBackend::Xfer CpuBackend::make_send(int peer, const void* buf, size_t bytes) {
    return Xfer{true, peer, (char*)buf, bytes, round16(bytes), 0, false, ncclInt8, ncclSum};
}
CpuBackend::Xfer CpuBackend::make_recv(int peer, void* buf, size_t bytes) {
    return Xfer{false, peer, (char*)buf, bytes, round16(bytes), 0, false, ncclInt8, ncclSum};
}
CpuBackend::Xfer CpuBackend::make_recv_reduce(int peer, void* buf, size_t bytes, ncclDataType_t dt, ncclRedOp_t op) {
    return Xfer{false, peer, (char*)buf, bytes, round16(bytes), 0, true, dt, op};
}

/** Move as much of one transfer as the FIFO allows right now; true when something moved. */
bool CpuBackend::step(Xfer& x) {
    if (x.done == x.padded) return false;
    const size_t cap = bs_->channel_bytes();
    if (x.is_send) {
        ShmChannel* ch = bs_->channel(rank_, x.peer);
        char* ring = (char*)(ch + 1);
        uint64_t head = ch->head.load(std::memory_order_relaxed);
        uint64_t tail = ch->tail.load(std::memory_order_acquire);
        size_t free_b = cap - (size_t)(head - tail);
        if (!free_b) return false;
        size_t pos = (size_t)(head % cap);
        size_t n = x.padded - x.done;
        if (n > free_b) n = free_b;
        if (n > cap - pos) n = cap - pos;
        size_t data_n = x.done < x.bytes ? (x.bytes - x.done < n ? x.bytes - x.done : n) : 0;
        if (data_n) memcpy(ring + pos, x.buf + x.done, data_n);
        ch->head.store(head + n, std::memory_order_release);
        x.done += n;
        bytes_sent_ += data_n;
        return true;
    }
    ShmChannel* ch = bs_->channel(x.peer, rank_);
    char* ring = (char*)(ch + 1);
    uint64_t tail = ch->tail.load(std::memory_order_relaxed);
    uint64_t head = ch->head.load(std::memory_order_acquire);
    size_t avail = (size_t)(head - tail);
    if (!avail) return false;
    size_t pos = (size_t)(tail % cap);
    size_t n = x.padded - x.done;
    if (n > avail) n = avail;
    if (n > cap - pos) n = cap - pos;
    size_t data_n = x.done < x.bytes ? (x.bytes - x.done < n ? x.bytes - x.done : n) : 0;
    if (data_n) {
        // FIFO positions advance in multiples of 16 bytes, so whole elements are always contiguous
        if (x.reduce) host_reduce(x.buf + x.done, ring + pos, data_n / size_of_type(x.dt), x.dt, x.op);
        else memcpy(x.buf + x.done, ring + pos, data_n);
    }
    ch->tail.store(tail + n, std::memory_order_release);
    x.done += n;
    return true;
}

ncclResult_t CpuBackend::progress(std::vector<Xfer>& xs) {
    int64_t last = mono_ms();
    unsigned idle = 0;
    while (true) {
        bool moved = false, pending = false;
        for (auto& x : xs) {
            if (x.done == x.padded) continue;
            while (step(x)) moved = true;
            if (x.done != x.padded) pending = true;
        }
        if (!pending) return ncclSuccess;
        if (moved) { idle = 0; last = mono_ms(); continue; }
        if (++idle < 64) { __builtin_ia32_pause(); continue; }
        sched_yield();
        if ((idle & 255) == 0) {
            if (bs_->aborted()) {
                dccl_error("host transfer abandoned: group aborted (rank %d failed)", bs_->failed_rank());
                return ncclRemoteError;
            }
            if (mono_ms() - last > timeout_ms_) {
                for (auto& x : xs)
                    if (x.done != x.padded)
                        dccl_error("host %s with rank %d made no progress for %d ms (%zu of %zu bytes moved)",
                                   x.is_send ? "send" : "recv", x.peer, timeout_ms_, x.done, x.padded);
                return ncclInternalError;
            }
        }
    }
}

ncclResult_t CpuBackend::sendrecv(Xfer s, Xfer r) {
    std::vector<Xfer> xs;
    xs.push_back(s);
    xs.push_back(r);
    return progress(xs);
}

/* ------------------------------------------------------------------ *
 * ring
 * ------------------------------------------------------------------ */

static inline int mod(int a, int n) { int m = a % n; return m < 0 ? m + n : m; }

/**
 * In-place ring reduce-scatter over the `world` slots of buf. Step s sends slot
 * (rank - s + shift) to rank+1 and folds the slot arriving from rank-1 into
 * slot (rank - s - 1 + shift). Afterwards this rank owns slot (rank + 1 + shift).
 */
ncclResult_t CpuBackend::ring_reduce_scatter(char* buf, size_t count, ncclDataType_t dt, ncclRedOp_t op, int shift) {
    const int n = world_;
    const size_t es = size_of_type(dt);
    const int next = mod(rank_ + 1, n), prev = mod(rank_ - 1, n);
    for (int s = 0; s < n - 1; s++) {
        size_t slo, shi, rlo, rhi;
        slot_range(count, n, mod(rank_ - s + shift, n), 1, &slo, &shi);
        slot_range(count, n, mod(rank_ - s - 1 + shift, n), 1, &rlo, &rhi);
        ncclResult_t r = sendrecv(make_send(next, buf + slo * es, (shi - slo) * es),
                                  make_recv_reduce(prev, buf + rlo * es, (rhi - rlo) * es, dt, op));
        if (r != ncclSuccess) return r;
    }
    return ncclSuccess;
}

/** Ring all-gather; this rank starts out owning slot (rank + owner_shift). */
ncclResult_t CpuBackend::ring_all_gather(char* buf, size_t count, ncclDataType_t dt, int owner_shift) {
    const int n = world_;
    const size_t es = size_of_type(dt);
    const int next = mod(rank_ + 1, n), prev = mod(rank_ - 1, n);
    const int own = mod(rank_ + owner_shift, n);
    for (int s = 0; s < n - 1; s++) {
        size_t slo, shi, rlo, rhi;
        slot_range(count, n, mod(own - s, n), 1, &slo, &shi);
        slot_range(count, n, mod(own - s - 1, n), 1, &rlo, &rhi);
        ncclResult_t r = sendrecv(make_send(next, buf + slo * es, (shi - slo) * es),
                                  make_recv(prev, buf + rlo * es, (rhi - rlo) * es));
        if (r != ncclSuccess) return r;
    }
    return ncclSuccess;
}

/* ------------------------------------------------------------------ *
 * recursive halving / doubling
 * ------------------------------------------------------------------ */

/**
 * Recursive-halving reduce-scatter among `vworld` (a power of two) virtual
 * ranks. At step k the partner is vrank XOR 2^k; a rank whose bit k is clear
 * keeps the lower half of its current region. The regions visited are pushed
 * on lo_stack/hi_stack so the all-gather can walk back. The last entry pushed
 * is the region this rank ends up owning.
 */
ncclResult_t CpuBackend::halving_reduce_scatter(char* buf, size_t count, ncclDataType_t dt, ncclRedOp_t op,
                                                int vrank, int vworld, const std::vector<int>& v2r,
                                                std::vector<size_t>* lo_stack, std::vector<size_t>* hi_stack) {
    const size_t es = size_of_type(dt);
    size_t lo = 0, hi = count;
    lo_stack->clear(); hi_stack->clear();
    const int steps = (int)log_two((uint32_t)vworld);
    for (int k = 0; k < steps; k++) {
        lo_stack->push_back(lo); hi_stack->push_back(hi);
        const int peer = v2r[vrank ^ (1 << k)];
        const size_t mid = lo + (hi - lo) / 2;
        size_t klo, khi, slo, shi;
        if (!((vrank >> k) & 1)) { klo = lo; khi = mid; slo = mid; shi = hi; }
        else { klo = mid; khi = hi; slo = lo; shi = mid; }
        ncclResult_t r = sendrecv(make_send(peer, buf + slo * es, (shi - slo) * es),
                                  make_recv_reduce(peer, buf + klo * es, (khi - klo) * es, dt, op));
        if (r != ncclSuccess) return r;
        lo = klo; hi = khi;
    }
    lo_stack->push_back(lo); hi_stack->push_back(hi);
    return ncclSuccess;
}

/**
 * Recursive-doubling all-gather that undoes halving_reduce_scatter: walking
 * the stacks backwards, each step sends the region held so far and receives
 * the sibling half, so the held region doubles every step (the step the
 * original's shipped code leaves commented out, reference
 * all_gather_recursive_doubling.cpp:75-86).
 */
ncclResult_t CpuBackend::doubling_all_gather(char* buf, ncclDataType_t dt, int vrank, int vworld, const std::vector<int>& v2r,
                                             const std::vector<size_t>& lo_stack, const std::vector<size_t>& hi_stack) {
    const size_t es = size_of_type(dt);
    const int steps = (int)log_two((uint32_t)vworld);
    size_t lo = lo_stack[steps], hi = hi_stack[steps];
    for (int k = steps - 1; k >= 0; k--) {
        const int peer = v2r[vrank ^ (1 << k)];
        const size_t plo = lo_stack[k], phi = hi_stack[k];
        size_t olo, ohi;  // the sibling half
        if (lo == plo) { olo = hi; ohi = phi; } else { olo = plo; ohi = lo; }
        ncclResult_t r = sendrecv(make_send(peer, buf + lo * es, (hi - lo) * es),
                                  make_recv(peer, buf + olo * es, (ohi - olo) * es));
        if (r != ncclSuccess) return r;
        lo = plo; hi = phi;
    }
    return ncclSuccess;
}

/**
 * Rabenseifner all-reduce in place. world = 2^e + rem: the first 2*rem ranks
 * pair up (even = leader, odd = follower), swap halves, reduce one half each
 * and the follower hands its half back, so the leader holds the pair's
 * reduction (same roles as reference
 * all_reduce_recursive_halving_and_doubling.cpp:50-153). Leaders and the
 * remaining ranks run halving + doubling; leaders finally copy the result to
 * their followers.
 */
ncclResult_t CpuBackend::rabenseifner(char* buf, size_t count, ncclDataType_t dt, ncclRedOp_t op) {
    const size_t es = size_of_type(dt);
    const int n = world_;
    const int p2 = 1 << log_two((uint32_t)n);
    const int rem = n - p2;
    enum { LEADER, FOLLOWER, INDEPENDENT } role = INDEPENDENT;
    int vrank;
    if (rank_ < 2 * rem) { role = (rank_ & 1) ? FOLLOWER : LEADER; vrank = rank_ / 2; }
    else vrank = rank_ - rem;
    std::vector<int> v2r(p2);
    for (int v = 0; v < p2; v++) v2r[v] = v < rem ? 2 * v : v + rem;
    ncclResult_t r;

    const size_t half = count / 2;
    if (role == LEADER) {
        const int f = rank_ + 1;
        r = sendrecv(make_send(f, buf + half * es, (count - half) * es), make_recv_reduce(f, buf, half * es, dt, op));
        if (r != ncclSuccess) return r;
        std::vector<Xfer> xs{make_recv(f, buf + half * es, (count - half) * es)};
        if ((r = progress(xs)) != ncclSuccess) return r;
    } else if (role == FOLLOWER) {
        const int l = rank_ - 1;
        r = sendrecv(make_send(l, buf, half * es), make_recv_reduce(l, buf + half * es, (count - half) * es, dt, op));
        if (r != ncclSuccess) return r;
        std::vector<Xfer> xs{make_send(l, buf + half * es, (count - half) * es)};
        if ((r = progress(xs)) != ncclSuccess) return r;
    }
    TIMESTAMP(TT_ALLREDUCE_RDH_PREPROCESS, rank_, op);

    if (role != FOLLOWER) {
        std::vector<size_t> los, his;
        if ((r = halving_reduce_scatter(buf, count, dt, op, vrank, p2, v2r, &los, &his)) != ncclSuccess) return r;
        if (op == ncclAvg) host_finish_avg(buf + los.back() * es, his.back() - los.back(), dt, (uint32_t)n);
        TIMESTAMP(TT_ALLREDUCE_REDUCESCATTER, rank_, op);
        if ((r = doubling_all_gather(buf, dt, vrank, p2, v2r, los, his)) != ncclSuccess) return r;
        TIMESTAMP(TT_ALLREDUCE_ALLGATHER, rank_, op);
    } else {
        TIMESTAMP(TT_ALLREDUCE_REDUCESCATTER, rank_, op);
        TIMESTAMP(TT_ALLREDUCE_ALLGATHER, rank_, op);
    }

    if (role == LEADER) {
        std::vector<Xfer> xs{make_send(rank_ + 1, buf, count * es)};
        if ((r = progress(xs)) != ncclSuccess) return r;
    } else if (role == FOLLOWER) {
        std::vector<Xfer> xs{make_recv(rank_ - 1, buf, count * es)};
        if ((r = progress(xs)) != ncclSuccess) return r;
    }
    TIMESTAMP(TT_ALLREDUCE_RDH_POSTPROCESS, rank_, op);
    return ncclSuccess;
}

/* ------------------------------------------------------------------ *
 * entry points
 * ------------------------------------------------------------------ */

ncclResult_t CpuBackend::all_reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, HostAlgo algo) {
    const size_t es = size_of_type(dt);
    if (send != recv) memmove(recv, send, count * es);
    TIMESTAMP(TT_ALLREDUCE_MEMCPY, rank_, op);
    if (world_ == 1 || count == 0) return ncclSuccess;   // the average of one value is the value
    char* buf = (char*)recv;
    if (algo == HOST_ALGO_RABENSEIFNER) return rabenseifner(buf, count, dt, op);
    ncclResult_t r = ring_reduce_scatter(buf, count, dt, op, 0);
    if (r != ncclSuccess) return r;
    if (op == ncclAvg) {
        size_t lo, hi;
        slot_range(count, world_, mod(rank_ + 1, world_), 1, &lo, &hi);
        host_finish_avg(buf + lo * es, hi - lo, dt, (uint32_t)world_);
    }
    TIMESTAMP(TT_ALLREDUCE_REDUCESCATTER, rank_, op);
    r = ring_all_gather(buf, count, dt, +1);
    TIMESTAMP(TT_ALLREDUCE_ALLGATHER, rank_, op);
    return r;
}

ncclResult_t CpuBackend::reduce_scatter(const void* send, void* recv, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op, HostAlgo algo) {
    const size_t es = size_of_type(dt);
    if (world_ == 1) { if (send != recv) memmove(recv, send, recvcount * es); return ncclSuccess; }
    const size_t total = recvcount * (size_t)world_;
    // the input must stay intact, so the exchange runs in a work copy held by the communicator
    char* work = scratch(total * es, 0);
    memcpy(work, send, total * es);
    ncclResult_t r;
    if (algo == HOST_ALGO_RABENSEIFNER && is_power_of_two((uint32_t)world_)) {
        // virtual rank = bit-reversed rank, so that rank r ends up with slice r
        const uint32_t bits = log_two((uint32_t)world_);
        std::vector<int> v2r(world_);
        for (int v = 0; v < world_; v++) v2r[v] = (int)reverse_bits((uint32_t)v, bits);
        std::vector<size_t> los, his;
        r = halving_reduce_scatter(work, total, dt, op, (int)reverse_bits((uint32_t)rank_, bits), world_, v2r, &los, &his);
        if (r != ncclSuccess) return r;
        if (los.back() != recvcount * (size_t)rank_ || his.back() - los.back() != recvcount) return ncclInternalError;
    } else {
        r = ring_reduce_scatter(work, total, dt, op, -1);
        if (r != ncclSuccess) return r;
    }
    char* mine = work + recvcount * (size_t)rank_ * es;
    if (op == ncclAvg) host_finish_avg(mine, recvcount, dt, (uint32_t)world_);
    memcpy(recv, mine, recvcount * es);
    return ncclSuccess;
}

ncclResult_t CpuBackend::all_gather(const void* send, void* recv, size_t sendcount, ncclDataType_t dt, HostAlgo algo) {
    const size_t es = size_of_type(dt);
    char* buf = (char*)recv;
    char* mine = buf + sendcount * (size_t)rank_ * es;
    if (send != (const void*)mine) memmove(mine, send, sendcount * es);
    if (world_ == 1 || sendcount == 0) return ncclSuccess;
    const size_t total = sendcount * (size_t)world_;
    if (algo == HOST_ALGO_RABENSEIFNER && is_power_of_two((uint32_t)world_)) {
        // rebuild the region stacks the halving phase would have produced for the bit-reversed rank
        const uint32_t bits = log_two((uint32_t)world_);
        const int vrank = (int)reverse_bits((uint32_t)rank_, bits);
        std::vector<int> v2r(world_);
        for (int v = 0; v < world_; v++) v2r[v] = (int)reverse_bits((uint32_t)v, bits);
        std::vector<size_t> los, his;
        size_t lo = 0, hi = total;
        for (uint32_t k = 0; k < bits; k++) {
            los.push_back(lo); his.push_back(hi);
            size_t mid = lo + (hi - lo) / 2;
            if (!((vrank >> k) & 1)) hi = mid; else lo = mid;
        }
        los.push_back(lo); his.push_back(hi);
        return doubling_all_gather(buf, dt, vrank, world_, v2r, los, his);
    }
    return ring_all_gather(buf, total, dt, 0);
}

ncclResult_t CpuBackend::broadcast(const void* send, void* recv, size_t count, ncclDataType_t dt, int root) {
    const size_t bytes = count * size_of_type(dt);
    const int n = world_;
    if (rank_ == root && send != recv) memmove(recv, send, bytes);
    if (n == 1 || bytes == 0) return ncclSuccess;
    // binomial tree on ranks renumbered so that the root is 0
    const int vr = mod(rank_ - root, n);
    int mask = 1;
    while (mask < n) {
        if (vr & mask) {
            std::vector<Xfer> xs{make_recv(mod(vr - mask + root, n), recv, bytes)};
            ncclResult_t r = progress(xs);
            if (r != ncclSuccess) return r;
            break;
        }
        mask <<= 1;
    }
    mask >>= 1;
    std::vector<Xfer> xs;
    while (mask > 0) {
        if (vr + mask < n) xs.push_back(make_send(mod(vr + mask + root, n), recv, bytes));
        mask >>= 1;
    }
    return xs.empty() ? ncclSuccess : progress(xs);
}

ncclResult_t CpuBackend::reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root) {
    const size_t es = size_of_type(dt);
    const int n = world_;
    if (n == 1) { if (send != recv) memmove(recv, send, count * es); return ncclSuccess; }
    // ring reduce-scatter in the receive buffer (root) or in scratch (others), then the root collects the slots
    char* work = rank_ == root ? (char*)recv : scratch(count * es, 0);
    if ((const void*)work != send) memmove(work, send, count * es);
    if (count == 0) return ncclSuccess;
    ncclResult_t r = ring_reduce_scatter(work, count, dt, op, -1);
    if (r != ncclSuccess) return r;
    size_t lo, hi;
    slot_range(count, n, rank_, 1, &lo, &hi);
    if (op == ncclAvg) host_finish_avg(work + lo * es, hi - lo, dt, (uint32_t)n);
    std::vector<Xfer> xs;
    if (rank_ == root) {
        for (int p = 0; p < n; p++) {
            if (p == root) continue;
            slot_range(count, n, p, 1, &lo, &hi);
            if (hi > lo) xs.push_back(make_recv(p, work + lo * es, (hi - lo) * es));
        }
    } else if (hi > lo) xs.push_back(make_send(root, work + lo * es, (hi - lo) * es));
    return xs.empty() ? ncclSuccess : progress(xs);
}

ncclResult_t CpuBackend::send(const void* buf, size_t bytes, int peer) {
    Xfer x = make_send(peer, buf, bytes);
    if (in_group()) { group_.push_back(x); return ncclSuccess; }
    std::vector<Xfer> xs{x};
    return progress(xs);
}

ncclResult_t CpuBackend::recv(void* buf, size_t bytes, int peer) {
    Xfer x = make_recv(peer, buf, bytes);
    if (in_group()) { group_.push_back(x); return ncclSuccess; }
    std::vector<Xfer> xs{x};
    return progress(xs);
}

ncclResult_t CpuBackend::group_end() {
    if (group_depth_ > 0) group_depth_--;
    if (group_depth_ > 0 || group_.empty()) return ncclSuccess;
    // Transfers to or from the same peer must keep their order; progress() steps each
    // transfer in list order, and a later transfer on the same channel only moves after
    // the earlier one has finished.
    std::vector<Xfer> all;
    all.swap(group_);
    std::vector<Xfer> batch;
    ncclResult_t r = ncclSuccess;
    while (!all.empty() && r == ncclSuccess) {
        batch.clear();
        std::vector<Xfer> rest;
        for (auto& x : all) {
            bool clash = false;
            for (auto& b : batch) if (b.peer == x.peer && b.is_send == x.is_send) clash = true;
            if (clash) rest.push_back(x); else batch.push_back(x);
        }
        r = progress(batch);
        all.swap(rest);
    }
    return r;
}

} // namespace dccl
