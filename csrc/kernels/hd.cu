/**
 * Rabenseifner all-reduce (recursive halving reduce-scatter + recursive doubling
 * all-gather) as one kernel, for any world size.
 *
 * Same exchange pattern as the original (reference
 * src/core/reduce_scatter_recursive_halving.cpp:66-111 and
 * all_gather_recursive_doubling.cpp:48-74): step k pairs rank r with r XOR 2^k,
 * the active region halves every step, and the gather walks back with the held
 * region doubling every step (the doubling the shipped original leaves commented
 * out). log2(n) exchanges each way instead of n-1. Halves are pushed into the
 * partner's staging at their absolute position, one area per halving step and
 * one for the gather. Work is dealt
 * to CTAs by absolute position (block-cyclic), so a CTA only ever reads
 * partial sums that it produced itself in the previous step and the only
 * synchronisation is the flag between CTA b and CTA b of the partner.
 *
 * A world that is not a power of two, n = 2^m + r, is folded onto 2^m ranks the
 * way the original does it (reference
 * src/core/all_reduce_recursive_halving_and_doubling.cpp:37-67,72-151,182-196):
 * the first 2r ranks pair up, even rank = leader, odd rank = follower. The
 * follower pushes its vector to the leader, which adds it to its own and takes
 * part in the exchange as rank old/2 of the sub-world (the others as old - r);
 * at the end the leader pushes the result to its follower. (The original splits
 * the pre-step between the two so that each adds one half; over NVLink the whole
 * vector crosses the link either way, and one add on the leader costs less than
 * a second exchange.)
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"
#include "../device/geometry.cuh"

namespace dccl {

constexpr size_t kHdChunkBytes = 16u << 10;   // dealing unit

/** Calls f(lo, n) for every piece of [lo,hi) (elements) that belongs to CTA bid. */
template <typename T, typename F>
__device__ __forceinline__ void for_my_pieces(size_t lo, size_t hi, int bid, int nb, F f) {
    constexpr size_t CE = kHdChunkBytes / sizeof(T);
    for (size_t ch = lo / CE; ch * CE < hi; ch++) {
        if ((int)(ch % (size_t)nb) != bid) continue;
        size_t a = ch * CE, b = a + CE;
        if (a < lo) a = lo;
        if (b > hi) b = hi;
        if (b > a) f(a, b - a);
    }
}

template <typename T, int OP>
__device__ __forceinline__ void hd_body(const CollArgs& a, const Ctx& x) {
    constexpr size_t VE = 16 / sizeof(T);
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank;
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    const size_t count = a.count;
    const size_t area = (count + VE - 1) / VE * VE;          // elements per staging area
    const bool avg = a.op == (int)ncclAvg;
    int steps = 0;
    while ((2 << steps) <= n) steps++;                        // sub-world of 2^steps ranks
    const int sub = 1 << steps, rem = n - sub;                // the first 2 * rem ranks are leader / follower pairs
    const bool paired = r < 2 * rem, follower = paired && (r & 1);
    const int nr = paired ? r / 2 : r - rem;                  // rank in the sub-world (followers: their leader's)
    auto old_of = [&](int v) { return v < rem ? 2 * v : v + rem; };
    const int areas = steps + 1 + (rem ? 1 : 0);
    if (!DCCL_BOUNDS_OK(c, steps <= 4, 1902, steps) || !stage_extent_ok<T>(c, (size_t)areas * area, 1902)) return;
    // one receive area per halving step (the regions received in successive steps are nested, so
    // they must not share memory), one for the gather (those regions are disjoint), and, in a world that is not a
    // power of two, one for the vector that travels between follower and leader
    T* my_stage = stage_ptr<T>(c, r, x.parity);
    T* my_ag = my_stage + (size_t)steps * area;
    T* my_pair = my_stage + (size_t)(steps + 1) * area;
    const int idx_pre = 2 * steps, idx_post = 2 * steps + 1;

    if (follower) {
        // hand the vector to the leader, then wait for the result
        const int leader = r - 1;
        T* dst = stage_ptr<T>(c, leader, x.parity) + (size_t)(steps + 1) * area;
        for_my_pieces<T>(0, count, x.bid, x.nb, [&](size_t p, size_t len) { copy_range<T>(dst + p, send + p, len); });
        cta_signal_peer(c, leader, x.bid, x.seq, idx_pre);
        if (!cta_wait_peer(c, leader, x.bid, x.seq, idx_post, 790)) return;
        for_my_pieces<T>(0, count, x.bid, x.nb, [&](size_t p, size_t len) { copy_range<T>(recv + p, my_pair + p, len); });
        return;
    }

    size_t los[4], his[4];
    size_t lo = 0, hi = count;
    const T* cur = send;                                     // where my current partial sums live
    if (paired) {
        // leader: add the follower's vector (this CTA's pieces: the pieces it will work on in every later step)
        if (!cta_wait_peer(c, r + 1, x.bid, x.seq, idx_pre, 780)) return;
        for_my_pieces<T>(0, count, x.bid, x.nb, [&](size_t p, size_t len) {
            const T* ins[1] = {my_pair + p};
            reduce_range<T, OP>(recv + p, nullptr, send + p, ins, 1, len, false, n);
        });
        __syncthreads();
        cur = recv;
    }
    for (int k = 0; k < steps; k++) {
        const int peer = old_of(nr ^ (1 << k));
        los[k] = lo; his[k] = hi;
        size_t mid = lo + ((hi - lo) / 2 + VE - 1) / VE * VE;
        if (mid > hi) mid = hi;
        size_t klo, khi, slo, shi;
        if (!((nr >> k) & 1)) { klo = lo; khi = mid; slo = mid; shi = hi; }
        else { klo = mid; khi = hi; slo = lo; shi = mid; }
        T* peer_rs = stage_ptr<T>(c, peer, x.parity) + (size_t)k * area;
        const T* my_rs = my_stage + (size_t)k * area;
        for_my_pieces<T>(slo, shi, x.bid, x.nb, [&](size_t p, size_t len) { copy_range<T>(peer_rs + p, cur + p, len); });
        cta_signal_peer(c, peer, x.bid, x.seq, k);
        if (!cta_wait_peer(c, peer, x.bid, x.seq, k, 700 + k)) return;
        const bool last = k == steps - 1;
        for_my_pieces<T>(klo, khi, x.bid, x.nb, [&](size_t p, size_t len) {
            const T* ins[1] = {my_rs + p};
            reduce_range<T, OP>(recv + p, nullptr, cur + p, ins, 1, len, last && avg, n);
        });
        __syncthreads();
        cur = recv;
        lo = klo; hi = khi;
    }
    if (steps == 0 && send != recv) for_my_pieces<T>(0, count, x.bid, x.nb, [&](size_t p, size_t len) { copy_range<T>(recv + p, send + p, len); });

    for (int k = steps - 1; k >= 0; k--) {
        const int peer = old_of(nr ^ (1 << k));
        const size_t plo = los[k], phi = his[k];
        size_t olo, ohi;
        if (lo == plo) { olo = hi; ohi = phi; } else { olo = plo; ohi = lo; }
        T* peer_ag = stage_ptr<T>(c, peer, x.parity) + (size_t)steps * area;
        for_my_pieces<T>(lo, hi, x.bid, x.nb, [&](size_t p, size_t len) { copy_range<T>(peer_ag + p, recv + p, len); });
        const int idx = steps + (steps - 1 - k);
        cta_signal_peer(c, peer, x.bid, x.seq, idx);
        if (!cta_wait_peer(c, peer, x.bid, x.seq, idx, 750 + k)) return;
        for_my_pieces<T>(olo, ohi, x.bid, x.nb, [&](size_t p, size_t len) { copy_range<T>(recv + p, my_ag + p, len); });
        __syncthreads();
        lo = plo; hi = phi;
    }
    if (paired) {
        // leader: the result for the follower
        T* dst = stage_ptr<T>(c, r + 1, x.parity) + (size_t)(steps + 1) * area;
        for_my_pieces<T>(0, count, x.bid, x.nb, [&](size_t p, size_t len) { copy_range<T>(dst + p, recv + p, len); });
        cta_signal_peer(c, r + 1, x.bid, x.seq, idx_post);
    }
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_hd(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    hd_body<T, OP>(a, x);
    finish_call(x);
}

size_t hd_capacity(int nranks, size_t es, size_t stage_bytes) {
    int steps = 0;
    while ((2 << steps) <= nranks) steps++;
    const int areas = steps + 1 + ((1 << steps) != nranks ? 1 : 0);
    const size_t ve = 16 / es;
    return stage_bytes / es / (size_t)areas / ve * ve;
}

cudaError_t launch_hd(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg) {
#define CALL(T, OP) return launch_coll(k_hd<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
