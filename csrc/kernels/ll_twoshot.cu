/**
 * Two-shot all-reduce with the flag carried inside the data, for the sizes
 * between the one-shot packet variant and the bandwidth-bound ones.
 *
 * The one-shot variant (oneshot_ll.cu) sends the whole vector to every peer:
 * n-1 copies, twice their size as packets. Beyond about 100 KB that traffic
 * costs more than the second hop it saves. Here the vector is cut into n
 * shards and crosses NVLink twice, like the staged two-shot variant, but both
 * crossings use 16-byte packets {data0, tag, data1, tag} that the receiver
 * polls, so there is still no barrier and no flag round trip:
 *
 *   A  push shard p of my input to rank p                       (n-1 shards out)
 *      fold the n-1 packets that arrive for my shard with my own part, in rank
 *      order (16-bit floats in fp32, one rounding, 1/world scale of ncclAvg)
 *   B  push the folded shard to every peer and store it locally  (n-1 shards out)
 *      copy the n-1 folded shards that arrive into the receive buffer
 *
 * Per GPU 2 (n-1)/n of the vector goes out, doubled by the packet format,
 * against (n-1) times the vector, doubled, for the one-shot form. Every rank
 * stores the bits the shard's owner computed. Packets live in their own region
 * of the pool (two generations by call parity, two phases, one slot per source
 * rank), so this variant never touches the packets of the other kernels. A rank
 * only finishes after it has seen phase-B packets of this call from every
 * peer, so every peer has entered the call and is done with the previous
 * generation: no acknowledgement is needed.
 *
 * Reduce to a root is the same kernel with phase B sent to the root only. Phase
 * A still makes every rank wait for every other rank (the root owns a shard
 * and contributes to all shards), which is what keeps a fast rank from
 * reaching the same packet generation again before the root has read it.
 *
 * The original has one algorithm per call for all sizes (ring or Rabenseifner,
 * reference src/core/dccl.cpp:412-496), each step a host-driven RDMA transfer.
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"

namespace dccl {

size_t ll_twoshot_capacity_bytes(int nranks) { return (size_t)nranks * (kLL2PhaseBytes / 2); }

__device__ __forceinline__ char* ll2_slot(const DevComm& c, int owner, int parity, int phase, int src) {
    return c.pool[owner] + kLL2Off + (((size_t)parity * kMaxPeers + (size_t)src) * 2 + (size_t)phase) * kLL2PhaseBytes;
}

namespace {

union Pk8 { uint2 u; unsigned char b[8]; };

__device__ __forceinline__ uint2 ld8(const char* p, int valid, bool fast) {
    Pk8 v;
    v.u = make_uint2(0u, 0u);
    if (fast && valid == 8) v.u = *reinterpret_cast<const uint2*>(p);
    else for (int k = 0; k < valid; k++) v.b[k] = (unsigned char)p[k];
    return v.u;
}
__device__ __forceinline__ void st8(char* p, uint2 u, int valid, bool fast) {
    if (fast && valid == 8) { *reinterpret_cast<uint2*>(p) = u; return; }
    Pk8 v;
    v.u = u;
    for (int k = 0; k < valid; k++) p[k] = (char)v.b[k];
}

/** Poll one packet until both halves carry `tag`; false after the timeout or on abort. */
__device__ __forceinline__ bool poll2(const DevComm& c, const char* slot, uint32_t tag, int peer, int site, uint2* out) {
    uint4 v = ld_volatile_v4(slot);
    uint32_t spins = 0;
    unsigned long long t0 = 0;
    while (v.y != tag || v.w != tag) {
        if ((++spins & 0xffu) == 0) {
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > c.timeout_ns) { report_failure(c, DEV_TIMEOUT, peer, site, tag); return false; }
            if ((spins & 0xfffu) == 0 && ld_volatile_u32(c.abort_word) != 0) { report_failure(c, DEV_ABORTED, peer, site, tag); return false; }
        }
        v = ld_volatile_v4(slot);
    }
    *out = make_uint2(v.x, v.z);
    return true;
}

} // namespace

template <typename T, int OP>
__device__ __forceinline__ void ll_twoshot_body(const CollArgs& a, const Ctx& x) {
    using A = typename Traits<T>::Acc;
    constexpr int N = 8 / (int)sizeof(T);
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank;
    const char* send = reinterpret_cast<const char*>(x.io->send);
    char* recv = reinterpret_cast<char*>(x.io->recv);
    const size_t nbytes = a.count * sizeof(T);
    const size_t npk = (nbytes + 7) / 8;                 // packets in the whole vector
    const size_t per = (npk + (size_t)n - 1) / (size_t)n;   // packets per shard; shard j = packets [j*per, (j+1)*per)
    const uint32_t tag = x.seq;
    const bool avg = a.op == (int)ncclAvg;
    const bool rooted = a.mode == LL2_REDUCE;             // the folded shards go to a.root only
    const int root = a.root;
    const bool fast_in = (reinterpret_cast<uintptr_t>(send) & 7u) == 0, fast_out = (reinterpret_cast<uintptr_t>(recv) & 7u) == 0;
    const size_t first = (size_t)x.bid * blockDim.x + threadIdx.x, step = (size_t)x.nb * blockDim.x;
    auto valid_of = [&](size_t gi) { return gi >= npk ? 0 : (nbytes - gi * 8 >= 8 ? 8 : (int)(nbytes - gi * 8)); };
    // A rank leaves a call only when it knows that every rank has entered it (which is what lets the two packet
    // generations alternate). Folding a shard means hearing from everybody, but a vector too short to give every
    // rank a shard leaves some ranks with nothing to fold: then the CTAs announce their entry with a flag instead.
    const bool announce = (size_t)(n - 1) * per >= npk;
    if (!DCCL_BOUNDS_OK(c, per * 16 <= kLL2PhaseBytes, 1905, per)) return;   // one shard of packets per source rank and phase
    if (announce && (int)threadIdx.x < n && (int)threadIdx.x != r) signal_peer(c, (int)threadIdx.x, x.bid, x.seq, 0);

    /* A: my part of every other rank's shard goes to its owner */
    for (size_t i = first; i < per; i += step)
        for (int k = 1; k < n; k++) {
            const int p = (r + k) % n;
            const size_t gi = (size_t)p * per + i;
            const int valid = valid_of(gi);
            if (!valid) continue;                          // beyond the end of the vector: the owner does not wait for it
            const uint2 d = ld8(send + gi * 8, valid, fast_in);
            st_volatile_v4(ll2_slot(c, p, x.parity, 0, r) + i * 16, make_uint4(d.x, tag, d.y, tag));
        }

    /* fold my shard, then B: the result goes to everybody */
    for (size_t i = first; i < per; i += step) {
        const size_t gi = (size_t)r * per + i;
        const int valid = valid_of(gi);
        if (!valid) continue;
        union { uint2 u; T e[N]; } mine, theirs, out;
        mine.u = ld8(send + gi * 8, valid, fast_in);
        A acc[N];
        for (int p = 0; p < n; p++) {
            if (p == r) theirs.u = mine.u;
            else if (!poll2(c, ll2_slot(c, r, x.parity, 0, p) + i * 16, tag, p, 330, &theirs.u)) return;
            if (p == 0) {
#pragma unroll
                for (int e = 0; e < N; e++) acc[e] = Traits<T>::up(theirs.e[e]);
            } else {
#pragma unroll
                for (int e = 0; e < N; e++) acc[e] = op_apply<OP, A>(acc[e], Traits<T>::up(theirs.e[e]));
            }
        }
#pragma unroll
        for (int e = 0; e < N; e++) out.e[e] = Traits<T>::down(avg ? avg_finish<A>(acc[e], n) : acc[e]);
        const uint4 pkt = make_uint4(out.u.x, tag, out.u.y, tag);
        if (!rooted) {
            for (int k = 1; k < n; k++) st_volatile_v4(ll2_slot(c, (r + k) % n, x.parity, 1, r) + i * 16, pkt);
            st8(recv + gi * 8, out.u, valid, fast_out);
        } else if (r == root) st8(recv + gi * 8, out.u, valid, fast_out);
        else st_volatile_v4(ll2_slot(c, root, x.parity, 1, r) + i * 16, pkt);
    }
    if (announce && (int)threadIdx.x < n && (int)threadIdx.x != r && !wait_peer(c, (int)threadIdx.x, x.bid, x.seq, 0, 335)) return;
    if (rooted && r != root) return;

    /* the other shards arrive folded */
    for (size_t i = first; i < per; i += step)
        for (int k = 1; k < n; k++) {
            const int p = (r + n - k) % n;
            const size_t gi = (size_t)p * per + i;
            const int valid = valid_of(gi);
            if (!valid) continue;
            uint2 d;
            if (!poll2(c, ll2_slot(c, r, x.parity, 1, p) + i * 16, tag, p, 340, &d)) return;
            st8(recv + gi * 8, d, valid, fast_out);
        }
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_ll_twoshot(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    ll_twoshot_body<T, OP>(a, x);
    finish_call(x);
}

cudaError_t launch_ll_twoshot(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg_in) {
    LaunchCfg cfg = cfg_in;
    const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                      : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
    const int n = a.emu ? cfg.ranks_in_launch : a.comm.nranks;
    const size_t npk = (a.count * es + 7) / 8;
    const size_t per = (npk + (size_t)n - 1) / (size_t)n;
    // every rank derives the same shape from the same arguments: one thread per packet of a shard where that fits
    int threads = (int)((per + 31) / 32 * 32);
    if (threads > 512) threads = 512;
    if (threads < 32) threads = 32;
    int ctas = (int)((per + (size_t)threads - 1) / (size_t)threads);
    if (ctas > cfg.ctas) ctas = cfg.ctas;
    if (ctas < 1) ctas = 1;
    cfg.threads = threads;
    cfg.ctas = ctas;
#define CALL(T, OP) return launch_coll(k_ll_twoshot<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
