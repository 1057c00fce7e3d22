/**
 * Flag-in-data (packet) variants of reduce-scatter, all-gather, broadcast and
 * reduce for small messages: same 16-byte packets {data0, tag, data1, tag} and
 * the same two packet generations as the one-shot all-reduce (oneshot_ll.cu).
 * One launch, one NVLink crossing, no barrier:
 *
 *   reduce-scatter  push shard p of my input to rank p; fold the n-1 packets that arrive
 *                   with my own shard, in rank order
 *   all-gather      push my slot to everybody; copy the n-1 slots that arrive
 *   broadcast       the root pushes, the others poll
 *   reduce          everybody pushes to the root, the root folds in rank order
 *
 * The two packet generations are safe to alternate as long as a rank that has
 * left call m knows that every rank has ENTERED call m (and so has left every
 * earlier call, in stream order): it can then reach the generation of call m-1
 * again only after everybody is done reading it. Reduce-scatter and all-gather
 * give that for free, a rank only finishes after it has seen every peer's
 * packets of this call. In the rooted forms a rank would otherwise hear from
 * the root only (or, as a sender of a reduce, from nobody), so there every CTA
 * announces its entry to the same CTA of every peer with a flag when it starts
 * and checks all peers' announcements before it leaves; by then they have
 * normally long arrived. This covers the other kernels as well: whatever ran
 * before or runs after a rooted call sees the same guarantee.
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"

namespace dccl {

__device__ __forceinline__ char* ll_slot2(const DevComm& c, int owner, int parity, int src) {
    return c.pool[owner] + kLLOff + ((size_t)parity * kMaxPeers + (size_t)src) * kLLSlotBytes;
}

union Pack8 { uint2 u; unsigned char b[8]; };

__device__ __forceinline__ uint2 load8(const char* p, int valid, bool fast) {
    Pack8 v;
    v.u = make_uint2(0u, 0u);
    if (fast && valid == 8) v.u = *reinterpret_cast<const uint2*>(p);
    else for (int k = 0; k < valid; k++) v.b[k] = (unsigned char)p[k];
    return v.u;
}
__device__ __forceinline__ void store8(char* p, uint2 u, int valid, bool fast) {
    if (fast && valid == 8) { *reinterpret_cast<uint2*>(p) = u; return; }
    Pack8 v;
    v.u = u;
    for (int k = 0; k < valid; k++) p[k] = (char)v.b[k];
}

/** Poll one packet until both halves carry `tag`; false after the timeout or on abort. */
__device__ __forceinline__ bool poll_packet(const DevComm& c, const char* slot, uint32_t tag, int peer, uint32_t seq, uint2* out) {
    uint4 v = ld_volatile_v4(slot);
    uint32_t spins = 0;
    unsigned long long t0 = 0;
    while (v.y != tag || v.w != tag) {
        if ((++spins & 0xffu) == 0) {
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > c.timeout_ns) { report_failure(c, DEV_TIMEOUT, peer, 310, seq); return false; }
            if ((spins & 0xfffu) == 0 && ld_volatile_u32(c.abort_word) != 0) { report_failure(c, DEV_ABORTED, peer, 310, seq); return false; }
        }
        v = ld_volatile_v4(slot);
    }
    *out = make_uint2(v.x, v.z);
    return true;
}

template <typename T, int OP>
__device__ __forceinline__ void ll_collective_body(const CollArgs& a, const Ctx& x) {
    using A = typename Traits<T>::Acc;
    constexpr int N = 8 / (int)sizeof(T);
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank, mode = a.mode, root = a.root;
    const char* send = reinterpret_cast<const char*>(x.io->send);
    char* recv = reinterpret_cast<char*>(x.io->recv);
    const size_t nbytes = a.count * sizeof(T);            // per-rank payload
    const size_t sbytes = a.stride * sizeof(T);           // distance between slots in the user buffer (RS / AG)
    const size_t npk = (nbytes + 7) / 8;
    const uint32_t tag = x.seq;
    const bool avg = a.op == (int)ncclAvg;
    const bool fin = (reinterpret_cast<uintptr_t>(send) & 7u) == 0 && (sbytes & 7u) == 0;
    const bool fout = (reinterpret_cast<uintptr_t>(recv) & 7u) == 0 && (sbytes & 7u) == 0;
    bool ok = true;
    if (!DCCL_BOUNDS_OK(c, npk * 16 <= kLLSlotBytes, 1904, npk)) return;   // one packet slot per source rank
    const bool rooted = mode == LL_BROADCAST || mode == LL_REDUCE;
    // entry announcement (see the file comment); nothing has to be ordered before it
    if (rooted && (int)threadIdx.x < n && (int)threadIdx.x != r) signal_peer(c, (int)threadIdx.x, x.bid, x.seq, 0);

    for (size_t i = (size_t)x.bid * blockDim.x + threadIdx.x; i < npk && ok; i += (size_t)x.nb * blockDim.x) {
        const size_t off = i * 8;
        const int valid = nbytes - off >= 8 ? 8 : (int)(nbytes - off);
        if (mode == LL_REDUCESCATTER || (mode == LL_REDUCE)) {
            const bool reducer = mode == LL_REDUCESCATTER || r == root;
            // senders: shard p of my input goes to rank p (reduce-scatter) / my input goes to the root (reduce)
            if (mode == LL_REDUCESCATTER) {
                for (int k = 1; k < n; k++) {
                    const int p = (r + k) % n;
                    const uint2 d = load8(send + (size_t)p * sbytes + off, valid, fin);
                    st_volatile_v4(ll_slot2(c, p, x.parity, r) + i * 16, make_uint4(d.x, tag, d.y, tag));
                }
            } else if (r != root) {
                const uint2 d = load8(send + off, valid, fin);
                st_volatile_v4(ll_slot2(c, root, x.parity, r) + i * 16, make_uint4(d.x, tag, d.y, tag));
            }
            if (reducer) {
                const size_t own_off = mode == LL_REDUCESCATTER ? (size_t)r * sbytes + off : off;
                A acc[N];
                for (int p = 0; p < n && ok; p++) {
                    union { uint2 u; T e[N]; } v;
                    if (p == r) v.u = load8(send + own_off, valid, fin);
                    else ok = poll_packet(c, ll_slot2(c, r, x.parity, p) + i * 16, tag, p, x.seq, &v.u);
                    if (!ok) break;
                    if (p == 0) {
#pragma unroll
                        for (int e = 0; e < N; e++) acc[e] = Traits<T>::up(v.e[e]);
                    } else {
#pragma unroll
                        for (int e = 0; e < N; e++) acc[e] = op_apply<OP, A>(acc[e], Traits<T>::up(v.e[e]));
                    }
                }
                if (ok) {
                    union { uint2 u; T e[N]; } o;
#pragma unroll
                    for (int e = 0; e < N; e++) o.e[e] = Traits<T>::down(avg ? avg_finish<A>(acc[e], n) : acc[e]);
                    store8(recv + off, o.u, valid, fout);
                }
            }
        } else if (mode == LL_ALLGATHER) {
            const uint2 d = load8(send + off, valid, fin);
            const uint4 pkt = make_uint4(d.x, tag, d.y, tag);
            for (int k = 1; k < n; k++) st_volatile_v4(ll_slot2(c, (r + k) % n, x.parity, r) + i * 16, pkt);
            if (recv + (size_t)r * sbytes != send) store8(recv + (size_t)r * sbytes + off, d, valid, fout);
            for (int k = 1; k < n && ok; k++) {
                const int p = (r + k) % n;
                uint2 v;
                ok = poll_packet(c, ll_slot2(c, r, x.parity, p) + i * 16, tag, p, x.seq, &v);
                if (ok) store8(recv + (size_t)p * sbytes + off, v, valid, fout);
            }
        } else {  // LL_BROADCAST
            if (r == root) {
                const uint2 d = load8(send + off, valid, fin);
                const uint4 pkt = make_uint4(d.x, tag, d.y, tag);
                for (int k = 1; k < n; k++) st_volatile_v4(ll_slot2(c, (r + k) % n, x.parity, r) + i * 16, pkt);
                if (recv != send) store8(recv + off, d, valid, fout);
            } else {
                uint2 v;
                ok = poll_packet(c, ll_slot2(c, r, x.parity, root) + i * 16, tag, root, x.seq, &v);
                if (ok) store8(recv + off, v, valid, fout);
            }
        }
    }

    // rooted forms: nobody leaves before everybody has entered
    if (rooted && ok && (int)threadIdx.x < n && (int)threadIdx.x != r) wait_peer(c, (int)threadIdx.x, x.bid, x.seq, 0, 320);
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_ll_collective(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    ll_collective_body<T, OP>(a, x);
    finish_call(x);
}

cudaError_t launch_ll_collective(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg_in) {
    LaunchCfg cfg = cfg_in;
    const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                      : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
    const size_t npk = (a.count * es + 7) / 8;
    int threads = (int)((npk + 31) / 32 * 32);
    if (threads > 512) threads = 512;
    if (threads < 32) threads = 32;
    int ctas = (int)((npk + threads - 1) / threads);
    if (ctas > cfg.ctas) ctas = cfg.ctas;
    if (ctas < 1) ctas = 1;
    cfg.threads = threads;
    cfg.ctas = ctas;
    if (a.mode == LL_ALLGATHER || a.mode == LL_BROADCAST) {
        CollArgs b = a;
        b.count = a.count * es;
        b.stride = a.stride * es;
        b.op = (int)ncclSum;
        return launch_coll(k_ll_collective<uint8_t, OP_SUM>, b, cfg);
    }
#define CALL(T, OP) return launch_coll(k_ll_collective<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
