/**
 * Zero-copy peer all-reduce for buffers that every rank can address: symmetric
 * memory from dcclMemAlloc, or buffers registered with dcclRegisterCacheMemory.
 *
 * Rank r owns shard r of the vector. It loads shard r of EVERY rank's send
 * buffer over NVLink, folds the values in registers (16-bit floats in fp32, one
 * rounding), applies the 1/world scale and stores the result into shard r of
 * every rank's receive buffer. One pass, no staging, loads and stores in flight
 * together in both link directions. A barrier before the pass tells the peers
 * that this rank's kernel has started (so its send buffer is complete and its
 * receive buffer may be overwritten); a barrier after it tells them that their
 * receive buffers are complete and their send buffers are no longer read.
 *
 * The original reaches registered buffers with one RDMA write per ring step
 * (reference src/core/internal_common.hpp:713-769); here the registered mapping
 * is read and written directly by the reducing threads. This variant is the
 * choice where the switch cannot reduce (no multicast binding) and at world
 * size two, where multimem fetches the local copy through the switch as well.
 * Every rank stores identical bits: a shard is folded by exactly one rank.
 *
 * Reduce-scatter has the same form with one destination: rank r folds slot r of
 * every rank's send buffer into its own receive buffer (only the send buffers
 * have to be addressable by the peers).
 *
 * Reduce (to a root) cuts the vector into world - 1 shards, one per rank other
 * than the root: the owner folds its shard of every send buffer (the root's
 * included) and stores the result into the root's receive buffer. The root
 * itself folds nothing: its links already carry its send buffer out and the
 * whole result in, so every rank moves one message length in each direction.
 *
 * Broadcast is a scatter and an all-gather by peer STORES, pipelined: rank j
 * (not the root) owns shard j of world - 1, cut into chunks. The root stores
 * chunk k of every shard into its owner's receive buffer and announces it; the
 * owner reads the chunk back from its own memory and stores it into the other
 * receivers' buffers, so the root sends every byte once and all traffic is
 * posted writes (peer loads reached 370-560 GB/s on a pair of B200s where
 * stores reach 630-650). A receiver is done when the root has announced all
 * chunks of its own shard and every other owner has forwarded all of its own.
 * (The original's broadcast is a Derecho multicast into host memory, reference
 * src/core/dccl.cpp:701-736.)
 */
#include "kernels.hpp"
#include "../device/geometry.cuh"
#include "../device/reduce_ops.cuh"

/* a function of its own with its own register allocation: inlined into the broadcast kernel, the copy loops spilled */
#ifdef DCCL_HOST_SIM
#define DCCL_NOINLINE __attribute__((noinline))
#else
#define DCCL_NOINLINE __noinline__
#endif

namespace dccl {

/**
 * out = fold over `n` sources of `nvec` 16-byte vectors, stored to `ndst` destinations.
 * NR > 0: number of sources known at compile time, U vectors per source in flight per thread
 * (NR x U = 8 loads outstanding); NR == 0: any number, one vector per source.
 */
template <typename T, int OP, int NR>
__device__ __forceinline__ void direct_pass(const char* const* srcs, char* const* dsts, int n, int ndst, size_t nvec, bool avg) {
    using A = typename Traits<T>::Acc;
    constexpr int N = Vec16<T>::N;
    constexpr int U = NR == 0 ? 1 : 8 / NR;
    constexpr int S = NR == 0 ? kMaxPeers : NR;
    const size_t tid = threadIdx.x, nt = blockDim.x;
    const char* src[S];
    char* dst[S];
#pragma unroll
    for (int s = 0; s < S; s++) {
        src[s] = srcs[s < n ? s : 0];
        dst[s] = dsts[s < ndst ? s : 0];
    }
    for (size_t i0 = tid; i0 < nvec; i0 += (size_t)U * nt) {
        Vec16<T> v[S][U];
#pragma unroll
        for (int s = 0; s < S; s++) {
            if (s < n) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const size_t i = i0 + (size_t)u * nt;
                    if (i < nvec) v[s][u] = ld_vec<T>(src[s] + i * 16);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const size_t i = i0 + (size_t)u * nt;
            if (i >= nvec) break;
            A acc[N];
#pragma unroll
            for (int e = 0; e < N; e++) acc[e] = Traits<T>::up(v[0][u].e[e]);
#pragma unroll
            for (int s = 1; s < S; s++) {
                if (s < n) {
#pragma unroll
                    for (int e = 0; e < N; e++) acc[e] = op_apply<OP, A>(acc[e], Traits<T>::up(v[s][u].e[e]));
                }
            }
            Vec16<T> out;
#pragma unroll
            for (int e = 0; e < N; e++) out.e[e] = Traits<T>::down(avg ? avg_finish<A>(acc[e], n) : acc[e]);
#pragma unroll
            for (int s = 0; s < S; s++)
                if (s < ndst) st_vec<T>(dst[s] + i * 16, out);
        }
    }
}

template <typename T, int OP>
__device__ __forceinline__ void direct_body(const CollArgs& a, const Ctx& x) {
    using A = typename Traits<T>::Acc;
    const DevComm& c = *x.c;
    const RankIO& io = *x.io;
    const int n = c.nranks, r = c.rank;
    const bool avg = a.op == (int)ncclAvg;
    const bool rs = a.mode == DIRECT_REDUCESCATTER, red = a.mode == DIRECT_REDUCE;
    // all-reduce: this rank folds shard r of one vector; reduce-scatter: slot r (count elements) of every send buffer;
    // reduce: the ranks other than the root own the shards, numbered from the root's right-hand neighbour
    const int shards = red ? n - 1 : n, mine = red ? (r - a.root - 1 + n) % n : r;
    const Geometry<T> g(rs ? GEO_WHOLE : GEO_SPLIT, a.count, rs ? 1 : shards, x.bid, x.nb);

    if (!rank_barrier(c, x.bid, x.seq, 0, 900)) return;

    const size_t len = rs ? a.count : red && r == a.root ? 0 : g.len(mine);
    const size_t lo = g.blo < len ? g.blo : len, hi = g.bhi < len ? g.bhi : len;
    if (hi > lo) {
        // shard and CTA boundaries are multiples of one vector; only the very end of the message can be ragged
        const size_t first = (rs ? (size_t)r * a.stride : (size_t)mine * g.per) + lo, cnt = hi - lo;
        const size_t nvec = cnt / Vec16<T>::N;
        const char* srcs[kMaxPeers];
        char* dsts[kMaxPeers];
        for (int s = 0; s < n; s++) {
            const int p = (r + s) % n;      // own copy first
            srcs[s] = io.send_peer[p] + first * sizeof(T);
            dsts[s] = rs ? reinterpret_cast<char*>(io.recv) + lo * sizeof(T) : io.recv_peer[red ? a.root : p] + first * sizeof(T);
        }
        const int ndst = rs || red ? 1 : n;
        if (n == 2) direct_pass<T, OP, 2>(srcs, dsts, n, ndst, nvec, avg);
        else if (n == 4) direct_pass<T, OP, 4>(srcs, dsts, n, ndst, nvec, avg);
        else if (n == 8) direct_pass<T, OP, 8>(srcs, dsts, n, ndst, nvec, avg);
        else direct_pass<T, OP, 0>(srcs, dsts, n, ndst, nvec, avg);
        for (size_t j = nvec * Vec16<T>::N + threadIdx.x; j < cnt; j += blockDim.x) {
            A acc = Traits<T>::up(reinterpret_cast<const T*>(srcs[0])[j]);
            for (int s = 1; s < n; s++) acc = op_apply<OP, A>(acc, Traits<T>::up(reinterpret_cast<const T*>(srcs[s])[j]));
            const T out = Traits<T>::down(avg ? avg_finish<A>(acc, n) : acc);
            for (int s = 0; s < ndst; s++) reinterpret_cast<T*>(dsts[s])[j] = out;
        }
    }
    rank_barrier(c, x.bid, x.seq, 1, 950);
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_direct(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    direct_body<T, OP>(a, x);
    finish_call(x);
}

/* ---------------- broadcast ---------------- */

constexpr int kDirectBcastMaxChunks = 24;      // chunk k is announced with flag index k + 1; 0 is the entry barrier
constexpr int kDirectBcastForwarded = 30;      // an owner has forwarded all of its shard
static_assert(kDirectBcastMaxChunks + 1 < kDirectBcastForwarded && kDirectBcastForwarded < kFlagVals, "chunk numbers and the closing flag share the per-call flag values");

/** Up to S copies of whole 16-byte vectors (source i -> destination i, len[i] bytes; the rest of a ragged end byte by
 *  byte), U vectors of each in flight per thread. Sources are local, destinations are peers' buffers. With `dual`
 *  every vector is also stored `local_delta` bytes away from where it was loaded (the root's own receive buffer). */
struct CopySet {
    const char* src[kMaxPeers];
    char* dst[kMaxPeers];
    size_t len[kMaxPeers];
};

template <int S, int U>
__device__ DCCL_NOINLINE void copy_set(const CopySet& p, int ns, bool dual, ptrdiff_t local_delta) {
    const size_t tid = threadIdx.x, nt = blockDim.x;
    const char* src[S];
    char* dst[S];
    size_t nv[S], maxv = 0;
#pragma unroll
    for (int s = 0; s < S; s++) {
        src[s] = p.src[s < ns ? s : 0];
        dst[s] = p.dst[s < ns ? s : 0];
        nv[s] = s < ns ? p.len[s] / 16 : 0;
        if (nv[s] > maxv) maxv = nv[s];
    }
    for (size_t i0 = tid; i0 < maxv; i0 += (size_t)U * nt) {
        uint4 v[S][U];
#pragma unroll
        for (int s = 0; s < S; s++) {
#pragma unroll
            for (int u = 0; u < U; u++) {
                const size_t i = i0 + (size_t)u * nt;
                if (i < nv[s]) v[s][u] = *reinterpret_cast<const uint4*>(src[s] + i * 16);
            }
        }
#pragma unroll
        for (int s = 0; s < S; s++) {
#pragma unroll
            for (int u = 0; u < U; u++) {
                const size_t i = i0 + (size_t)u * nt;
                if (i < nv[s]) {
                    *reinterpret_cast<uint4*>(dst[s] + i * 16) = v[s][u];
                    if (dual) *reinterpret_cast<uint4*>(const_cast<char*>(src[s]) + local_delta + i * 16) = v[s][u];
                }
            }
        }
    }
    // only the end of the message can be ragged
    for (int s = 0; s < ns; s++) {
        for (size_t j = p.len[s] / 16 * 16 + tid; j < p.len[s]; j += nt) {
            p.dst[s][j] = p.src[s][j];
            if (dual) const_cast<char*>(p.src[s])[local_delta + (ptrdiff_t)j] = p.src[s][j];
        }
    }
}

/** `len` bytes from a local source to the same offset of up to D peers' buffers: every vector is loaded once. */
template <int D>
__device__ DCCL_NOINLINE void fan_out(const char* src, char* const* dsts, int nd, size_t len) {
    constexpr int U = 4;
    const size_t tid = threadIdx.x, nt = blockDim.x, nv = len / 16;
    char* dst[D];
#pragma unroll
    for (int d = 0; d < D; d++) dst[d] = dsts[d < nd ? d : 0];
    for (size_t i0 = tid; i0 < nv; i0 += (size_t)U * nt) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const size_t i = i0 + (size_t)u * nt;
            if (i < nv) v[u] = *reinterpret_cast<const uint4*>(src + i * 16);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const size_t i = i0 + (size_t)u * nt;
            if (i >= nv) break;
#pragma unroll
            for (int d = 0; d < D; d++)
                if (d < nd) *reinterpret_cast<uint4*>(dst[d] + i * 16) = v[u];
        }
    }
    for (size_t j = nv * 16 + tid; j < len; j += nt)
        for (int d = 0; d < nd; d++) dsts[d][j] = src[j];
}

/**
 * a.count: BYTES; a.stride: chunks per shard; the root's io.send and every io.recv_peer[] 16-byte aligned.
 *
 * The CTAs form two teams (even and odd CTA numbers) that take the chunks in turn: before a root CTA may announce a
 * chunk its stores must have arrived, and while it waits for that the other team keeps the links busy.
 */
__device__ __forceinline__ void direct_bcast_body(const CollArgs& a, const Ctx& x) {
    const DevComm& c = *x.c;
    const RankIO& io = *x.io;
    const int n = c.nranks, r = c.rank, root = a.root, m = n - 1, C = (int)a.stride;
    const size_t bytes = a.count;
    __shared__ int s_fail;
    if (!DCCL_BOUNDS_OK(c, C >= 1 && C <= kDirectBcastMaxChunks && root >= 0 && root < n, 1911, C)) return;
    // everybody has entered: every receive buffer may be written
    if (!rank_barrier(c, x.bid, x.seq, 0, 910)) return;

    auto up16 = [](size_t v) { return (v + 15) / 16 * 16; };
    char* recv = reinterpret_cast<char*>(io.recv);
    const char* send = reinterpret_cast<const char*>(io.send);
    const int P = C >= 2 && x.nb >= 2 ? 2 : 1, team = x.bid % P, gi = x.bid / P, team_size = (x.nb - team + P - 1) / P;
    const size_t per = up16((bytes + m - 1) / m), chunk = up16((per + C - 1) / C), epb = up16((chunk + team_size - 1) / team_size);
    // this CTA's slice of chunk k of a shard, as a byte range of the message
    auto span = [&](int shard, int k, size_t* off, size_t* len) {
        const size_t slo = (size_t)shard * per, shi = slo + per < bytes ? slo + per : bytes;
        const size_t clo = slo + (size_t)k * chunk, chi = clo + chunk < shi ? clo + chunk : shi;
        const size_t lo = clo + epb * (size_t)gi, hi = lo + epb < chi ? lo + epb : chi;
        *off = lo;
        *len = hi > lo ? hi - lo : 0;
    };
    if (r == root) {
        for (int k = team; k < C; k += P) {
            // chunk k of every shard to its owner
            CopySet p;
            p.src[0] = nullptr; p.dst[0] = nullptr; p.len[0] = 0;
            int ns = 0;
            for (int o = 0; o < m; o++) {
                size_t off, len;
                span(o, k, &off, &len);
                if (len) { p.src[ns] = send + off; p.dst[ns] = io.recv_peer[(root + 1 + o) % n] + off; p.len[ns] = len; ns++; }
            }
            // out of place, the root's own copy rides along: each vector is loaded once and stored twice
            const bool dual = recv != send;
            const ptrdiff_t delta = recv - send;
            if (ns <= 1) copy_set<1, 8>(p, ns, dual, delta);
            else if (ns <= 3) copy_set<3, 4>(p, ns, dual, delta);
            else copy_set<kMaxPeers - 1, 2>(p, ns, dual, delta);
            __syncthreads();
            if ((int)threadIdx.x < n && (int)threadIdx.x != root) signal_peer(c, (int)threadIdx.x, x.bid, x.seq, k + 1);
        }
        return;
    }
    const int o = (r - root - 1 + n) % n;                       // my shard
    char* others[kMaxPeers];
    int nd = 0;
    for (int s = 1; s < m; s++) others[nd++] = io.recv_peer[(root + 1 + (o + s) % m) % n];
    for (int k = team; k < C; k += P) {
        if (!cta_wait_peer(c, root, x.bid, x.seq, k + 1, 920)) return;
        size_t off, len;
        span(o, k, &off, &len);
        if (len && nd) {
            char* dsts[kMaxPeers];
            for (int d = 0; d < nd; d++) dsts[d] = others[d] + off;
            if (nd <= 2) fan_out<2>(recv + off, dsts, nd, len);
            else fan_out<kMaxPeers - 2>(recv + off, dsts, nd, len);
        }
    }
    if (nd) {
        // my shard is everywhere; the message is complete here when every other owner says the same
        __syncthreads();
        if (threadIdx.x == 0) s_fail = 0;
        __syncthreads();
        if ((int)threadIdx.x < n && (int)threadIdx.x != r && (int)threadIdx.x != root) {
            signal_peer(c, (int)threadIdx.x, x.bid, x.seq, kDirectBcastForwarded);
            if (!wait_peer(c, (int)threadIdx.x, x.bid, x.seq, kDirectBcastForwarded, 930)) s_fail = 1;
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(512) k_direct_bcast(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    direct_bcast_body(a, x);
    finish_call(x);
}

int direct_bcast_chunks(size_t bytes, int nranks) {
    if (nranks <= 2) return 1;                          // nobody forwards anything: nothing to overlap
    const size_t per = bytes / (size_t)(nranks - 1);
    size_t k = per / (1u << 20);
    if (k < 2) k = per >= (128u << 10) ? 2 : 1;        // two chunks give both teams of CTAs work
    if (k > (size_t)kDirectBcastMaxChunks) k = kDirectBcastMaxChunks;
    return (int)k;
}

cudaError_t launch_direct_bcast(const CollArgs& a_in, size_t bytes, int nranks, const LaunchCfg& cfg, int chunks) {
    CollArgs a = a_in;
    a.count = bytes;
    a.stride = (size_t)(chunks >= 1 && chunks <= kDirectBcastMaxChunks ? chunks : direct_bcast_chunks(bytes, nranks));
    return launch_coll(k_direct_bcast, a, cfg);
}

cudaError_t launch_direct(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg) {
#define CALL(T, OP) return launch_coll(k_direct<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
