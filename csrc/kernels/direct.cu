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
 */
#include "kernels.hpp"
#include "../device/geometry.cuh"
#include "../device/reduce_ops.cuh"

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
    const bool rs = a.mode == DIRECT_REDUCESCATTER;
    // all-reduce: this rank folds shard r of one vector; reduce-scatter: slot r (count elements) of every send buffer
    const Geometry<T> g(rs ? GEO_WHOLE : GEO_SPLIT, a.count, rs ? 1 : n, x.bid, x.nb);

    if (!rank_barrier(c, x.bid, x.seq, 0, 900)) return;

    const size_t len = rs ? a.count : g.len(r);
    const size_t lo = g.blo < len ? g.blo : len, hi = g.bhi < len ? g.bhi : len;
    if (hi > lo) {
        // shard and CTA boundaries are multiples of one vector; only the very end of the message can be ragged
        const size_t first = (rs ? (size_t)r * a.stride : (size_t)r * g.per) + lo, cnt = hi - lo;
        const size_t nvec = cnt / Vec16<T>::N;
        const char* srcs[kMaxPeers];
        char* dsts[kMaxPeers];
        for (int s = 0; s < n; s++) {
            const int p = (r + s) % n;      // own copy first
            srcs[s] = io.send_peer[p] + first * sizeof(T);
            dsts[s] = rs ? reinterpret_cast<char*>(io.recv) + lo * sizeof(T) : io.recv_peer[p] + first * sizeof(T);
        }
        const int ndst = rs ? 1 : n;
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

cudaError_t launch_direct(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg) {
#define CALL(T, OP) return launch_coll(k_direct<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
