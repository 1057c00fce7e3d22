/**
 * Staging-based peer-to-peer collectives: all-reduce (reduce-scatter +
 * all-gather in one launch, the "two-shot" variant), reduce-scatter,
 * all-gather, broadcast (scatter + all-gather, or direct pull for small
 * messages) and reduce.
 *
 * Same data flow as the Rabenseifner idea of the original (reduce-scatter then
 * all-gather, reference src/core/all_reduce_recursive_halving_and_doubling.cpp)
 * but flattened for a switch where every peer is one hop away:
 *
 *   phase 0  every rank PUSHES shard j of its input straight from the user
 *            buffer into slot [rank] of rank j's staging area (remote stores)
 *   barrier
 *   phase 1  every rank reduces the n slots of its own shard (its own part comes
 *            straight from the user buffer), applies the 1/world scale of
 *            ncclAvg, and writes the result shard to staging (+ its own output)
 *   barrier
 *   phase 2  every rank PULLS the other result shards from the peers' staging
 *            straight into the user's receive buffer (remote loads)
 *
 * No byte is copied twice: user buffers need no registration and there is no
 * copy-in / copy-out pass. CTA b of every rank works on the same sub-range of
 * every shard, so the barriers only pair CTA b with CTA b of the peers.
 * Staging alternates between two halves from call to call, which is what
 * makes a trailing barrier unnecessary (a rank can only be two calls ahead of
 * a peer after that peer has left the older call).
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"
#include "../device/geometry.cuh"

namespace dccl {

template <typename T, int OP>
__device__ __forceinline__ void twoshot_body(const CollArgs& a, const Ctx& x) {
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank, mode = a.mode;
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    Geometry<T> g(mode == TS_REDUCESCATTER || mode == TS_ALLGATHER ? GEO_SLOTS : mode == TS_BROADCAST_DIRECT ? GEO_WHOLE : GEO_SPLIT,
                  a.count, n, x.bid, x.nb);
    if (mode == TS_ALLREDUCE || mode == TS_REDUCESCATTER || mode == TS_REDUCE) g.res_off = g.slot_stride * (size_t)n;
    const size_t stride = (mode == TS_REDUCESCATTER || mode == TS_ALLGATHER) ? a.stride : g.per;
    if (!stage_extent_ok<T>(c, g.res_off + g.slot_stride, 1900)) return;   // n receive slots and the result area
    T* my_stage = stage_ptr<T>(c, r, x.parity);
    const bool avg = a.op == (int)ncclAvg;
    auto lo_of = [&](int j) { size_t l = g.len(j); return g.blo < l ? g.blo : l; };
    auto hi_of = [&](int j) { size_t l = g.len(j); return g.bhi < l ? g.bhi : l; };

    /* ---- large reduce-scatter: push and reduce overlap ---- */
    // The CTA's range is cut into K pieces. Piece k+1 is pushed to the peers (posted remote stores) before
    // piece k, which every peer has signalled by then, is folded from staging: the NVLink writes of one
    // piece are in flight while the HBM reads of the previous one run. All ranks derive the same K.
    if (mode == TS_REDUCESCATTER) {
        constexpr size_t VE = Geometry<T>::VE;
        const size_t lo0 = lo_of(0), hi0 = hi_of(0);          // all shards have the same length here
        const size_t span = g.bhi - g.blo;                     // derived from geometry only: equal on all ranks
        int K = (int)(span * sizeof(T) / (256u << 10));
        if (K > 12) K = 12;
        if (K >= 2) {
            const size_t piece = ((span + K - 1) / K + VE - 1) / VE * VE;
            auto piece_lo = [&](int k) { size_t v = g.blo + piece * (size_t)k; return v < hi0 ? (v > lo0 ? v : lo0) : hi0; };
            auto push = [&](int k) {
                const size_t lo = piece_lo(k), hi = piece_lo(k + 1);
                if (hi > lo)
                    for (int q = 1; q < n; q++) {
                        const int p = (r + q) % n;
                        copy_range<T>(stage_ptr<T>(c, p, x.parity) + (size_t)r * g.slot_stride + lo, send + (size_t)p * stride + lo, hi - lo);
                    }
                __syncthreads();
                if ((int)threadIdx.x < n) signal_peer(c, (int)threadIdx.x, x.bid, x.seq, k);
            };
            auto fold = [&](int k) -> bool {
                __shared__ int s_fail;
                if (threadIdx.x == 0) s_fail = 0;
                __syncthreads();
                if ((int)threadIdx.x < n && !wait_peer(c, (int)threadIdx.x, x.bid, x.seq, k, 150)) s_fail = 1;
                __syncthreads();
                if (s_fail) return false;
                const size_t lo = piece_lo(k), hi = piece_lo(k + 1);
                if (hi > lo) {
                    const T* ins[kMaxPeers];
                    int cnt = 0;
                    for (int p = 0; p < n; p++) if (p != r) ins[cnt++] = my_stage + (size_t)p * g.slot_stride + lo;
                    reduce_range<T, OP>(recv + lo, nullptr, send + (size_t)r * stride + lo, ins, cnt, hi - lo, avg, n);
                }
                return true;
            };
            push(0);
            for (int k = 1; k < K; k++) {
                push(k);
                if (!fold(k - 1)) return;
            }
            fold(K - 1);
            return;
        }
    }

    /* ---- phase 0 ---- */
    if (mode == TS_ALLREDUCE || mode == TS_REDUCESCATTER || mode == TS_REDUCE) {
        for (int k = 1; k < n; k++) {
            const int p = (r + k) % n;
            const size_t lo = lo_of(p), hi = hi_of(p);
            if (hi > lo) copy_range<T>(stage_ptr<T>(c, p, x.parity) + (size_t)r * g.slot_stride + lo, send + (size_t)p * stride + lo, hi - lo);
        }
    } else if (mode == TS_ALLGATHER) {
        const size_t lo = lo_of(0), hi = hi_of(0);   // every shard has the same length here
        if (hi > lo) copy_range<T>(my_stage + g.res_off + lo, send + lo, hi - lo);
    } else if (mode == TS_BROADCAST) {
        if (r == a.root) {
            for (int k = 0; k < n; k++) {
                const int p = (r + k) % n;
                const size_t lo = lo_of(p), hi = hi_of(p);
                if (hi > lo) copy_range<T>(stage_ptr<T>(c, p, x.parity) + g.res_off + lo, send + (size_t)p * stride + lo, hi - lo);
            }
        }
    } else {  // TS_BROADCAST_DIRECT
        if (r == a.root) {
            const size_t lo = lo_of(0), hi = hi_of(0);
            if (hi > lo) copy_range<T>(my_stage + lo, send + lo, hi - lo);
        }
    }
    if (!rank_barrier(c, x.bid, x.seq, 0, 100 + mode)) return;

    /* ---- phase 1: reduce my shard ---- */
    if (mode == TS_ALLREDUCE || mode == TS_REDUCESCATTER || mode == TS_REDUCE) {
        const size_t lo = lo_of(r), hi = hi_of(r);
        if (hi > lo) {
            const T* ins[kMaxPeers];
            int k = 0;
            for (int p = 0; p < n; p++) if (p != r) ins[k++] = my_stage + (size_t)p * g.slot_stride + lo;
            const T* own = send + (size_t)r * stride + lo;
            T *out0, *out1 = nullptr;
            if (mode == TS_REDUCESCATTER) out0 = recv + lo;
            else {
                out0 = my_stage + g.res_off + lo;
                if (mode == TS_ALLREDUCE || r == a.root) out1 = recv + (size_t)r * stride + lo;
            }
            reduce_range<T, OP>(out0, out1, own, ins, k, hi - lo, avg, n);
        }
        if (mode == TS_REDUCESCATTER) return;
        if (!rank_barrier(c, x.bid, x.seq, 1, 200 + mode)) return;
    }

    /* ---- phase 2: collect ---- */
    if (mode == TS_ALLREDUCE || mode == TS_ALLGATHER || (mode == TS_REDUCE && r == a.root) || (mode == TS_BROADCAST && r != a.root)) {
        for (int k = 1; k < n; k++) {
            const int p = (r + k) % n;
            const size_t lo = lo_of(p), hi = hi_of(p);
            if (hi > lo) copy_range<T>(recv + (size_t)p * stride + lo, stage_ptr<T>(c, p, x.parity) + g.res_off + lo, hi - lo);
        }
        const size_t lo = lo_of(r), hi = hi_of(r);
        if (mode == TS_ALLGATHER) {
            if (recv + (size_t)r * stride != send && hi > lo) copy_range<T>(recv + (size_t)r * stride + lo, send + lo, hi - lo);
        } else if (mode == TS_BROADCAST) {
            if (hi > lo) copy_range<T>(recv + (size_t)r * stride + lo, my_stage + g.res_off + lo, hi - lo);
        }
    } else if (mode == TS_BROADCAST && r == a.root) {
        if (recv != send)
            for (int p = 0; p < n; p++) {
                const size_t lo = lo_of(p), hi = hi_of(p);
                if (hi > lo) copy_range<T>(recv + (size_t)p * stride + lo, send + (size_t)p * stride + lo, hi - lo);
            }
    } else if (mode == TS_BROADCAST_DIRECT) {
        const size_t lo = lo_of(0), hi = hi_of(0);
        if (hi > lo) {
            if (r != a.root) copy_range<T>(recv + lo, stage_ptr<T>(c, a.root, x.parity) + lo, hi - lo);
            else if (recv != send) copy_range<T>(recv + lo, send + lo, hi - lo);
        }
    }
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_twoshot(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    twoshot_body<T, OP>(a, x);
    finish_call(x);
}

size_t twoshot_capacity(int mode, int nranks, size_t es, size_t stage_bytes) {
    const size_t ve = 16 / es, stage_elems = stage_bytes / es, n = (size_t)nranks;
    auto floor_ve = [&](size_t x) { return x / ve * ve; };
    switch (mode) {
    case TS_ALLREDUCE: case TS_REDUCE: return n * floor_ve(stage_elems / (n + 1));
    case TS_REDUCESCATTER: return floor_ve(stage_elems / (n + 1));
    case TS_ALLGATHER: return floor_ve(stage_elems);
    case TS_BROADCAST: return n * floor_ve(stage_elems);
    default: return floor_ve(stage_elems);
    }
}

cudaError_t launch_twoshot(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg) {
    if (a.mode == TS_ALLGATHER || a.mode == TS_BROADCAST || a.mode == TS_BROADCAST_DIRECT) {
        // pure data movement: run on bytes
        CollArgs b = a;
        const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                          : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
        b.count = a.count * es;
        b.stride = a.stride * es;
        return launch_coll(k_twoshot<uint8_t, OP_SUM>, b, cfg);
    }
#define CALL(T, OP) return launch_coll(k_twoshot<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
