/**
 * Ring reduce-scatter, all-gather and all-reduce as ONE persistent kernel each.
 *
 * Same schedule as the original (reference src/core/reduce_scatter_ring.cpp:71-101,
 * all_gather_ring.cpp:44-52, all_reduce_ring.cpp:59-75): n-1 reduce steps in
 * which slot (r - s) travels to rank r+1, then n-1 gather steps. What changes:
 * no host is involved after the launch. A step is "wait for the previous
 * rank's flag, fold the incoming partial with my own input, and write the new
 * partial STRAIGHT INTO the next rank's staging area" - the reduction and the
 * transfer are the same loop, and the last reduce step also seeds the gather.
 * The input buffer is never modified, so reduce-scatter needs no work copy
 * (the original makes one per call, reference src/core/dccl.cpp:576-609).
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"
#include "../device/geometry.cuh"

namespace dccl {

template <typename T, int OP>
__device__ __forceinline__ void ring_body(const CollArgs& a, const Ctx& x) {
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank, mode = a.mode;
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    const bool slots = mode != RING_ALLREDUCE;
    const Geometry<T> g(slots ? GEO_SLOTS : GEO_SPLIT, a.count, n, x.bid, x.nb);
    const size_t stride = slots ? a.stride : g.per;
    const int next = (r + 1) % n, prev = (r + n - 1) % n;
    const bool avg = a.op == (int)ncclAvg;
    if (!stage_extent_ok<T>(c, (size_t)(2 * n - 1) * g.slot_stride, 1901)) return;   // areas 0 .. 2n-2
    T* my_stage = stage_ptr<T>(c, r, x.parity);
    T* next_stage = stage_ptr<T>(c, next, x.parity);
    auto lo_of = [&](int j) { size_t l = g.len(j); return g.blo < l ? g.blo : l; };
    auto hi_of = [&](int j) { size_t l = g.len(j); return g.bhi < l ? g.bhi : l; };
    auto md = [&](int v) { int m = v % n; return m < 0 ? m + n : m; };
    auto area = [&](T* stage, int k) { return stage + (size_t)k * g.slot_stride; };

    int own = r;   // shard this rank holds complete before the gather phase
    if (mode == RING_ALLREDUCE || mode == RING_REDUCESCATTER) {
        // rank r must end with shard r for reduce-scatter (shift -1), with shard r+1 for all-reduce
        const int sh = mode == RING_REDUCESCATTER ? -1 : 0;
        own = md(r + 1 + sh);
        {   // step 0: my own input of shard (r + sh) goes to the next rank
            const int j = md(r + sh);
            const size_t lo = lo_of(j), hi = hi_of(j);
            if (hi > lo) copy_range<T>(area(next_stage, 0) + lo, send + (size_t)j * stride + lo, hi - lo);
            cta_signal_peer(c, next, x.bid, x.seq, 0);
        }
        for (int s = 0; s < n - 1; s++) {
            if (!cta_wait_peer(c, prev, x.bid, x.seq, s, 600 + s)) return;
            const int j = md(r - s - 1 + sh);
            const size_t lo = lo_of(j), hi = hi_of(j);
            const bool last = s == n - 2;
            if (hi > lo) {
                const T* ins[1] = {area(my_stage, s) + lo};
                const T* mine = send + (size_t)j * stride + lo;
                if (!last) reduce_range<T, OP>(area(next_stage, s + 1) + lo, nullptr, mine, ins, 1, hi - lo, false, n);
                else if (mode == RING_REDUCESCATTER) reduce_range<T, OP>(recv + lo, nullptr, mine, ins, 1, hi - lo, avg, n);
                else reduce_range<T, OP>(recv + (size_t)j * stride + lo, area(next_stage, n - 1) + lo, mine, ins, 1, hi - lo, avg, n);
            }
            if (!last) cta_signal_peer(c, next, x.bid, x.seq, s + 1);
            else if (mode == RING_ALLREDUCE) cta_signal_peer(c, next, x.bid, x.seq, n - 1);
        }
        if (mode == RING_REDUCESCATTER) return;
    } else {
        // all-gather: seed the ring with my slot
        const size_t lo = lo_of(r), hi = hi_of(r);
        if (hi > lo) {
            copy_range<T>(area(next_stage, n - 1) + lo, send + lo, hi - lo);
            if (recv + (size_t)r * stride != send) copy_range<T>(recv + (size_t)r * stride + lo, send + lo, hi - lo);
        }
        cta_signal_peer(c, next, x.bid, x.seq, n - 1);
    }

    /* gather: at step t shard (own - t - 1) arrives; keep it and pass it on */
    for (int t = 0; t < n - 1; t++) {
        if (!cta_wait_peer(c, prev, x.bid, x.seq, n - 1 + t, 650 + t)) return;
        const int j = md(own - t - 1);
        const size_t lo = lo_of(j), hi = hi_of(j);
        if (hi > lo) {
            const T* src = area(my_stage, n - 1 + t) + lo;
            if (t < n - 2) copy_range<T>(area(next_stage, n + t) + lo, src, hi - lo);
            copy_range<T>(recv + (size_t)j * stride + lo, src, hi - lo);
        }
        if (t < n - 2) cta_signal_peer(c, next, x.bid, x.seq, n + t);
    }
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_ring(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    ring_body<T, OP>(a, x);
    finish_call(x);
}

size_t ring_capacity(int mode, int nranks, size_t es, size_t stage_bytes) {
    const size_t ve = 16 / es, stage_elems = stage_bytes / es, n = (size_t)nranks;
    const size_t areas = 2 * n;   // n-1 reduce areas + n-1 gather areas, rounded up
    auto floor_ve = [&](size_t v) { return v / ve * ve; };
    if (mode == RING_ALLREDUCE) return n * floor_ve(stage_elems / areas);
    return floor_ve(stage_elems / areas);   // per-rank count
}

cudaError_t launch_ring(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg) {
    if (a.mode == RING_ALLGATHER) {
        const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                          : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
        CollArgs b = a;
        b.count = a.count * es;
        b.stride = a.stride * es;
        b.op = (int)ncclSum;
        return launch_coll(k_ring<uint8_t, OP_SUM>, b, cfg);
    }
#define CALL(T, OP) return launch_coll(k_ring<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
