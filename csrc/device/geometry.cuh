/**
 * How a message is cut into per-rank shards and per-CTA ranges. Shared by the
 * staging-based kernels so that CTA b of every rank always covers the same
 * sub-range of every shard (which is what lets barriers pair CTA b with CTA b).
 * Shard boundaries and CTA ranges are multiples of a 16-byte vector; the last
 * shard / last CTA take the remainder, so any element count is accepted (the
 * original needed count % world == 0, reference src/core/all_reduce_ring.cpp:51-55).
 */
#pragma once
#include "prims.cuh"

namespace dccl {

enum { GEO_SPLIT = 0,    // one vector of `count` elements cut into n shards (all-reduce, broadcast, reduce)
       GEO_SLOTS = 1,    // n slots of `count` elements each (reduce-scatter, all-gather)
       GEO_WHOLE = 2 };  // one shard holding everything

template <typename T> struct Geometry {
    static constexpr size_t VE = 16 / sizeof(T);
    size_t per, total, slot_stride, res_off, blo, bhi;
    int shards;
    __host__ __device__ static size_t roundup(size_t x, size_t m) { return (x + m - 1) / m * m; }
    __device__ Geometry(int kind, size_t count, int n, int bid, int nb) {
        if (kind == GEO_SLOTS) { per = count; total = count * (size_t)n; shards = n; }
        else if (kind == GEO_WHOLE) { per = count; total = count; shards = 1; }
        else { per = roundup((count + n - 1) / n, VE); total = count; shards = n; }
        slot_stride = roundup(per, VE);
        res_off = 0;
        size_t epb = roundup((per + nb - 1) / nb, VE);
        blo = epb * (size_t)bid; if (blo > per) blo = per;
        bhi = blo + epb; if (bhi > per) bhi = per;
    }
    __device__ size_t len(int j) const { size_t o = per * (size_t)j; return o >= total ? 0 : (total - o < per ? total - o : per); }
};

template <typename T>
__device__ __forceinline__ T* stage_ptr(const DevComm& c, int p, int parity) {
    return reinterpret_cast<T*>(c.pool[p] + kStageOff + (size_t)parity * c.stage_bytes);
}

/** Debug build (DCCL_DEBUG_BOUNDS): the kernel is about to use the first `elems` elements of a staging half.
 *  The recorded value is the extent in KB. Always true in the normal build. */
template <typename T>
__device__ __forceinline__ bool stage_extent_ok(const DevComm& c, size_t elems, int site) {
    return DCCL_BOUNDS_OK(c, elems * sizeof(T) <= c.stage_bytes, site, (elems * sizeof(T)) >> 10);
}

} // namespace dccl
