/**
 * Pipelined switch (NVLS) all-reduce for ORDINARY device buffers.
 *
 * The staged switch variant (nvls.cu) copies the input into the multicast-bound
 * staging area, runs the in-switch reduction, and copies the result out, one
 * phase after the other; for large messages the two local copies cost about a
 * third of the time. Here the message is cut into chunks and three groups of
 * CTAs work as an assembly line in ONE launch:
 *
 *   IN   copies chunk k of the user's send buffer into staging        (local HBM)
 *   NV   multimem.ld_reduce's its shard of chunk k from all ranks,
 *        applies the 1/world scale, multimem.st's it to all ranks     (NVLink / switch)
 *   OUT  copies chunk k from staging into the user's receive buffer   (local HBM)
 *
 * so that the copies of chunks k+1 and k-1 run while the switch works on chunk
 * k. CTA triple g (IN_g, NV_g, OUT_g) owns sub-range g of every shard of every
 * chunk on every rank; IN_g of all ranks signal NV_g of all ranks ("chunk k is
 * staged everywhere"), NV_g of all ranks signal OUT_g of all ranks ("chunk k is
 * reduced everywhere"). The flags are the usual peer flag words, one row per
 * (triple, stage). The whole message sits in one staging half, so no staging
 * byte is reused within a launch and the hand-over needs no back pressure.
 */
#include "kernels.hpp"
#include "../device/geometry.cuh"
#include "../device/multimem.cuh"

namespace dccl {

constexpr int kPipeMaxChunks = 24;    // flag values per call are limited (kFlagVals)
static_assert(kPipeMaxChunks < kFlagVals, "chunk numbers must fit the per-call flag values");

/** wait until the same-index CTA of EVERY rank has signalled point idx on flag row `row` */
__device__ __forceinline__ bool wait_all_ranks(const DevComm& c, int row, uint32_t seq, int idx, int site) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    if ((int)threadIdx.x < c.nranks)
        if (!wait_peer(c, (int)threadIdx.x, row, seq, idx, site)) s_fail = 1;
    __syncthreads();
    const bool ok = s_fail == 0;
    __syncthreads();
    return ok;
}

/** all writes of this CTA are done -> tell flag row `row` of every rank */
__device__ __forceinline__ void signal_all_ranks(const DevComm& c, int row, uint32_t seq, int idx) {
    __syncthreads();
    if ((int)threadIdx.x < c.nranks) signal_peer(c, (int)threadIdx.x, row, seq, idx);
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_nvls_pipe(const __grid_constant__ CollArgs a) {
    constexpr size_t ES = sizeof(T);
    constexpr size_t VE = 16 / ES;
    const Ctx x = make_ctx(a);
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank;
    const int G = x.nb / 3;                       // CTA triples per rank
    const int role = x.bid / G, g = x.bid - role * G;
    if (role > 2) return;                          // left-over CTAs when the grid is not a multiple of 3
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    const bool avg = a.op == (int)ncclAvg;
    const size_t stage_off = kStageOff + (size_t)a.parity * c.stage_bytes;
    T* my_stage = reinterpret_cast<T*>(c.pool[r] + stage_off);
    char* mc_stage = c.mc_pool + stage_off;

    // chunks: equal pieces, each a multiple of n vectors so that every chunk splits into aligned shards
    const int nchunks = a.mode;                    // chosen by the host, 1..kPipeMaxChunks
    size_t chunk = (a.count + nchunks - 1) / nchunks;
    chunk = (chunk + VE * n - 1) / (VE * n) * (VE * n);
    const int row_a = 2 * g, row_b = 2 * g + 1;

    for (int k = 0; k < nchunks; k++) {
        const size_t base = (size_t)k * chunk;
        if (base >= a.count) {
            // nothing left: still keep the hand-over counts in step
            if (role == 0) signal_all_ranks(c, row_a, a.seq, k);
            else if (role == 1) { if (!wait_all_ranks(c, row_a, a.seq, k, 560)) return; signal_all_ranks(c, row_b, a.seq, k); }
            else if (!wait_all_ranks(c, row_b, a.seq, k, 570)) return;
            continue;
        }
        const size_t cnt = a.count - base < chunk ? a.count - base : chunk;
        const Geometry<T> geo(GEO_SPLIT, cnt, n, g, G);
        auto lo_of = [&](int j) { size_t l = geo.len(j); return geo.blo < l ? geo.blo : l; };
        auto hi_of = [&](int j) { size_t l = geo.len(j); return geo.bhi < l ? geo.bhi : l; };
        // chunk k lives at the same element offsets in staging as in the user buffers; shard j of the chunk
        // starts at base + j * geo.per (geo.per is a multiple of a vector, base a multiple of n vectors)
        if (role == 0) {
            for (int j = 0; j < n; j++) {
                const size_t lo = lo_of(j), hi = hi_of(j), off = base + (size_t)j * geo.per + lo;
                if (hi > lo) copy_range<T>(my_stage + off, send + off, hi - lo);
            }
            signal_all_ranks(c, row_a, a.seq, k);
        } else if (role == 1) {
            if (!wait_all_ranks(c, row_a, a.seq, k, 560)) return;
            const size_t lo = lo_of(r), hi = hi_of(r);
            if (hi > lo) {
                const size_t off = (base + (size_t)r * geo.per + lo) * ES;
                nvls_pass<T, OP>(mc_stage + off, mc_stage + off, nullptr, ((hi - lo) * ES + 15) / 16, 0, avg, n, a.unroll);
            }
            signal_all_ranks(c, row_b, a.seq, k);
        } else {
            if (!wait_all_ranks(c, row_b, a.seq, k, 570)) return;
            for (int j = 0; j < n; j++) {
                const size_t lo = lo_of(j), hi = hi_of(j), off = base + (size_t)j * geo.per + lo;
                if (hi > lo) copy_range<T>(recv + off, my_stage + off, hi - lo);
            }
        }
    }
}

size_t nvls_pipe_capacity(size_t es, size_t stage_bytes) {
    // the whole message (plus rounding of the last vector) sits in one staging half
    return (stage_bytes / es / 64) * 64 - 64;
}

int nvls_pipe_chunks(size_t bytes) {
    size_t k = (bytes + (8u << 20) - 1) / (8u << 20);
    if (k < 2) k = 2;
    if (k > (size_t)kPipeMaxChunks) k = kPipeMaxChunks;
    return (int)k;
}

cudaError_t launch_nvls_pipe(const CollArgs& a_in, ncclDataType_t dt, const LaunchCfg& cfg_in) {
    CollArgs a = a_in;
    LaunchCfg cfg = cfg_in;
    cfg.ctas = cfg.ctas / 3 * 3;                  // whole triples
    if (cfg.ctas < 3) cfg.ctas = 3;
    const size_t es = dt == ncclFloat64 || dt == ncclInt64 || dt == ncclUint64 ? 8 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2 : 4;
    a.mode = nvls_pipe_chunks(a.count * es);
    const int op = a.op == (int)ncclAvg ? (int)ncclSum : a.op;
    switch (dt) {
#define PIPE_CASE(DT, T)                                                                    \
    case DT:                                                                                \
        if (op == (int)ncclSum) return launch_coll(k_nvls_pipe<T, OP_SUM>, a, cfg);         \
        if (op == (int)ncclMax) return launch_coll(k_nvls_pipe<T, OP_MAX>, a, cfg);         \
        if (op == (int)ncclMin) return launch_coll(k_nvls_pipe<T, OP_MIN>, a, cfg);         \
        break;
#define PIPE_CASE_SUM(DT, T)                                                                \
    case DT:                                                                                \
        if (op == (int)ncclSum) return launch_coll(k_nvls_pipe<T, OP_SUM>, a, cfg);         \
        break;
    PIPE_CASE_SUM(ncclFloat32, float)
    PIPE_CASE_SUM(ncclFloat64, double)
    PIPE_CASE(ncclFloat16, __half)
    PIPE_CASE(ncclBfloat16, __nv_bfloat16)
    PIPE_CASE(ncclInt32, int32_t)
    PIPE_CASE(ncclUint32, uint32_t)
    PIPE_CASE(ncclInt64, long long)
    PIPE_CASE(ncclUint64, unsigned long long)
#undef PIPE_CASE
#undef PIPE_CASE_SUM
    default: break;
    }
    return cudaErrorInvalidValue;
}

} // namespace dccl
