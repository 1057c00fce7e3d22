/**
 * Pipelined switch (NVLS) all-reduce and reduce-scatter for ORDINARY device buffers.
 *
 * The staged switch variant (nvls.cu) copies the input into the multicast-bound
 * staging area, runs the in-switch reduction, and copies the result out, one
 * phase after the other; for large messages the local copies cost about a third
 * of the time. Here the message is cut into chunks and three groups of CTAs
 * work as an assembly line in ONE launch:
 *
 *   IN   copies chunk k of the user's send buffer into staging         (local HBM)
 *   NV   multimem.ld_reduce's its shard of chunk k from all ranks, applies the
 *        1/world scale, and multimem.st's it to all ranks (all-reduce) or stores
 *        it straight into the receive buffer (reduce-scatter)          (NVLink / switch)
 *   OUT  copies chunk k from staging into the user's receive buffer    (local HBM;
 *        all-reduce only)
 *
 * so that the copies of chunks k+1 and k-1 run while the switch works on chunk
 * k. Every NV CTA g is fed by kPipeFan IN CTAs and drained by kPipeFan OUT CTAs
 * that split its sub-range (equal thirds, kPipeFan = 1, measured best on 8 x B200).
 * Hand-over: IN CTA (g,m) of every rank signals flag row g*fan+m of every rank;
 * NV_g waits for all fan x n of
 * them, then signals row B_g of every rank, which the OUT CTAs (g, *) wait on.
 * The whole message sits in one staging half, so no staging byte is reused
 * within a launch and the hand-over needs no back pressure.
 */
#include "kernels.hpp"
#include "../device/geometry.cuh"
#include "../device/multimem.cuh"

namespace dccl {

constexpr int kPipeMaxChunks = 24;    // flag values per call are limited (kFlagVals)
constexpr int kPipeFan = 1;           // copy CTAs per switch CTA, on each side (measured on 8 x B200: 1 beats 4)
static_assert(kPipeMaxChunks < kFlagVals, "chunk numbers must fit the per-call flag values");

/** wait until point idx was signalled on flag rows [row0, row0 + rows) by EVERY rank */
__device__ __forceinline__ bool wait_rows_all_ranks(const DevComm& c, int row0, int rows, uint32_t seq, int idx, int site) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    const int t = (int)threadIdx.x;
    if (t < c.nranks * rows)
        if (!wait_peer(c, t % c.nranks, row0 + t / c.nranks, seq, idx, site)) s_fail = 1;
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

/** sub-range [lo,hi) of [0,len) for part m of `parts`, in whole vectors of VE elements */
__device__ __forceinline__ void split_range(size_t lo, size_t hi, int m, int parts, size_t ve, size_t* plo, size_t* phi) {
    const size_t len = hi - lo;
    size_t per = ((len + parts - 1) / parts + ve - 1) / ve * ve;
    size_t a = lo + per * (size_t)m, b = a + per;
    if (a > hi) a = hi;
    if (b > hi) b = hi;
    *plo = a; *phi = b;
}

template <typename T, int OP>
__device__ __forceinline__ void nvls_pipe_body(const CollArgs& a, const Ctx& x) {
    constexpr size_t ES = sizeof(T);
    constexpr size_t VE = 16 / ES;
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank;
    const bool rs = a.root != 0;                   // reduce-scatter (count = per-rank elements) instead of all-reduce
    const int nroles = rs ? 1 + kPipeFan : 1 + 2 * kPipeFan;
    const int G = x.nb / nroles;                   // switch CTAs per rank
    // CTA order: [IN (G*fan)] [NV (G)] [OUT (G*fan)]
    int role, g, m = 0;
    if (x.bid < G * kPipeFan) { role = 0; g = x.bid / kPipeFan; m = x.bid % kPipeFan; }
    else if (x.bid < G * kPipeFan + G) { role = 1; g = x.bid - G * kPipeFan; }
    else if (!rs && x.bid < G * (1 + 2 * kPipeFan)) { role = 2; const int o = x.bid - G * (kPipeFan + 1); g = o / kPipeFan; m = o % kPipeFan; }
    else return;                                   // left-over CTAs
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    const bool avg = a.op == (int)ncclAvg;
    const size_t stage_off = kStageOff + (size_t)x.parity * c.stage_bytes;
    T* my_stage = reinterpret_cast<T*>(c.pool[r] + stage_off);
    char* mc_stage = c.mc_pool + stage_off;
    const int nchunks = a.mode;                    // chosen by the host, 1..kPipeMaxChunks
    const int row_a0 = g * kPipeFan;               // rows [row_a0, row_a0 + fan): IN (g, m) -> NV g
    const int row_b = G * kPipeFan + g;            // NV g -> OUT (g, *)
    // reduce-scatter: rank j's slot sits at j * stride in the user buffer and at j * slot in staging
    const size_t slot = (a.count + VE - 1) / VE * VE;
    size_t chunk = (a.count + nchunks - 1) / nchunks;
    chunk = rs ? (chunk + VE - 1) / VE * VE : (chunk + VE * n - 1) / (VE * n) * (VE * n);
    // the whole message sits in one staging half; chunk numbers are flag values; rows: fan per switch CTA, then one each
    if (!stage_extent_ok<T>(c, rs ? (size_t)n * slot : slot, 1908) ||
        !DCCL_BOUNDS_OK(c, nchunks >= 1 && nchunks <= kFlagVals && G * (kPipeFan + 1) <= kMaxCtas, 1908, nchunks)) return;

    for (int k = 0; k < nchunks; k++) {
        const size_t base = (size_t)k * chunk;
        const size_t cnt = base >= a.count ? 0 : (a.count - base < chunk ? a.count - base : chunk);
        // geometry of this chunk: all-reduce splits it into n shards; reduce-scatter has the same chunk in every slot
        const Geometry<T> geo(rs ? GEO_WHOLE : GEO_SPLIT, cnt, rs ? 1 : n, g, G);
        auto lo_of = [&](int j) { size_t l = rs ? cnt : geo.len(j); return geo.blo < l ? geo.blo : l; };
        auto hi_of = [&](int j) { size_t l = rs ? cnt : geo.len(j); return geo.bhi < l ? geo.bhi : l; };
        if (role == 0) {
            for (int j = 0; j < n && cnt; j++) {
                size_t lo, hi;
                split_range(lo_of(j), hi_of(j), m, kPipeFan, VE, &lo, &hi);
                if (hi <= lo) continue;
                if (rs) copy_range<T>(my_stage + (size_t)j * slot + base + lo, send + (size_t)j * a.stride + base + lo, hi - lo);
                else { const size_t off = base + (size_t)j * geo.per + lo; copy_range<T>(my_stage + off, send + off, hi - lo); }
            }
            signal_all_ranks(c, row_a0 + m, x.seq, k);
        } else if (role == 1) {
            if (!wait_rows_all_ranks(c, row_a0, kPipeFan, x.seq, k, 560)) return;
            const size_t lo = lo_of(r), hi = hi_of(r);
            if (hi > lo) {
                if (rs) {
                    const size_t off = ((size_t)r * slot + base + lo) * ES;
                    nvls_pass<T, OP>(mc_stage + off, nullptr, reinterpret_cast<char*>(recv + base + lo), ((hi - lo) * ES + 15) / 16, (hi - lo) * ES, avg, n, a.unroll);
                } else {
                    const size_t off = (base + (size_t)r * geo.per + lo) * ES;
                    nvls_pass<T, OP>(mc_stage + off, mc_stage + off, nullptr, ((hi - lo) * ES + 15) / 16, 0, avg, n, a.unroll);
                }
            }
            if (!rs) signal_all_ranks(c, row_b, x.seq, k);
        } else {
            if (!wait_rows_all_ranks(c, row_b, 1, x.seq, k, 570)) return;
            for (int j = 0; j < n && cnt; j++) {
                size_t lo, hi;
                split_range(lo_of(j), hi_of(j), m, kPipeFan, VE, &lo, &hi);
                if (hi <= lo) continue;
                const size_t off = base + (size_t)j * geo.per + lo;
                copy_range<T>(recv + off, my_stage + off, hi - lo);
            }
        }
    }
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_nvls_pipe(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    nvls_pipe_body<T, OP>(a, x);
    finish_call(x);
}

size_t nvls_pipe_capacity(size_t es, size_t stage_bytes, int nranks, bool reduce_scatter) {
    // the whole message (plus rounding of the last vector) sits in one staging half
    const size_t elems = (stage_bytes / es / 64) * 64 - 64;
    return reduce_scatter ? (elems / (size_t)nranks / 64) * 64 : elems;
}

static size_t g_pipe_chunk_bytes = 8u << 20;   // target chunk size; every rank must use the same value

void nvls_pipe_set_chunk_bytes(size_t bytes) { if (bytes >= (256u << 10)) g_pipe_chunk_bytes = bytes; }

int nvls_pipe_chunks(size_t bytes) {
    size_t k = (bytes + g_pipe_chunk_bytes - 1) / g_pipe_chunk_bytes;
    if (k < 2) k = 2;
    if (k > (size_t)kPipeMaxChunks) k = kPipeMaxChunks;
    return (int)k;
}

cudaError_t launch_nvls_pipe(const CollArgs& a_in, ncclDataType_t dt, const LaunchCfg& cfg_in, bool reduce_scatter) {
    CollArgs a = a_in;
    LaunchCfg cfg = cfg_in;
    const int nroles = reduce_scatter ? 1 + kPipeFan : 1 + 2 * kPipeFan;
    cfg.ctas = cfg.ctas / nroles * nroles;          // whole groups
    if (cfg.ctas < nroles) cfg.ctas = nroles;
    const size_t es = dt == ncclFloat64 || dt == ncclInt64 || dt == ncclUint64 ? 8 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2 : 4;
    a.mode = nvls_pipe_chunks(a.count * es * (reduce_scatter ? (size_t)a.comm.nranks : 1));
    a.root = reduce_scatter ? 1 : 0;
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
