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
 * k. Between two chunks a switch CTA has dead time: its multicast stores must
 * have landed everywhere before it may signal, and the first reductions of the
 * next chunk take a round trip through the switch before data flows (about
 * 10 us, measured as the difference between 16 and 24 chunks per launch). The
 * NV CTAs therefore form P teams (a.pipe_teams, 2 by default) that take the
 * chunks in turn, so that one team streams while the other is between chunks;
 * eight CTAs already saturate the switch pass. The groups have sizes of their own: the switch pass is bound by latency
 * and saturates with about 16 CTAs, the copies are bound by HBM and want long
 * contiguous ranges. Each copy CTA therefore moves ONE contiguous slice of a
 * chunk (a piece of a few tens of KB per source would leave the unrolled copy
 * loop idle and run at a fraction of HBM speed), and the hand-over is per
 * chunk, not per range: every CTA signals its own flag row at every rank after
 * each chunk; an NV CTA waits for the IN rows of all ranks, an OUT CTA for the
 * NV rows of all ranks. A staging half holds R chunks and is used as a ring:
 * chunk k lives in slot k % R, so one launch serves a message of any length
 * (one fill and one drain of the pipeline per call instead of one per staging
 * half). IN may run ahead by R chunks; before it overwrites a slot it waits for
 * the chunk that lived there to be gone: for the local OUT group to have
 * copied it out (which had waited for every rank's switch pass over it), in a
 * reduce-scatter for every rank's switch pass over it. Chunk numbers beyond
 * the flag values of one call continue in the call numbers of the same parity
 * that the host reserves for the launch (nvls_pipe_extra_seqs).
 *
 * Leaving the call: an all-reduce rank leaves after its OUT group has seen every
 * rank's NV flags of the last chunk, a reduce-scatter rank after its NV group has
 * seen every rank's IN flags, so a rank that leaves knows that every rank has
 * entered the call, which is what the alternation of staging halves needs.
 */
#include "kernels.hpp"
#include "../device/geometry.cuh"
#include "../device/multimem.cuh"

namespace dccl {

constexpr int kPipeMaxChunks = 24;    // flag values per call are limited (kFlagVals)
static_assert(kPipeMaxChunks < kFlagVals, "chunk numbers must fit the per-call flag values");

/** wait until point idx was signalled on the `rows` flag rows row0, row0 + stride, ... by EVERY rank */
__device__ __forceinline__ bool wait_rows_all_ranks(const DevComm& c, int row0, int rows, int stride, uint32_t seq, int idx, int site) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    for (int t = (int)threadIdx.x; t < c.nranks * rows; t += (int)blockDim.x)
        if (!wait_peer(c, t % c.nranks, row0 + (t / c.nranks) * stride, seq, idx, site)) s_fail = 1;
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
__device__ __forceinline__ void split_range(size_t len, int m, int parts, size_t ve, size_t* plo, size_t* phi) {
    size_t per = ((len + parts - 1) / parts + ve - 1) / ve * ve;
    size_t a = per * (size_t)m, b = a + per;
    if (a > len) a = len;
    if (b > len) b = len;
    *plo = a; *phi = b;
}

/** wait until point idx was signalled on the `rows` flag rows row0, row0 + 1, ... by rank `src` alone */
__device__ __forceinline__ bool wait_rows_one_rank(const DevComm& c, int src, int row0, int rows, uint32_t seq, int idx, int site) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    for (int t = (int)threadIdx.x; t < rows; t += (int)blockDim.x)
        if (!wait_peer(c, src, row0 + t, seq, idx, site)) s_fail = 1;
    __syncthreads();
    const bool ok = s_fail == 0;
    __syncthreads();
    return ok;
}

template <typename T, int OP>
__device__ __forceinline__ void nvls_pipe_body(const CollArgs& a, const Ctx& x) {
    constexpr size_t ES = sizeof(T);
    constexpr size_t VE = 16 / ES;
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank;
    const bool rs = a.root != 0;                   // reduce-scatter (count = per-rank elements) instead of all-reduce
    const int Gn = a.pipe_nv, Gc = a.pipe_copy;    // switch CTAs; copy CTAs on each side
    const int P = a.pipe_teams < 1 ? 1 : (a.pipe_teams > Gn ? Gn : a.pipe_teams);   // NV CTA g belongs to team g % P, which takes chunks k with k % P == g % P
    // CTA order: [NV (Gn)] [IN (Gc)] [OUT (Gc), all-reduce only]; a CTA's flag row is its index
    enum { ROLE_IN, ROLE_NV, ROLE_OUT };
    int role, g;
    if (x.bid < Gn) { role = ROLE_NV; g = x.bid; }
    else if (x.bid < Gn + Gc) { role = ROLE_IN; g = x.bid - Gn; }
    else if (!rs && x.bid < Gn + 2 * Gc) { role = ROLE_OUT; g = x.bid - Gn - Gc; }
    else return;                                   // left-over CTAs
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    const bool avg = a.op == (int)ncclAvg;
    const size_t stage_off = kStageOff + (size_t)x.parity * c.stage_bytes;
    T* my_stage = reinterpret_cast<T*>(c.pool[r] + stage_off);
    char* mc_stage = c.mc_pool + stage_off;
    // chosen by the host (nvls_pipe_plan): chunks of `chunk` elements (whole vectors; all-reduce: whole vectors per rank),
    // `R` of which fit a staging half. Reduce-scatter: a chunk is the same range of every rank's slot, n pieces in staging.
    const int nchunks = a.mode, R = a.pipe_ring;
    const size_t chunk = a.pipe_chunk;
    if (!stage_extent_ok<T>(c, (size_t)R * chunk * (rs ? (size_t)n : 1), 1908) ||
        !DCCL_BOUNDS_OK(c, nchunks >= 1 && R >= 1 && chunk % VE == 0 && Gn >= 1 && Gc >= 1 && Gn + 2 * Gc <= kMaxCtas, 1908, nchunks)) return;
    const int parts = rs ? (Gc + n - 1) / n : 1;   // reduce-scatter copy-in: every slot's chunk is cut into `parts` slices
    // flag value of chunk k: the first kPipeMaxChunks chunks use this call's number, later ones the following numbers of
    // the same parity, which the host has set aside for this launch
    auto seq_of = [&](int k) { return x.seq + 2u * (uint32_t)(k / kPipeMaxChunks); };
    auto idx_of = [&](int k) { return k % kPipeMaxChunks; };

    for (int k = 0; k < nchunks; k++) {
        const size_t base = (size_t)k * chunk;     // in the user buffers
        const size_t cnt = base >= a.count ? 0 : (a.count - base < chunk ? a.count - base : chunk);
        // in staging: slot k % R of the ring; reduce-scatter keeps the n pieces of a chunk side by side
        const size_t sbase = (size_t)(k % R) * chunk * (rs ? (size_t)n : 1);
        if (role == ROLE_IN) {
            if (k >= R) {
                // the slot's previous tenant, chunk k - R, must be gone
                const int kp = k - R;
                if (rs) { if (!wait_rows_all_ranks(c, kp % P, (Gn - kp % P + P - 1) / P, P, seq_of(kp), idx_of(kp), 555)) return; }
                else if (!wait_rows_one_rank(c, r, Gn + Gc, Gc, seq_of(kp), idx_of(kp), 556)) return;
            }
            size_t lo, hi;
            if (rs) {
                for (int u = g; u < n * parts && cnt; u += Gc) {      // unit u: slice u / n of slot u % n
                    const int j = u % n;
                    split_range(cnt, u / n, parts, VE, &lo, &hi);
                    if (hi > lo) copy_range<T>(my_stage + sbase + (size_t)j * chunk + lo, send + (size_t)j * a.stride + base + lo, hi - lo);
                }
            } else {
                split_range(cnt, g, Gc, VE, &lo, &hi);
                if (hi > lo) copy_range<T>(my_stage + sbase + lo, send + base + lo, hi - lo);
            }
            signal_all_ranks(c, x.bid, seq_of(k), idx_of(k));
        } else if (role == ROLE_NV) {
            if (k % P != g % P) continue;
            const int team = (Gn - g % P + P - 1) / P, gi = g / P;      // CTAs of this team, this CTA's place in it
            if (!wait_rows_all_ranks(c, Gn, Gc, 1, seq_of(k), idx_of(k), 560)) return;
            // this rank's shard of the chunk: the whole chunk of its slot (reduce-scatter) or the r-th n-th of it
            const size_t per = rs ? cnt : ((cnt + n - 1) / n + VE - 1) / VE * VE;
            const size_t s_lo = rs ? 0 : (per * (size_t)r < cnt ? per * (size_t)r : cnt);
            const size_t s_len = rs ? cnt : (cnt - s_lo < per ? cnt - s_lo : per);
            size_t lo, hi;
            split_range(s_len, gi, team, VE, &lo, &hi);
            if (hi > lo) {
                if (rs) {
                    const size_t off = (sbase + (size_t)r * chunk + lo) * ES;
                    char* dst = reinterpret_cast<char*>(recv + base + lo);
                    if (aligned16(dst)) nvls_pass<T, OP>(mc_stage + off, nullptr, dst, ((hi - lo) * ES + 15) / 16, (hi - lo) * ES, avg, n, a.unroll);
                    else {
                        // unaligned output: reduce into the own piece in staging (read through the switch by nobody but this
                        // rank: peers fold THEIR piece of this rank's staging), then copy
                        char* tmp = reinterpret_cast<char*>(my_stage + sbase + (size_t)r * chunk + lo);
                        nvls_pass<T, OP>(mc_stage + off, nullptr, tmp, ((hi - lo) * ES + 15) / 16, ((hi - lo) * ES + 15) / 16 * 16, avg, n, a.unroll);
                        __syncthreads();
                        copy_range<T>(recv + base + lo, reinterpret_cast<const T*>(tmp), hi - lo);
                    }
                } else {
                    const size_t off = (sbase + s_lo + lo) * ES;
                    nvls_pass<T, OP>(mc_stage + off, mc_stage + off, nullptr, ((hi - lo) * ES + 15) / 16, 0, avg, n, a.unroll);
                }
            }
            // all-reduce: the copy-out groups wait for this; reduce-scatter: the copy-in groups, before they reuse the slot
            signal_all_ranks(c, x.bid, seq_of(k), idx_of(k));
        } else {
            // the team that reduced chunk k: rows k % P, k % P + P, ...
            if (!wait_rows_all_ranks(c, k % P, (Gn - k % P + P - 1) / P, P, seq_of(k), idx_of(k), 570)) return;
            size_t lo, hi;
            split_range(cnt, g, Gc, VE, &lo, &hi);
            if (hi > lo) copy_range<T>(recv + base + lo, my_stage + sbase + lo, hi - lo);
            // the slot is free for this rank's copy-in group (a local flag: nobody else reads it)
            __syncthreads();
            if (threadIdx.x == 0) signal_peer(c, r, x.bid, seq_of(k), idx_of(k));
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
    // the whole message sits in one staging half; chunk and shard boundaries are rounded up to whole vectors, which a
    // capacity that is itself a multiple of 64 elements always leaves room for (the plan rounds chunks up to whole vectors
    // per rank: keep a margin of one such unit per chunk slot)
    const size_t elems = (stage_bytes / es / 64) * 64;
    const size_t margin = (size_t)kPipeMaxChunks * 16 * (size_t)nranks / es;
    const size_t cap = elems > 2 * margin ? elems - margin : elems / 2;
    return reduce_scatter ? (cap / (size_t)nranks / 64) * 64 : (cap / 64) * 64;
}

static size_t g_pipe_chunk_bytes = 16u << 20;  // target chunk size; every rank must use the same value

void nvls_pipe_set_chunk_bytes(size_t bytes) { if (bytes >= 4096) g_pipe_chunk_bytes = bytes; }

void nvls_pipe_plan(size_t count, size_t es, size_t stage_bytes, int nranks, bool reduce_scatter, bool single_seq, int* nchunks, size_t* chunk, int* ring) {
    const size_t n = (size_t)nranks, ve = 16 / es;
    const size_t unit = reduce_scatter ? ve : ve * n;                 // chunks are whole vectors (per rank, in an all-reduce)
    const size_t pieces = reduce_scatter ? n : 1;                      // a reduce-scatter chunk has one piece per rank in staging
    const size_t stage_elems = stage_bytes / es / pieces;
    // the target chunk size, but at least four slots to the ring (so that copy-in can run ahead of the switch pass) and at
    // least two chunks to a message (so that the copies overlap the switch pass at all)
    size_t target = g_pipe_chunk_bytes / es / pieces;
    if (target > stage_elems / 4) target = stage_elems / 4;
    if (target < unit) target = unit;
    size_t k = (count + target - 1) / target;
    if (k < 2) k = 2;
    if (single_seq && k > (size_t)kPipeMaxChunks) k = kPipeMaxChunks;  // only this call's flag values (and no slot twice: see the capacity)
    size_t c = ((count + k - 1) / k + unit - 1) / unit * unit;         // balanced chunks
    if (c < unit) c = unit;
    size_t r = stage_elems / c;
    k = (count + c - 1) / c;
    if (k < 1) k = 1;
    if (r > k) r = k;
    if (r < 1) r = 1;
    *nchunks = (int)k;
    *chunk = c;
    *ring = (int)r;
}

int nvls_pipe_extra_seqs(size_t count, size_t es, size_t stage_bytes, int nranks, bool reduce_scatter, bool single_seq) {
    int k, r;
    size_t c;
    nvls_pipe_plan(count, es, stage_bytes, nranks, reduce_scatter, single_seq, &k, &c, &r);
    return 2 * ((k - 1) / kPipeMaxChunks);
}

void nvls_pipe_split(int ctas, int nv, bool reduce_scatter, int* nv_out, int* copy_out) {
    const int sides = reduce_scatter ? 1 : 2;
    if (ctas < 1 + sides) ctas = 1 + sides;
    if (nv <= 0) nv = ctas / (1 + 2 * sides);       // by default the copy groups are twice the switch group
    if (nv < 1) nv = 1;
    if (nv > ctas - sides) nv = ctas - sides;
    int copy = (ctas - nv) / sides;
    if (nv + sides * copy > kMaxCtas) copy = (kMaxCtas - nv) / sides;
    *nv_out = nv;
    *copy_out = copy;
}

cudaError_t launch_nvls_pipe(const CollArgs& a_in, ncclDataType_t dt, const LaunchCfg& cfg_in, bool reduce_scatter, size_t stage_bytes, int nv_ctas, int teams, bool single_seq) {
    CollArgs a = a_in;
    LaunchCfg cfg = cfg_in;
    a.pipe_teams = teams;
    nvls_pipe_split(cfg.ctas, nv_ctas, reduce_scatter, &a.pipe_nv, &a.pipe_copy);
    cfg.ctas = a.pipe_nv + (reduce_scatter ? 1 : 2) * a.pipe_copy;
    const size_t es = dt == ncclFloat64 || dt == ncclInt64 || dt == ncclUint64 ? 8 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2 : 4;
    const int n = a.emu ? cfg.ranks_in_launch : a.comm.nranks;
    nvls_pipe_plan(a.count, es, stage_bytes, n, reduce_scatter, single_seq, &a.mode, &a.pipe_chunk, &a.pipe_ring);
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
