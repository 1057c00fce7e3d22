/**
 * Pipelined switch (NVLS) broadcast and reduce for large ORDINARY device buffers.
 *
 * The staged forms in nvls.cu run their phases one after the other: broadcast
 * pushes the whole message through the switch into every rank's staging and
 * then every rank copies it out; reduce copies everything into staging and then
 * the root pulls the reduction through the switch. Here the message is cut
 * into chunks and the local copies of one chunk run while the switch works on
 * the next, in ONE launch:
 *
 *   broadcast  root CTA g:   multimem.st its part of chunk k to all ranks, signal row g of every rank
 *              other ranks:  CTA g waits for the root CTAs that pushed chunk k, copies its slice of the chunk
 *                            from staging to the user buffer
 *   reduce     every rank, CTA g (first half of the grid): copy its slice of chunk k into staging, signal row g of the root
 *              root, CTA G+g (second half):                wait for the copies of chunk k of every rank,
 *                                                          multimem.ld_reduce its part of the chunk into the user buffer
 *
 * The CTAs that talk to the switch (the root's) form two teams that take the chunks in turn: between two chunks such
 * a CTA has dead time (its multicast stores must have landed everywhere before it may signal, and the first accesses of
 * the next chunk take a round trip through the switch), during which the other team keeps the links busy.
 *
 * The whole message sits in one staging half, so no byte of it is reused within
 * a launch and the hand-over needs no back pressure. The side that waits for
 * nobody during the pipeline (the root of a broadcast, the non-roots of a
 * reduce) waits at the end for the others, so that a later call cannot reach
 * the same staging half while it is still being read. Like every kernel of the
 * library, a rank also leaves only when it knows that every rank has entered
 * this call (that is what lets staging halves and packet generations alternate
 * without trailing barriers): the pipeline alone tells a receiver about the
 * root only, so every CTA announces its entry to all peers when it starts
 * (flag index 0; chunk k uses index k+1) and checks the announcements at the end.
 *
 * The original's broadcast is a Derecho multicast into host memory followed by
 * a memcpy, and its reduce a gather of slots to the root (reference
 * src/core/dccl.cpp:701-736, 745-846); neither takes device buffers.
 */
#include "kernels.hpp"
#include "../device/geometry.cuh"
#include "../device/multimem.cuh"

namespace dccl {

constexpr int kRootedMaxChunks = 24;
constexpr int kRootedDone = 31;        // flag index of the trailing hand-shake
static_assert(kRootedMaxChunks + 1 < kRootedDone && kRootedDone < kFlagVals, "chunk numbers and the trailing index share the per-call flag values");

template <typename T, int OP>
__device__ __forceinline__ void nvls_rooted_body(const CollArgs& a, const Ctx& x) {
    constexpr size_t ES = sizeof(T);
    constexpr size_t VE = 16 / ES;
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank, root = a.root;
    const bool reduce = a.mode == ROOTED_REDUCE;
    const int nchunks = (int)a.stride;
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    const bool avg = a.op == (int)ncclAvg;
    const size_t stage_off = kStageOff + (size_t)x.parity * c.stage_bytes;
    T* my_stage = reinterpret_cast<T*>(c.pool[r] + stage_off);
    char* mc_stage = c.mc_pool + stage_off;
    const size_t chunk = ((a.count + nchunks - 1) / nchunks + VE - 1) / VE * VE;
    auto vecs = [&](size_t elems) { return (elems * ES + 15) / 16; };
    __shared__ int s_fail;
    if (!stage_extent_ok<T>(c, (a.count + VE - 1) / VE * VE, 1909) ||
        !DCCL_BOUNDS_OK(c, nchunks >= 1 && nchunks <= kRootedMaxChunks, 1909, nchunks)) return;

    // reduce: the first half of the grid copies in (every rank), the second half is the root's switch pass
    const int G = reduce ? x.nb / 2 : x.nb;
    const bool second = reduce && x.bid >= G;
    const int g = second ? x.bid - G : x.bid;
    if (reduce && (x.bid >= 2 * G || (second && r != root))) return;
    // the CTAs that use the switch (root of a broadcast, second group of a reduce) work in P teams: CTA g belongs to
    // team g % P, which takes the chunks k with k % P == g % P
    const int P = G >= 2 ? 2 : 1;
    const int team_of_g = g % P, gi = g / P, team_size = (G - team_of_g + P - 1) / P;
    // entry announcement; the root's second group shares rows with its first and leaves it to that one
    if (!second && (int)threadIdx.x < n && (int)threadIdx.x != r) signal_peer(c, (int)threadIdx.x, g, x.seq, 0);

    for (int k = 0; k < nchunks; k++) {
        const size_t base = (size_t)k * chunk;
        const size_t cnt = base >= a.count ? 0 : (a.count - base < chunk ? a.count - base : chunk);
        // a copy CTA's slice of the chunk (1/G), and a switch CTA's part of it (1/team size)
        const Geometry<T> whole(GEO_WHOLE, cnt, 1, g, G), part(GEO_WHOLE, cnt, 1, gi, team_size);
        const bool mine = k % P == team_of_g;
        if (!reduce) {
            if (r == root) {
                if (!mine) continue;
                const size_t lo = part.blo < cnt ? part.blo : cnt, hi = part.bhi < cnt ? part.bhi : cnt, off = base + lo;
                if (hi > lo) {
                    const T* src = send + off;
                    if (aligned16(src)) nvls_push(mc_stage + off * ES, reinterpret_cast<const char*>(src), vecs(hi - lo));
                    else {   // multimem.st wants whole aligned vectors: go through the own staging copy
                        copy_range<T>(my_stage + off, src, hi - lo);
                        __syncthreads();
                        nvls_push(mc_stage + off * ES, reinterpret_cast<const char*>(my_stage + off), vecs(hi - lo));
                    }
                    if (recv != send) copy_range<T>(recv + off, src, hi - lo);
                }
                __syncthreads();
                if ((int)threadIdx.x < n) signal_peer(c, (int)threadIdx.x, g, x.seq, k + 1);
            } else {
                // the root CTAs of the team that pushed chunk k: rows k % P, k % P + P, ...
                const int t0 = k % P, rows = (G - t0 + P - 1) / P;
                if (threadIdx.x == 0) s_fail = 0;
                __syncthreads();
                for (int t = (int)threadIdx.x; t < rows; t += (int)blockDim.x)
                    if (!wait_peer(c, root, t0 + t * P, x.seq, k + 1, 580)) s_fail = 1;
                __syncthreads();
                if (s_fail) return;
                const size_t lo = whole.blo < cnt ? whole.blo : cnt, hi = whole.bhi < cnt ? whole.bhi : cnt, off = base + lo;
                if (hi > lo) copy_range<T>(recv + off, my_stage + off, hi - lo);
                __syncthreads();
            }
        } else if (!second) {
            const size_t lo = whole.blo < cnt ? whole.blo : cnt, hi = whole.bhi < cnt ? whole.bhi : cnt, off = base + lo;
            if (hi > lo) copy_range<T>(my_stage + off, send + off, hi - lo);
            cta_signal_peer(c, root, g, x.seq, k + 1);
        } else {
            if (!mine) continue;
            if (threadIdx.x == 0) s_fail = 0;
            __syncthreads();
            // every copy CTA of every rank has brought its slice of chunk k
            for (int t = (int)threadIdx.x; t < n * G; t += (int)blockDim.x)
                if (!wait_peer(c, t % n, t / n, x.seq, k + 1, 590)) s_fail = 1;
            __syncthreads();
            if (s_fail) return;
            const size_t lo = part.blo < cnt ? part.blo : cnt, hi = part.bhi < cnt ? part.bhi : cnt, off = base + lo;
            if (hi > lo) {
                char* dst = reinterpret_cast<char*>(recv + off);
                if (aligned16(dst)) nvls_pass<T, OP>(mc_stage + off * ES, nullptr, dst, vecs(hi - lo), (hi - lo) * ES, avg, n, a.unroll);
                else {   // unaligned output: reduce into the own staging copy (each vector is read once, then replaced), then copy
                    nvls_pass<T, OP>(mc_stage + off * ES, nullptr, reinterpret_cast<char*>(my_stage + off), vecs(hi - lo), vecs(hi - lo) * 16, avg, n, a.unroll);
                    __syncthreads();
                    copy_range<T>(recv + off, my_stage + off, hi - lo);
                }
            }
            __syncthreads();
        }
    }

    // trailing hand-shake: whoever waited for nobody so far waits for the others now
    if (!reduce) {
        if (r != root) cta_signal_peer(c, root, g, x.seq, kRootedDone);
        else if ((int)threadIdx.x < n && (int)threadIdx.x != root) wait_peer(c, (int)threadIdx.x, g, x.seq, kRootedDone, 585);
    } else if (second) {
        __syncthreads();
        if ((int)threadIdx.x < n && (int)threadIdx.x != root) signal_peer(c, (int)threadIdx.x, g, x.seq, kRootedDone);
    } else if (r != root) {
        if (threadIdx.x == 0) wait_peer(c, root, g, x.seq, kRootedDone, 595);
    }
    // nobody leaves before everybody has entered (the announcements have normally long arrived)
    if (!second && (int)threadIdx.x < n && (int)threadIdx.x != r) wait_peer(c, (int)threadIdx.x, g, x.seq, 0, 597);
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_nvls_rooted(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    nvls_rooted_body<T, OP>(a, x);
    finish_call(x);
}

int nvls_rooted_chunks(size_t bytes) {
    size_t k = (bytes + (8u << 20) - 1) / (8u << 20);
    if (k < 2) k = 2;
    if (k > (size_t)kRootedMaxChunks) k = kRootedMaxChunks;
    return (int)k;
}

cudaError_t launch_nvls_rooted(const CollArgs& a_in, ncclDataType_t dt, const LaunchCfg& cfg_in) {
    CollArgs a = a_in;
    LaunchCfg cfg = cfg_in;
    const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                      : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
    if (a.mode == ROOTED_REDUCE) {
        cfg.ctas = cfg.ctas / 2 * 2;                 // copy-in half and switch half
        if (cfg.ctas < 2) cfg.ctas = 2;
    }
    if (a.mode == ROOTED_BROADCAST) {
        // pure data movement: run on bytes
        a.count = a.count * es;
        a.stride = (size_t)nvls_rooted_chunks(a.count);
        return launch_coll(k_nvls_rooted<uint8_t, OP_SUM>, a, cfg);
    }
    a.stride = (size_t)nvls_rooted_chunks(a.count * es);
    const int op = a.op == (int)ncclAvg ? (int)ncclSum : a.op;
    switch (dt) {
#define ROOTED_CASE(DT, T)                                                                    \
    case DT:                                                                                  \
        if (op == (int)ncclSum) return launch_coll(k_nvls_rooted<T, OP_SUM>, a, cfg);         \
        if (op == (int)ncclMax) return launch_coll(k_nvls_rooted<T, OP_MAX>, a, cfg);         \
        if (op == (int)ncclMin) return launch_coll(k_nvls_rooted<T, OP_MIN>, a, cfg);         \
        break;
#define ROOTED_CASE_SUM(DT, T)                                                                \
    case DT:                                                                                  \
        if (op == (int)ncclSum) return launch_coll(k_nvls_rooted<T, OP_SUM>, a, cfg);         \
        break;
    ROOTED_CASE_SUM(ncclFloat32, float)
    ROOTED_CASE_SUM(ncclFloat64, double)
    ROOTED_CASE(ncclFloat16, __half)
    ROOTED_CASE(ncclBfloat16, __nv_bfloat16)
    ROOTED_CASE(ncclInt32, int32_t)
    ROOTED_CASE(ncclUint32, uint32_t)
    ROOTED_CASE(ncclInt64, long long)
    ROOTED_CASE(ncclUint64, unsigned long long)
#undef ROOTED_CASE
#undef ROOTED_CASE_SUM
    default: break;
    }
    return cudaErrorInvalidValue;
}

} // namespace dccl
