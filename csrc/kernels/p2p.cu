/**
 * ncclSend / ncclRecv: stream-ordered peer copies through a small FIFO in the
 * receiver's pool.
 *
 * The original moves a message with one matched zero-copy RDMA send/recv pair,
 * blocking the host, host memory only (reference src/core/dccl.cpp:865-911).
 * Here the sender's kernel writes 1 MB chunks straight into the receiver's
 * FIFO over NVLink and bumps a head counter there; the receiver's kernel
 * copies chunks out as they arrive and returns credit through a tail counter
 * in the sender's pool. Matching is FIFO per peer, like the original; the
 * counters are cumulative chunk numbers, one pair per FIFO slot, so nothing is ever reset. A send of
 * up to kP2pDepth chunks completes without the receiver having started.
 * Several sends and receives recorded between dcclGroupStart/End run in ONE
 * launch with a group of CTAs per operation, so a ring in which every rank
 * sends and receives cannot deadlock.
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"

namespace dccl {

// One head and one tail word per (peer, FIFO slot, CTA): several operations of one launch may address the
// same peer (a window of sends), each works on its own slot and must not see another slot's progress.
__device__ __forceinline__ unsigned long long* p2p_head(char* pool, int src, unsigned long long chunk, int cta) {
    return reinterpret_cast<unsigned long long*>(pool + kP2pFlagOff) + ((src * kP2pDepth + (int)(chunk % kP2pDepth)) * kP2pCtas + cta);
}
__device__ __forceinline__ unsigned long long* p2p_tail(char* pool, int dst, unsigned long long chunk, int cta) {
    return reinterpret_cast<unsigned long long*>(pool + kP2pFlagOff) + (kMaxPeers * kP2pDepth * kP2pCtas + (dst * kP2pDepth + (int)(chunk % kP2pDepth)) * kP2pCtas + cta);
}
__device__ __forceinline__ char* p2p_fifo(char* pool, int src, unsigned long long chunk) {
    return pool + kP2pOff + (size_t)src * kP2pBytesPerSrc + (size_t)(chunk % kP2pDepth) * kP2pChunk;
}

__global__ void __launch_bounds__(512) k_p2p(const __grid_constant__ P2pArgs a) {
    const DevComm* cp;
    const P2pOp* ops;
    int nops, bid;
    if (a.emu) {
        const int vr = blockIdx.x / a.ctas_per_rank;
        cp = a.emu + vr;
        ops = a.emu_ops + (size_t)vr * kMaxP2pOps;
        nops = a.emu_nops[vr];
        bid = blockIdx.x - vr * a.ctas_per_rank;
    } else {
        cp = &a.comm;
        ops = a.ops;
        nops = a.nops;
        bid = blockIdx.x;
    }
    const DevComm& c = *cp;
    const int opi = bid / a.ctas_per_op, b = bid - opi * a.ctas_per_op, B = a.ctas_per_op;
    if (opi >= nops) return;
    if (!DCCL_BOUNDS_OK(c, B >= 1 && B <= kP2pCtas && nops <= kMaxP2pOps, 1906, B)) return;   // head / tail words per pair: one per CTA
    const P2pOp op = ops[opi];
    const int r = c.rank, peer = op.peer;
    const size_t nchunks = (op.bytes + kP2pChunk - 1) / kP2pChunk;
    __shared__ int s_ok;

    for (size_t ci = 0; ci < nchunks; ci++) {
        const unsigned long long G = op.chunk_base + ci;
        const size_t coff = ci * kP2pChunk;
        const size_t clen = op.bytes - coff < kP2pChunk ? op.bytes - coff : kP2pChunk;
        // This CTA's 16-byte aligned part of the chunk. The cut is that of a FULL chunk whatever the chunk's length, so
        // that CTA b always owns the same bytes of a FIFO slot: its credit word then covers exactly what it overwrites,
        // also when the slot's previous tenant was the short last chunk of a message (a cut that followed the chunk's
        // length would let CTA b overwrite bytes that another receiving CTA has not read yet). Short chunks are
        // served by the first CTAs only.
        const size_t sub = ((kP2pChunk + B - 1) / B + 15) / 16 * 16;
        size_t lo = sub * (size_t)b; if (lo > clen) lo = clen;
        size_t hi = lo + sub; if (hi > clen) hi = clen;
        if (op.is_send) {
            if (threadIdx.x == 0) {
                s_ok = 1;
                if (G >= (unsigned long long)kP2pDepth)   // wait until the slot's previous tenant was consumed
                    s_ok = wait_flag64_ge(c, p2p_tail(c.pool[r], peer, G, b), G - kP2pDepth + 1, peer, 800, 0) ? 1 : 0;
            }
            __syncthreads();
            if (!s_ok) return;
            if (hi > lo) copy_bytes(p2p_fifo(c.pool[peer], r, G) + lo, op.buf + coff + lo, hi - lo);
            __syncthreads();
            if (threadIdx.x == 0) {
                st_release_sys64(p2p_head(c.pool[peer], r, G, b), G + 1);
            }
        } else {
            if (threadIdx.x == 0) s_ok = wait_flag64_ge(c, p2p_head(c.pool[r], peer, G, b), G + 1, peer, 810, 0) ? 1 : 0;
            __syncthreads();
            if (!s_ok) return;
            if (hi > lo) copy_bytes(op.buf + coff + lo, p2p_fifo(c.pool[r], peer, G) + lo, hi - lo);
            __syncthreads();
            if (threadIdx.x == 0) {
                st_release_sys64(p2p_tail(c.pool[peer], r, G, b), G + 1);
            }
        }
    }
}

cudaError_t launch_p2p(const P2pArgs& a, const LaunchCfg& cfg) {
    return launch_kernel(k_p2p, &a, cfg);
}

} // namespace dccl
