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
 *
 * Large messages (kP2pRdvMinBytes and more; both ends know the size) are
 * rendezvous messages, the form of the original's matched transfer: the
 * receiver's kernel posts where its buffer lies (a segment of symmetric memory,
 * or an allocation it has exported) in the SENDER's pool; the sender's kernel
 * looks that up among the mappings it was launched with. When it has the buffer
 * mapped it says so (path word), its CTAs store the message straight into the
 * receiver's memory, and the last of them to finish raises the done word: one
 * pass over NVLink, no staging, no credit round trips. Otherwise it says
 * "FIFO" and both ends run the chunk loop. The receiver of a direct message
 * hands back the FIFO credit of the chunk numbers the message would have used,
 * so chunk numbers stay the cumulative count both hosts keep.
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

/* Rendezvous words at kP2pRdvOff of a pool, per (other rank, slot): a 64-byte post {kind, a, id, offset, -, -, -, seq}
 * written by the receiver into the sender's pool; then the path word and the done word, written by the sender into the
 * receiver's pool; then the sender's own arrival counter. Values are 1 + the pair's rendezvous number (path: twice
 * that, plus 1 for "direct"), so they are never reset. */
__device__ __forceinline__ unsigned long long* rdv_post(char* pool, int other, unsigned long long idx) {
    return reinterpret_cast<unsigned long long*>(pool + kP2pRdvOff) + ((size_t)other * kP2pRdvSlots + (size_t)(idx % kP2pRdvSlots)) * 8;
}
__device__ __forceinline__ unsigned long long* rdv_word(char* pool, int which, int other, unsigned long long idx) {
    return reinterpret_cast<unsigned long long*>(pool + kP2pRdvOff + (size_t)kMaxPeers * kP2pRdvSlots * 64) +
           ((size_t)which * kMaxPeers + (size_t)other) * kP2pRdvSlots + (size_t)(idx % kP2pRdvSlots);
}
enum { RDV_PATH = 0, RDV_DONE = 1, RDV_ARRIVE = 2 };

/** One thread waits until *p >= val; every thread of the CTA then reads the word itself (0: the wait gave up).
 *  Only a success flag goes through shared memory. */
__device__ __forceinline__ unsigned long long cta_wait64(const DevComm& c, const unsigned long long* p, unsigned long long val, int peer, int site) {
    __shared__ int s_fine;
    if (threadIdx.x == 0) s_fine = wait_flag64_ge(c, p, val, peer, site, 0) ? 1 : 0;
    __syncthreads();
    const bool fine = s_fine != 0;
    __syncthreads();
    return fine ? ld_acquire_sys64(p) : 0ull;
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

    if (op.rdv) {
        const unsigned long long want = op.rdv_index + 1;
        if (!op.is_send) {
            // tell the sender where the buffer lies, then learn which way the data comes
            if (b == 0 && threadIdx.x == 0) {
                unsigned long long* post = rdv_post(c.pool[peer], r, op.rdv_index);
                volatile unsigned long long* pv = post;
                pv[0] = (unsigned long long)op.dst_kind; pv[1] = op.dst_a; pv[2] = op.dst_id; pv[3] = op.dst_off;
                st_release_sys64(post + 7, want);
            }
            const unsigned long long path = cta_wait64(c, rdv_word(c.pool[r], RDV_PATH, peer, op.rdv_index), 2 * want, peer, 820);
            if (!path) return;
            if (path & 1ull) {
                if (!cta_wait64(c, rdv_word(c.pool[r], RDV_DONE, peer, op.rdv_index), want, peer, 830)) return;
                // the FIFO slots of the chunk numbers this message did not use count as consumed: credit for whoever
                // comes next (every CTA word of a slot, so that the number of CTAs on the other side does not matter)
                if (b == 0) {
                    const size_t last = nchunks < (size_t)kP2pDepth ? nchunks : (size_t)kP2pDepth;
                    for (size_t t = threadIdx.x; t < last * kP2pCtas; t += blockDim.x) {
                        const unsigned long long G = op.chunk_base + nchunks - 1 - t / kP2pCtas;
                        st_release_sys64(p2p_tail(c.pool[peer], r, G, (int)(t % kP2pCtas)), G + 1);
                    }
                }
                return;
            }
        } else {
            unsigned long long* post = rdv_post(c.pool[r], peer, op.rdv_index);
            if (!cta_wait64(c, post + 7, want, peer, 840)) return;
            const volatile unsigned long long* pv = post;
            const unsigned long long kind = pv[0], da = pv[1], did = pv[2], doff = pv[3];
            char* dst = nullptr;
            for (int m = 0; m < a.nmaps && kind != P2P_DST_NONE; m++) {
                const P2pMap& mp = a.maps[m];
                if (mp.peer == peer && (unsigned long long)mp.kind == kind && mp.a == da && mp.id == did && doff + op.bytes <= mp.size) { dst = mp.mapped + doff; break; }
            }
            if (b == 0 && threadIdx.x == 0) st_release_sys64(rdv_word(c.pool[peer], RDV_PATH, r, op.rdv_index), 2 * want + (dst ? 1ull : 0ull));
            if (dst) {
                // this CTA's contiguous part; the cut keeps source and destination equally aligned
                const size_t per = ((op.bytes + B - 1) / B + 15) / 16 * 16;
                size_t lo = per * (size_t)b; if (lo > op.bytes) lo = op.bytes;
                size_t hi = lo + per; if (hi > op.bytes) hi = op.bytes;
                if (hi > lo) copy_bytes(dst + lo, op.buf + lo, hi - lo);
                __syncthreads();
                if (threadIdx.x == 0) {
                    // the last CTA of this operation to get here has seen, through the counter, that the others' stores
                    // are done (fence, counter, fence), and publishes the message
                    __threadfence_system();
                    unsigned int* arrive = reinterpret_cast<unsigned int*>(rdv_word(c.pool[r], RDV_ARRIVE, peer, op.rdv_index));
                    if (atomicAdd(arrive, 1u) == (unsigned int)(B - 1)) {
                        *reinterpret_cast<volatile unsigned int*>(arrive) = 0u;
                        __threadfence_system();
                        st_release_sys64(rdv_word(c.pool[peer], RDV_DONE, r, op.rdv_index), want);
                    }
                }
                return;
            }
        }
    }

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
                // the head word carries, above the chunk number, how many CTAs serve this operation here: both ends cut a
                // chunk by that number, and the receiver checks that they agree
                st_release_sys64(p2p_head(c.pool[peer], r, G, b), (G + 1) | ((unsigned long long)B << 56));
            }
        } else {
            if (threadIdx.x == 0) {
                const unsigned long long* hp = p2p_head(c.pool[r], peer, G, b);
                s_ok = wait_flag64_ge(c, hp, G + 1, peer, 810, 0, (1ull << 56) - 1) ? 1 : 0;
                if (s_ok && (int)(ld_acquire_sys64(hp) >> 56) != B) {
                    // the sender cut this chunk for another number of CTAs (p2p_ctas or the shape of a group differs
                    // between the ranks): the bytes of this CTA's part may not be there. Say so instead of copying.
                    report_failure(c, DEV_MISMATCH, peer, 811, (uint32_t)(ld_acquire_sys64(hp) >> 56));
                    s_ok = 0;
                }
            }
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
