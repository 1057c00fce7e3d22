/**
 * Device-side building blocks shared by every collective kernel:
 * the per-rank communicator view (DevComm), the layout of the symmetric pool,
 * system-scope flag operations with BOUNDED waits, and the cross-GPU barrier.
 *
 * These replace the host-side wait_for_oob_op(timeout) of the original
 * (reference src/core/internal_common.hpp:771-792): a step is complete when a
 * flag word in this GPU's pool, written by the peer GPU after its data, reaches
 * the expected value. A wait that runs out of time (or sees the abort word)
 * records {code, peer, site, sequence} in a status block the host can read and
 * makes the kernel return normally; it never traps and never spins forever.
 */
#pragma once
#include <cstdint>
#include <cstddef>
#include <cuda_runtime.h>
#ifdef DCCL_HOST_SIM
#include <time.h>
#endif

namespace dccl {

constexpr int kMaxPeers = 8;            // one NVSwitch domain
constexpr int kMaxCtas = 256;           // flag rows per pool
constexpr int kFlagVals = 32;           // flag values reserved per collective call

/* ---- symmetric pool layout (byte offsets from the pool base) ---- */
constexpr size_t kFlagOff = 0;                          // uint32 flags[kMaxCtas][kMaxPeers]
constexpr size_t kP2pFlagOff = 16u << 10;               // uint64 head[kMaxPeers][kP2pDepth][kP2pCtas], then tail[...] likewise
constexpr int kP2pCtas = 32;                            // CTAs that can serve one direction of a pair
constexpr size_t kP2pRdvOff = 32u << 10;                // rendezvous words of zero-copy send / recv (p2p.cu), 12 KB
constexpr int kP2pRdvSlots = 16;                        // large messages per pair that one launch can hold
constexpr size_t kLLOff = 64u << 10;                    // flag-in-data packets
constexpr size_t kLLSlotBytes = 256u << 10;             // packets per source rank (half of it is payload)
constexpr size_t kLLBytes = 2 * kMaxPeers * kLLSlotBytes;   // two generations
constexpr size_t kLLMaxPayload = kLLSlotBytes / 2;
constexpr size_t kP2pOff = 8u << 20;                    // send/recv FIFOs, one per source rank
constexpr size_t kP2pChunk = 1u << 20;
constexpr int kP2pDepth = 4;
constexpr size_t kP2pBytesPerSrc = kP2pChunk * kP2pDepth;
constexpr size_t kLL2Off = 40u << 20;                   // packets of the two-shot packet all-reduce
constexpr size_t kLL2PhaseBytes = 1u << 20;             // per generation, source rank and phase (half of it is payload)
constexpr size_t kStageOff = 80u << 20;                 // two staging halves follow
static_assert(kLLOff + kLLBytes <= kP2pOff, "LL region overlaps the p2p FIFOs");
static_assert(kP2pFlagOff + 2 * kMaxPeers * 4 * kP2pCtas * 8 <= kP2pRdvOff, "p2p flag words overlap the rendezvous words");
static_assert(kP2pRdvOff + kMaxPeers * kP2pRdvSlots * (64 + 8 + 8 + 8) <= kLLOff, "rendezvous words overlap the packet region");
static_assert(kP2pOff + kMaxPeers * kP2pBytesPerSrc <= kLL2Off, "p2p FIFOs overlap the second packet region");
static_assert(kLL2Off + 2 * kMaxPeers * 2 * kLL2PhaseBytes <= kStageOff, "second packet region overlaps the staging area");

/* ---- status block (pinned host memory, or device memory in single-GPU emulation) ---- */
enum : uint32_t { ST_CODE = 0, ST_PEER = 1, ST_SITE = 2, ST_SEQ = 3, ST_KERNEL = 4, ST_WORDS = 8 };
enum : uint32_t { DEV_OK = 0, DEV_TIMEOUT = 1, DEV_ABORTED = 2, DEV_BOUNDS = 3,
                  DEV_MISMATCH = 4 };   // the two ends of a send / recv were launched with different CTA counts per operation

/** What a kernel needs to know about the communicator; passed by value. */
struct DevComm {
    int rank;
    int nranks;
    char* pool[kMaxPeers];        // every rank's pool as mapped into this rank's address space
    char* mc_pool;                // multicast mapping of the pool, or nullptr
    uint32_t* status;             // status block
    const uint32_t* abort_word;   // non-zero: stop waiting
    unsigned long long timeout_ns;
    size_t stage_bytes;           // bytes of one staging half
    // Sequence number kept on the device (nullptr: the host counts and passes it with every launch).
    // seq_word holds the number of the NEXT call; the last CTA of a call to finish advances it, so a
    // captured launch can be replayed without the host knowing how often it ran.
    uint32_t* seq_word;
    uint32_t* done_word;          // CTAs of the running call that have finished
};

/** User buffers of one (virtual) rank. */
struct RankIO {
    const void* send;
    void* recv;
    // when the buffer lies in symmetric memory: the same offset in every peer's mapping, and its multicast alias
    const char* send_peer[kMaxPeers];
    char* recv_peer[kMaxPeers];
    const char* send_mc;
    char* recv_mc;
};

/** Common kernel arguments. With `emu` set, one launch plays all ranks on one GPU:
 *  CTA b belongs to virtual rank b / ctas_per_rank (cooperative launch, every CTA resident). */
struct CollArgs {
    DevComm comm;
    RankIO io;
    const DevComm* emu;
    const RankIO* emu_io;
    int ctas_per_rank;
    size_t count;          // elements; per-kernel meaning
    size_t stride;         // reduce-scatter / all-gather: distance between two ranks' slots in the user buffer
    uint32_t seq;          // collective sequence number of this call
    int parity;            // staging half / LL generation
    int op;                // ncclRedOp_t
    int root;
    int mode;
    int symmetric;         // user buffers are in symmetric memory (zero-copy variant)
    int unroll;            // vectors in flight per thread in the switch pass (2, 4 or 8)
    int pipe_nv;           // pipelined switch kernels: CTAs of the switch group ...
    int pipe_copy;         // ... and of each copy group
    int pipe_teams;        // ... and how many teams the switch group forms (they take the chunks in turn)
    int pipe_ring;         // ... chunk slots in a staging half
    size_t pipe_chunk;     // ... and elements per chunk
};

struct Ctx {
    const DevComm* c;
    const RankIO* io;
    int bid;               // CTA index within the rank
    int nb;                // CTAs per rank
    uint32_t seq;          // sequence number of this call (from the host, or read from the device counter)
    int parity;            // staging half / LL generation of this call
};

__device__ __forceinline__ Ctx make_ctx(const CollArgs& a) {
    Ctx x;
    if (a.emu) {
        int vr = blockIdx.x / a.ctas_per_rank;
        x.c = a.emu + vr;
        x.io = a.emu_io + vr;
        x.bid = blockIdx.x - vr * a.ctas_per_rank;
        x.nb = a.ctas_per_rank;
    } else {
        x.c = &a.comm;
        x.io = &a.io;
        x.bid = blockIdx.x;
        x.nb = gridDim.x;
    }
    x.seq = a.seq;
    x.parity = a.parity;
    if (x.c->seq_word != nullptr) {
        // every CTA of the call reads the same value: the counter only moves after all of them have finished
#ifdef DCCL_HOST_SIM
        x.seq = __atomic_load_n(x.c->seq_word, __ATOMIC_ACQUIRE);
#else
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(x.seq) : "l"(x.c->seq_word) : "memory");
#endif
        x.parity = (int)(x.seq & 1u);
    }
    return x;
}

/** Sequence number after `seq`; 0 is never used (a zeroed packet slot must not look like a valid tag). */
__host__ __device__ __forceinline__ uint32_t next_seq(uint32_t seq) { return seq + 1u ? seq + 1u : 1u; }

/** Last statement of every collective kernel. With a device-side sequence counter, the CTA that finishes
 *  last advances it for the next call on the stream; with a host-side counter there is nothing to do. */
__device__ __forceinline__ void finish_call(const Ctx& x) {
    const DevComm& c = *x.c;
    if (c.seq_word == nullptr) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(c.done_word, 1u) == (uint32_t)(x.nb - 1)) {
            *reinterpret_cast<volatile uint32_t*>(c.done_word) = 0u;
            *reinterpret_cast<volatile uint32_t*>(c.seq_word) = next_seq(x.seq);
        }
    }
}

/* ---- system-scope memory operations ---- */

#ifdef DCCL_HOST_SIM
/* Host simulation (make SIM=1): the same operations on host memory. Loads that are polled yield the processor,
 * a 16-byte packet access is two 8-byte atomic halves {data, tag}, which is what the packet protocol relies on. */
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) { ::dccl_sim::pause(); return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
__device__ __forceinline__ void st_release_sys64(unsigned long long* p, unsigned long long v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
__device__ __forceinline__ unsigned long long ld_acquire_sys64(const unsigned long long* p) { ::dccl_sim::pause(); return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    ::dccl_sim::pause();
    const unsigned long long* q = static_cast<const unsigned long long*>(p);
    const unsigned long long a = __atomic_load_n(q, __ATOMIC_ACQUIRE), b = __atomic_load_n(q + 1, __ATOMIC_ACQUIRE);
    return make_uint4((unsigned)a, (unsigned)(a >> 32), (unsigned)b, (unsigned)(b >> 32));
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
    unsigned long long* q = static_cast<unsigned long long*>(p);
    __atomic_store_n(q, (unsigned long long)v.x | ((unsigned long long)v.y << 32), __ATOMIC_RELEASE);
    __atomic_store_n(q + 1, (unsigned long long)v.z | ((unsigned long long)v.w << 32), __ATOMIC_RELEASE);
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (unsigned long long)ts.tv_sec * 1000000000ull + (unsigned long long)ts.tv_nsec;
}
#else
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#endif

/** Record a failure for the host. The first report is kept (checked without an atomic, because the
 *  block may live in pinned host memory; two reports racing only mix two true failures). */
__device__ __forceinline__ void report_failure(const DevComm& c, uint32_t code, int peer, int site, uint32_t seq) {
    if (ld_volatile_u32(c.status + ST_CODE) == 0u) {
        volatile uint32_t* st = c.status;
        st[ST_PEER] = (uint32_t)peer;
        st[ST_SITE] = (uint32_t)site;
        st[ST_SEQ] = seq;
        __threadfence_system();
        st[ST_CODE] = code;
        __threadfence_system();
    }
}

/**
 * Range checks of a debug build (compile with -DDCCL_DEBUG_BOUNDS, `make BOUNDS=1`). Every kernel checks, before its
 * first access, that the part of the pool it is about to use (staging areas, packet slots, flag rows) lies inside the
 * region reserved for it; signal / wait check their flag row and index. A failed check records
 * {DEV_BOUNDS, own rank, site, offending value} in the status block and the kernel returns without touching memory;
 * nothing traps. In the normal build the macro is the constant `true` and the checks cost nothing.
 */
#ifdef DCCL_DEBUG_BOUNDS
__device__ __forceinline__ bool bounds_ok(const DevComm& c, bool cond, int site, size_t value) {
    if (!cond) report_failure(c, DEV_BOUNDS, c.rank, site, value > 0xffffffffull ? 0xffffffffu : (uint32_t)value);
    return cond;
}
#define DCCL_BOUNDS_OK(c, cond, site, value) (::dccl::bounds_ok((c), (cond), (site), (size_t)(value)))
#else
#define DCCL_BOUNDS_OK(c, cond, site, value) (true)
#endif

/** Spin until *p has reached `val` (wrap-safe). False after timeout_ns or when the abort word is set. */
__device__ __forceinline__ bool wait_flag_ge(const DevComm& c, const uint32_t* p, uint32_t val, int peer, int site, uint32_t seq) {
    uint32_t spins = 0;
    unsigned long long t0 = 0;
    while ((int32_t)(ld_acquire_sys(p) - val) < 0) {
        if ((++spins & 0xffu) == 0) {
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > c.timeout_ns) { report_failure(c, DEV_TIMEOUT, peer, site, seq); return false; }
            if ((spins & 0xfffu) == 0 && ld_volatile_u32(c.abort_word) != 0) { report_failure(c, DEV_ABORTED, peer, site, seq); return false; }
        }
    }
    return true;
}

/** `mask` selects the bits that count (a word may carry other information above its counter). */
__device__ __forceinline__ bool wait_flag64_ge(const DevComm& c, const unsigned long long* p, unsigned long long val, int peer, int site, uint32_t seq,
                                               unsigned long long mask = ~0ull) {
    uint32_t spins = 0;
    unsigned long long t0 = 0;
    while ((ld_acquire_sys64(p) & mask) < val) {
        if ((++spins & 0xffu) == 0) {
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > c.timeout_ns) { report_failure(c, DEV_TIMEOUT, peer, site, seq); return false; }
            if ((spins & 0xfffu) == 0 && ld_volatile_u32(c.abort_word) != 0) { report_failure(c, DEV_ABORTED, peer, site, seq); return false; }
        }
    }
    return true;
}

__device__ __forceinline__ uint32_t* flag_slot(char* pool, int cta, int src) {
    return reinterpret_cast<uint32_t*>(pool + kFlagOff) + (cta * kMaxPeers + src);
}
__device__ __forceinline__ uint32_t flag_value(uint32_t seq, int idx) { return seq * (uint32_t)kFlagVals + (uint32_t)idx; }

/** Tell `peer` that CTA `bid` of this rank has reached point `idx` of call `seq`.
 *  Call from ONE thread after a __syncthreads() that follows the CTA's data writes. */
__device__ __forceinline__ void signal_peer(const DevComm& c, int peer, int bid, uint32_t seq, int idx) {
    // the release store orders everything that happened before it, including the other threads' writes
    // that the preceding CTA barrier made visible to this thread; no separate fence is needed
    if (!DCCL_BOUNDS_OK(c, bid >= 0 && bid < kMaxCtas && peer >= 0 && peer < c.nranks && idx >= 0 && idx < kFlagVals, 1990, bid)) return;
    st_release_sys(flag_slot(c.pool[peer], bid, c.rank), flag_value(seq, idx));
}

/** Wait until CTA `bid` of rank `src` has signalled point `idx` of call `seq`. One thread. */
__device__ __forceinline__ bool wait_peer(const DevComm& c, int src, int bid, uint32_t seq, int idx, int site) {
    if (!DCCL_BOUNDS_OK(c, bid >= 0 && bid < kMaxCtas && src >= 0 && src < c.nranks && idx >= 0 && idx < kFlagVals, 1991, bid)) return false;
    return wait_flag_ge(c, flag_slot(c.pool[c.rank], bid, src), flag_value(seq, idx), src, site, seq);
}

/**
 * Barrier between the CTAs with index `bid` of all ranks. Every thread of the
 * CTA calls it. Data written by this CTA before the barrier is visible to the
 * same-index CTA of every peer after it. Returns false (for all threads) when a
 * wait gave up; the caller must then leave the kernel.
 */
__device__ __forceinline__ bool rank_barrier(const DevComm& c, int bid, uint32_t seq, int idx, int site) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    if ((int)threadIdx.x < c.nranks) {
        const int p = (int)threadIdx.x;
        signal_peer(c, p, bid, seq, idx);
        if (!wait_peer(c, p, bid, seq, idx, site)) s_fail = 1;
    }
    __syncthreads();
    return s_fail == 0;
}

/** thread 0 waits, everybody learns the outcome */
__device__ __forceinline__ bool cta_wait_peer(const DevComm& c, int src, int bid, uint32_t seq, int idx, int site) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = wait_peer(c, src, bid, seq, idx, site) ? 1 : 0;
    __syncthreads();
    const bool ok = s_ok != 0;
    __syncthreads();
    return ok;
}

/** all data writes of the CTA are done -> one thread publishes the flag */
__device__ __forceinline__ void cta_signal_peer(const DevComm& c, int peer, int bid, uint32_t seq, int idx) {
    __syncthreads();
    if (threadIdx.x == 0) signal_peer(c, peer, bid, seq, idx);
}

} // namespace dccl
