/**
 * Host-callable launchers of the collective kernels. One launch = one whole
 * collective (all algorithm steps of reference src/core/algorithms.hpp run
 * inside the kernel). `ranks_in_launch` > 1 means single-GPU emulation: the
 * grid is ranks x ctas and is launched cooperatively so every CTA is resident.
 */
#pragma once
#include "../device/prims.cuh"
#include <dccl/dccl.hpp>

namespace dccl {

struct LaunchCfg {
    int ctas = 32;               // CTAs per rank
    int threads = 512;
    cudaStream_t stream = nullptr;
    int ranks_in_launch = 1;     // > 1: emulation, cooperative launch
};

/* twoshot.cu: staging-based peer-to-peer variants */
enum { TS_ALLREDUCE = 0, TS_REDUCESCATTER, TS_ALLGATHER, TS_BROADCAST, TS_BROADCAST_DIRECT, TS_REDUCE };
/** Elements one launch can take for `mode` with n ranks and the given staging half. */
size_t twoshot_capacity(int mode, int nranks, size_t elem_size, size_t stage_bytes);
cudaError_t launch_twoshot(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);

/* direct.cu: zero-copy peer all-reduce (io.send_peer / io.recv_peer hold every rank's buffers, 16-byte aligned) and
 * reduce-scatter (io.send_peer, io.recv; count = per-rank elements, stride = slot distance, slots 16-byte aligned) */
enum { DIRECT_ALLREDUCE = 0, DIRECT_REDUCESCATTER, DIRECT_REDUCE };
cudaError_t launch_direct(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);
/* zero-copy broadcast of `bytes` bytes from a.root (io.send_peer[root], io.recv_peer[*], all 16-byte aligned): scatter and
 * all-gather by peer loads, pipelined in `chunks` chunks per shard (0: direct_bcast_chunks(), about 1 MB each, at most 24) */
int direct_bcast_chunks(size_t bytes, int nranks);
cudaError_t launch_direct_bcast(const CollArgs& a, size_t bytes, int nranks, const LaunchCfg& cfg, int chunks = 0);

/* oneshot_ll.cu: flag-in-data all-reduce for small messages */
size_t oneshot_ll_capacity_bytes();
cudaError_t launch_oneshot_ll(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);

/* ll_twoshot.cu: two-shot all-reduce on packets (shard to its owner, folded shard to everybody), no barrier;
 * LL2_REDUCE sends the folded shards to a.root only */
enum { LL2_ALLREDUCE = 0, LL2_REDUCE };
size_t ll_twoshot_capacity_bytes(int nranks);
cudaError_t launch_ll_twoshot(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);

/* ll_collectives.cu: flag-in-data reduce-scatter / all-gather / broadcast / reduce for small messages;
 * count = per-rank elements, at most oneshot_ll_capacity_bytes() per rank */
enum { LL_REDUCESCATTER = 0, LL_ALLGATHER, LL_BROADCAST, LL_REDUCE };
cudaError_t launch_ll_collective(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);

/* nvls.cu: in-switch reduction / multicast variants */
enum { NV_ALLREDUCE = 0, NV_REDUCESCATTER, NV_ALLGATHER, NV_BROADCAST, NV_REDUCE };
bool nvls_supports(ncclDataType_t dt, ncclRedOp_t op);
size_t nvls_capacity(int mode, int nranks, size_t elem_size, size_t stage_bytes);
cudaError_t launch_nvls(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);

/* nvls_pipe.cu: all-reduce / reduce-scatter of ordinary buffers with copy-in, switch pass and copy-out overlapped
 * chunk by chunk (reduce-scatter: count = per-rank elements, stride = slot distance in the send buffer). The staging
 * half (stage_bytes) is a ring of chunk slots, so ONE launch takes a message of any length; chunk numbers beyond the flag
 * values of one call use nvls_pipe_extra_seqs() further call numbers, which the caller must skip after the launch.
 * nvls_pipe_capacity is the largest message that needs no further call numbers and no slot twice (the limit when
 * sequence numbers are counted on the device). */
size_t nvls_pipe_capacity(size_t elem_size, size_t stage_bytes, int nranks, bool reduce_scatter);
int nvls_pipe_extra_seqs(size_t count, size_t elem_size, size_t stage_bytes, int nranks, bool reduce_scatter, bool single_seq = false);
/** cfg.ctas is the whole grid; nv_ctas of it form the switch group (0: a fifth / a third of the grid), the rest is
 *  split evenly between copy-in and copy-out (all-reduce) or is the copy-in group (reduce-scatter). The switch CTAs
 *  form `teams` teams that take the chunks in turn. single_seq: the message is at most nvls_pipe_capacity and must not
 *  use further call numbers (sequence numbers counted on the device). */
cudaError_t launch_nvls_pipe(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg, bool reduce_scatter, size_t stage_bytes, int nv_ctas = 0, int teams = 2,
                             bool single_seq = false);
/** Target chunk size of the pipeline (default 8 MB, at most 24 chunks per launch); a tuning knob, the same on every rank. */
void nvls_pipe_set_chunk_bytes(size_t bytes);

/* nvls_rooted.cu: broadcast / reduce of large ordinary buffers through the switch with the local copies overlapped
 * chunk by chunk (count elements, at most nvls_pipe_capacity(..., false); root in a.root) */
enum { ROOTED_BROADCAST = 0, ROOTED_REDUCE };
cudaError_t launch_nvls_rooted(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);

/* ring.cu / hd.cu: the two algorithms of the original as single kernels */
enum { RING_ALLREDUCE = 0, RING_REDUCESCATTER, RING_ALLGATHER };
size_t ring_capacity(int mode, int nranks, size_t elem_size, size_t stage_bytes);
cudaError_t launch_ring(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);
size_t hd_capacity(int nranks, size_t elem_size, size_t stage_bytes);
cudaError_t launch_hd(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg);

/* local.cu: one-rank paths (copy, scale) and a pairwise reduce */
cudaError_t launch_local_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream);
cudaError_t launch_local_reduce(void* acc, const void* in, size_t count, ncclDataType_t dt, ncclRedOp_t op, cudaStream_t stream);

/* p2p.cu: send / recv. Small messages go through the per-pair FIFOs; a large message is written straight into the
 * receiver's buffer when the sender has that buffer mapped (rendezvous), else through the FIFO as well. */
enum { P2P_DST_NONE = 0,     // the receive buffer cannot be reached by peers: FIFO
       P2P_DST_SYM = 1,      // it lies in symmetric memory: (segment number, offset)
       P2P_DST_IPC = 2 };    // it lies in an exported allocation: (base address at the owner, buffer id, offset)
struct P2pOp {
    int is_send;
    int peer;
    char* buf;
    size_t bytes;
    unsigned long long chunk_base;   // chunks already moved on this (peer, direction) before this op
    int rdv;                         // 1: a large message: sender and receiver meet before data moves
    int dst_kind;                    // receives only: where the buffer lies (P2P_DST_*)
    unsigned long long rdv_index;    // large messages on this (peer, direction) before this op
    unsigned long long dst_a, dst_id, dst_off;   // receives only: segment number or base address, buffer id, offset
};
/** What a sender knows about a peer's memory: where a segment / allocation of `peer` is mapped in this process. */
struct P2pMap {
    int peer;
    int kind;                        // P2P_DST_SYM or P2P_DST_IPC
    unsigned long long a, id;        // segment number, or base address at the owner and buffer id
    unsigned long long size;
    char* mapped;
};
constexpr int kMaxP2pOps = 16;
constexpr int kMaxP2pMaps = 24;
constexpr size_t kP2pRdvMinBytes = 512u << 10;   // messages from this size on are rendezvous messages (both ends know the size)
struct P2pArgs {
    DevComm comm;
    const DevComm* emu;              // emulation: array of per-rank DevComm
    const P2pOp* emu_ops;            // emulation: [ranks][kMaxP2pOps]
    const int* emu_nops;
    int ctas_per_op;
    int ctas_per_rank;
    int nops;
    int nmaps;
    P2pOp ops[kMaxP2pOps];
    P2pMap maps[kMaxP2pMaps];        // the mappings of the peers this launch sends to (most recent first)
};
cudaError_t launch_p2p(const P2pArgs& a, const LaunchCfg& cfg);
inline size_t p2p_chunks(size_t bytes) { return (bytes + kP2pChunk - 1) / kP2pChunk; }

/* bounded-wait self test: waits on a flag nobody sets, must come back with a timeout status */
cudaError_t launch_wait_probe(const DevComm& c, cudaStream_t stream);

#ifdef DCCL_HOST_SIM
/** Host simulation: the launch runs every CUDA thread as an OS thread and returns when the kernel has finished.
 *  DCCL_SIM_THREADS (default 8, at least the world size) replaces the block size; the kernels take any. */
template <typename A>
inline cudaError_t launch_kernel(void (*kernel)(const A), const void* args_struct, const LaunchCfg& cfg) {
    struct Call { void (*k)(const A); const A* a; };
    Call call{kernel, static_cast<const A*>(args_struct)};
    const char* e = getenv("DCCL_SIM_THREADS");
    int threads = e ? atoi(e) : 8;
    if (threads < 8) threads = 8;
    if (threads > cfg.threads) threads = cfg.threads;
    ::dccl_sim::launch([](const void* p) { const Call* c = static_cast<const Call*>(p); c->k(*c->a); }, &call,
                       (unsigned)(cfg.ctas * cfg.ranks_in_launch), (unsigned)threads);
    return cudaSuccess;
}
#else
template <typename K>
inline cudaError_t launch_kernel(K kernel, const void* args_struct, const LaunchCfg& cfg) {
    void* params[] = {const_cast<void*>(args_struct)};
    dim3 grid((unsigned)(cfg.ctas * cfg.ranks_in_launch)), block((unsigned)cfg.threads);
    if (cfg.ranks_in_launch > 1) return cudaLaunchCooperativeKernel((const void*)kernel, grid, block, params, 0, cfg.stream);
    return cudaLaunchKernel((const void*)kernel, grid, block, params, 0, cfg.stream);
}
#endif

/** Launch a collective kernel; fixes up the CTA count per rank that the kernel derives its ranges from. */
template <typename K>
inline cudaError_t launch_coll(K kernel, CollArgs a, const LaunchCfg& cfg) {
    a.ctas_per_rank = cfg.ctas;
    return launch_kernel(kernel, &a, cfg);
}

} // namespace dccl
