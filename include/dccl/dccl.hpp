/**
 * @file dccl.hpp
 * @brief Public API of the B200-native DCCL collective communication library.
 *
 * The names, enum values and call signatures follow the NCCL-compatible API of
 * the original DCCL (reference: include/dccl/dccl.hpp:59-474), so a client
 * written against that header compiles against this one. Everything lives in
 * namespace dccl, so the nccl* names never clash with a real libnccl that may
 * be loaded in the same process.
 *
 * What is different underneath: instead of a Derecho group over RDMA, a
 * communicator is a set of processes on ONE multi-GPU box. Host buffers are
 * reduced over POSIX shared memory; device buffers are reduced by sm_100a
 * kernels that read and write peer GPU memory over NVLink / NVSwitch
 * (plain peer loads/stores, or multimem.ld_reduce / multimem.st when the
 * switch supports in-fabric reduction).
 */
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#if defined(__CUDACC__) || defined(DCCL_WITH_CUDA_RUNTIME)
#include <cuda_runtime_api.h>
#else
/* Same definition the CUDA headers use; lets host-only clients compile. */
typedef struct CUstream_st* cudaStream_t;
#endif

#ifndef CACHELINE_SIZE
#define CACHELINE_SIZE 64
#endif
#ifndef CUDA_L1_CACHELINE_SIZE
#define CUDA_L1_CACHELINE_SIZE 128
#endif
#ifndef CUDA_L2_CACHELINE_SIZE
#define CUDA_L2_CACHELINE_SIZE 32
#endif
#ifndef ENABLE_EVALUATION
#define ENABLE_EVALUATION 1
#endif

/* Configuration keys (INI "SECTION/key" spelling, reference dccl.hpp:38-46). */
#define DCCL_ALLREDUCE_ALGORITHM_CONFSTR        "DCCL/allreduce_algorithm"
#define DCCL_REDUCESCATTER_ALGORITHM_CONFSTR    "DCCL/reducescatter_algorithm"
#define DCCL_ALLGATHER_ALGORITHM_CONFSTR        "DCCL/allgather_algorithm"
#define DCCL_ALLREDUCE_RING                     "ring"
#define DCCL_ALLREDUCE_RABENSEIFNER             "rabenseifner"
#define DCCL_ALLREDUCE_ONESHOT                  "oneshot"
#define DCCL_ALLREDUCE_TWOSHOT                  "twoshot"
#define DCCL_ALLREDUCE_NVLS                     "nvls"
#define DCCL_ALLREDUCE_AUTO                     "auto"

namespace dccl {

/** Error types (values identical to NCCL / reference dccl.hpp:59-67). */
typedef enum { ncclSuccess                 =  0,
               ncclUnhandledCudaError      =  1,
               ncclSystemError             =  2,
               ncclInternalError           =  3,
               ncclInvalidArgument         =  4,
               ncclInvalidUsage            =  5,
               ncclRemoteError             =  6,
               ncclInProgress              =  7,
               ncclNumResults              =  8 } ncclResult_t;

/** Data types. bfloat16 is always available in this build. */
typedef enum { ncclInt8       = 0, ncclChar       = 0,
               ncclUint8      = 1,
               ncclInt32      = 2, ncclInt        = 2,
               ncclUint32     = 3,
               ncclInt64      = 4,
               ncclUint64     = 5,
               ncclFloat16    = 6, ncclHalf       = 6,
               ncclFloat32    = 7, ncclFloat      = 7,
               ncclFloat64    = 8, ncclDouble     = 8,
               ncclBfloat16   = 9,
               ncclNumTypes   = 10 } ncclDataType_t;

typedef enum { ncclNumOps_dummy = 5 } ncclRedOp_dummy_t;

/** Reduction operators. All five are implemented for every data type. */
typedef enum { ncclSum        = 0,
               ncclProd       = 1,
               ncclMax        = 2,
               ncclMin        = 3,
               ncclAvg        = 4,
               ncclNumOps     = 5,
               ncclMaxRedOp   = 0x7fffffff>>(32-8*sizeof(ncclRedOp_dummy_t))
             } ncclRedOp_t;

struct dcclComm;
typedef struct dcclComm* ncclComm_t;

/** 128-byte rendezvous token, produced on rank 0 and handed to every rank. */
typedef struct { char internal[128]; } dcclUniqueId;

/* ------------------------------------------------------------------ *
 * Communicator life cycle
 * ------------------------------------------------------------------ */

/**
 * Create a communicator from the environment or from configuration files.
 * Rank / world size / rendezvous address are taken, in this order, from
 * DCCL_RANK, DCCL_WORLD_SIZE, DCCL_MASTER_ADDR, DCCL_MASTER_PORT; from the
 * torchrun variables RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT; or from a
 * derecho.cfg + layout.json pair in the working directory (local_id is the
 * rank, contact_ip/contact_port the rendezvous address, min_nodes_by_shard the
 * world size), which keeps the "cd cfg/n3 && dccl_cli ..." recipe of the
 * original working (reference dccl.cpp:287-332). Blocks until every rank joined.
 */
ncclResult_t  ncclCommInit(ncclComm_t* comm);

/** Produce a rendezvous token on the calling process (which becomes the server). */
ncclResult_t  dcclGetUniqueId(dcclUniqueId* id);

/** Explicit-argument variant of ncclCommInit, used by the PyTorch backend. */
ncclResult_t  dcclCommInitRank(ncclComm_t* comm, int nranks, dcclUniqueId id, int rank);

/** Leave the group and free every resource of the communicator. */
ncclResult_t  ncclCommFinalize(ncclComm_t comm);

/** Mark the communicator as failed: device waits and host waits return early. */
ncclResult_t  dcclCommAbort(ncclComm_t comm);

/**
 * Continue without the ranks that are gone (no counterpart in the original, which
 * leaves a failed group to time out). After a communicator has failed, every
 * surviving rank calls this; it returns a new communicator over the survivors,
 * ranks renumbered densely in the old order. Members are the ranks whose process
 * still exists and that were not the rank reported as failed. The old communicator
 * stays valid for dcclGetLastError and must still be finalized (that does not block).
 */
ncclResult_t  dcclCommShrink(ncclComm_t comm, ncclComm_t* newcomm);

/**
 * Report the asynchronous state of the communicator: ncclSuccess, or the error
 * that a kernel or the watchdog recorded (a peer that stopped answering is
 * ncclRemoteError). msg, when not null, receives a one-line description.
 */
ncclResult_t  dcclGetLastError(ncclComm_t comm, ncclResult_t* async_error, char* msg, size_t msg_len);

uint32_t dcclGetWorldSize(ncclComm_t comm);
uint32_t dcclGetMyRank(ncclComm_t comm);

/* ------------------------------------------------------------------ *
 * Memory
 * ------------------------------------------------------------------ */

/**
 * Register a user buffer (reference dccl.cpp:503-542). buffer and size must be
 * multiples of CACHELINE_SIZE, otherwise ncclInvalidArgument. Host memory needs
 * no mapping and is only checked. Device memory is exported to every peer
 * process so the kernels can read it in place; this variant is COLLECTIVE for
 * device memory: every rank must call it in the same order. An all-reduce whose
 * send and receive buffers both lie inside registered (or dcclMemAlloc) memory
 * may run without staging, peers folding the buffers directly; such a call must
 * use the same offset into the registered buffer on every rank.
 */
ncclResult_t  dcclRegisterCacheMemory(ncclComm_t comm, void* buffer, size_t size);
ncclResult_t  dcclDeregisterCacheMemory(ncclComm_t comm, void* buffer, size_t size = 0UL);

/**
 * Collective allocation of `size` bytes of symmetric device memory: every rank
 * gets a buffer that all peers can address and, where the NVSwitch supports it,
 * that is bound to a multicast object, so collectives on it run without any
 * staging copy. Every rank must call with the same size, in the same order.
 */
ncclResult_t  dcclMemAlloc(ncclComm_t comm, void** ptr, size_t size);
ncclResult_t  dcclMemFree(ncclComm_t comm, void* ptr);

/* ------------------------------------------------------------------ *
 * Collectives (stream-ordered for device buffers, blocking for host buffers)
 * ------------------------------------------------------------------ */

ncclResult_t  ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count,
    ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);

ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff,
    size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);

ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count,
    ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);

ncclResult_t ncclBcast(void* buff, size_t count,
    ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);

ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count,
    ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream);

ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount,
    ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);

ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t datatype,
    int peer, ncclComm_t comm, cudaStream_t stream);

ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer,
    ncclComm_t comm, cudaStream_t stream);

/**
 * Group several ncclSend / ncclRecv calls into one launch. Between Start and
 * End the calls are only recorded; End issues them together, so a ring in
 * which every rank sends before it receives cannot deadlock. On the device up
 * to 16 operations share one launch; a longer group runs as consecutive
 * launches of 16 in recording order, so the two ends of a transfer must fall
 * into the same batch (they do when all ranks record in matching order).
 */
ncclResult_t  dcclGroupStart();
ncclResult_t  dcclGroupEnd();

/**
 * Collectives composed of grouped send / recv (no counterpart in the original,
 * whose API stops at ncclSend / ncclRecv). Buffers are all on the host or all
 * on the device; device calls are ONE launch on `stream` plus a local copy of
 * the rank's own block.
 *   dcclAllToAll   block p (count elements) of sendbuff goes to rank p, block p of recvbuff comes from rank p
 *   dcclAllToAllv  the same with per-peer counts and displacements (in elements; arrays of world size)
 *   dcclGather     root receives count elements from every rank into block <rank> of recvbuff
 *   dcclScatter    root sends block p of sendbuff (count elements) to rank p's recvbuff
 * recvbuff (gather) and sendbuff (scatter) are only read on the root.
 */
ncclResult_t  dcclAllToAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
    ncclComm_t comm, cudaStream_t stream);
ncclResult_t  dcclAllToAllv(const void* sendbuff, const size_t* sendcounts, const size_t* sdispls,
    void* recvbuff, const size_t* recvcounts, const size_t* rdispls, ncclDataType_t datatype,
    ncclComm_t comm, cudaStream_t stream);
ncclResult_t  dcclGather(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root,
    ncclComm_t comm, cudaStream_t stream);
ncclResult_t  dcclScatter(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root,
    ncclComm_t comm, cudaStream_t stream);

/**
 * Force an algorithm for one collective ("allreduce", "reducescatter",
 * "allgather", "broadcast", "reduce") on this communicator. name is one of
 * auto, ring, rabenseifner, oneshot, twoshot, twoshot_ll, nvls. Unknown names give
 * ncclInvalidArgument; a variant that cannot serve a call (for example nvls
 * with ncclProd) falls back to the automatic choice for that call.
 */
ncclResult_t  dcclSetAlgorithm(ncclComm_t comm, const char* collective, const char* name);

/**
 * The box as the communicator found it, as one JSON object: per rank the GPU (name, PCI address, SMs, memory,
 * multicast support, NVLink links up and how many of them end in a switch; -1 where NVML was not available),
 * and the matrices "peer_access" / "peer_atomics" (1 yes, 0 no, 2 same GPU, 255 not visible to that process).
 * Needs the device side (ncclInvalidUsage before a device was bound). The text is cut to len - 1 characters.
 */
ncclResult_t  dcclGetTopology(ncclComm_t comm, char* json, size_t len);

/**
 * Host-side barrier over the control plane: returns when every rank of the communicator has called it (the
 * counterpart of the group barrier the original's tools take from Derecho, reference
 * src/application/p2p_perf.cpp:287). It does not wait for work queued on CUDA streams; synchronise the stream first
 * where that matters. ncclRemoteError when a rank failed or the group was aborted while waiting.
 */
ncclResult_t  dcclBarrier(ncclComm_t comm);

/**
 * Debug aid. With `DCCL/debug_bounds = 1` (DCCL_DEBUG_BOUNDS=1) the unused bytes between the regions of the
 * communicator's device pool hold guard words; this call reads them back and returns ncclInternalError when a
 * kernel wrote there (dcclGetLastError then says where). ncclSuccess when intact, when guarding is off and when
 * no device is bound. It waits for the device; it is also run at ncclCommFinalize. A library whose kernels were
 * compiled with -DDCCL_DEBUG_BOUNDS (make BOUNDS=1) additionally checks its pool ranges before it uses them and
 * reports a violation like a time-out, through dcclGetLastError.
 */
ncclResult_t  dcclDebugCheck(ncclComm_t comm);

/** Name of the variant the last call of `collective` used (for tools and tests). */
const char*   dcclGetLastAlgorithm(ncclComm_t comm, const char* collective);

/**
 * Tuning knob of the communicator's device side, for sweeps and tools: "ctas" (0: the table's value), "threads",
 * "unroll", "p2p_ctas", "p2p_rendezvous", "pipe_ctas", "pipe_nv_ctas", "pipe_teams", "pipe_unroll", "pipe_chunk_kb",
 * "pipe_min_mb", "rooted_pipe", "auto_register_min_kb" (0: no lazy registration), "direct_rs", "direct_rs_min_mb",
 * "direct_rooted" (zero-copy reduce / broadcast), "direct_rooted_ctas", "direct_bcast_ctas", "direct_bcast_min_kb",
 * "direct_reduce_small_worlds", "device_seq". Every rank sets the same value at the
 * same point of its call order. ncclInvalidArgument for an unknown name or a value out of range, ncclInvalidUsage
 * before a device was bound.
 */
ncclResult_t  dcclSetParam(ncclComm_t comm, const char* name, int value);

/** A counter of the device side: "launches" (kernels launched), "zero_copy_calls" (calls that peer kernels served
 *  straight out of / into user memory: symmetric, registered or lazily registered buffers). 0 for unknown names. */
unsigned long long dcclGetStat(ncclComm_t comm, const char* name);

const char*   dcclGetErrorString(ncclResult_t r);

/* ------------------------------------------------------------------ *
 * NCCL spellings of the calls above, for code written against NCCL
 * (the original stops at the names it implements; these are thin inline
 * aliases and add no behaviour).
 * ------------------------------------------------------------------ */
typedef dcclUniqueId ncclUniqueId;
inline ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { return dcclGetUniqueId(id); }
inline ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) { return dcclCommInitRank(comm, nranks, id, rank); }
inline ncclResult_t ncclCommDestroy(ncclComm_t comm) { return ncclCommFinalize(comm); }
inline ncclResult_t ncclCommAbort(ncclComm_t comm) { return dcclCommAbort(comm); }
inline ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) { if (!count) return ncclInvalidArgument; *count = (int)dcclGetWorldSize(comm); return ncclSuccess; }
inline ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) { if (!rank) return ncclInvalidArgument; *rank = (int)dcclGetMyRank(comm); return ncclSuccess; }
inline ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* async_error) { return dcclGetLastError(comm, async_error, nullptr, 0); }
inline const char*  ncclGetErrorString(ncclResult_t r) { return dcclGetErrorString(r); }
inline ncclResult_t ncclGroupStart() { return dcclGroupStart(); }
inline ncclResult_t ncclGroupEnd() { return dcclGroupEnd(); }
/* the composed collectives under the names NCCL 2.28 gives them */
inline ncclResult_t ncclAlltoAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream) {
    return dcclAllToAll(sendbuff, recvbuff, count, datatype, comm, stream);
}
inline ncclResult_t ncclGather(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    return dcclGather(sendbuff, recvbuff, count, datatype, root, comm, stream);
}
inline ncclResult_t ncclScatter(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    return dcclScatter(sendbuff, recvbuff, count, datatype, root, comm, stream);
}
/* registration: NCCL hands out a handle; here the buffer's address is the handle */
inline ncclResult_t ncclCommRegister(const ncclComm_t comm, void* buff, size_t size, void** handle) {
    const ncclResult_t r = dcclRegisterCacheMemory(comm, buff, size);
    if (handle) *handle = r == ncclSuccess ? buff : nullptr;
    return r;
}
inline ncclResult_t ncclCommDeregister(const ncclComm_t comm, void* handle) { return dcclDeregisterCacheMemory(comm, handle, 0); }

#define CACHELINE_OFFSET(addr)          ( ((uint64_t)(addr))%CACHELINE_SIZE)
#define CUDA_L1_CACHELINE_OFFSET(addr)  ( ((uint64_t)(addr))%CUDA_L1_CACHELINE_SIZE)
#define CUDA_L2_CACHELINE_OFFSET(addr)  ( ((uint64_t)(addr))%CUDA_L2_CACHELINE_SIZE)

#ifdef ENABLE_EVALUATION

/**
 * In-memory timestamp log (reference dccl.hpp:485-577, dccl.cpp:913-991).
 * An entry is four 64-bit words: tag, rank, extra, nanoseconds. flush() writes
 * the text format that the original tools produce:
 *
 *     # number of entries:<N>
 *     # tag rank extra tsns
 *     <tag> <rank> <extra> <ts_ns>
 *
 * The buffer is allocated on first use and grows on demand, so loading the
 * library costs nothing.
 */
class Timestamp {
private:
    uint64_t*   _log;
    size_t      capacity;
    size_t      position;
    volatile int lck;
    Timestamp(size_t num_entries = 0);
    void instance_log(uint64_t tag, uint64_t rank, uint64_t extra, uint64_t ts_ns);
    void instance_flush(const std::string& filename, bool clear);
    void instance_clear();
    size_t instance_size();
    static Timestamp _t;
public:
    virtual ~Timestamp();
    /** Nanosecond wall clock used for every entry. */
    static uint64_t now_ns();
    static inline void log(uint64_t tag, uint64_t rank, uint64_t extra = 0ull) {
        _t.instance_log(tag, rank, extra, now_ns());
    }
    /** Log with a caller-supplied time (device-side stamps converted to host time). */
    static inline void log_at(uint64_t tag, uint64_t rank, uint64_t extra, uint64_t ts_ns) {
        _t.instance_log(tag, rank, extra, ts_ns);
    }
    static inline void flush(const std::string& filename, bool clear = true) {
        _t.instance_flush(filename, clear);
    }
    static inline void clear() { _t.instance_clear(); }
    static inline size_t size() { return _t.instance_size(); }
};

#define     TT_DCCL(x)                      (1000000 + (x))
// overall
#define     TT_WARMUP_START                 TT_DCCL(1)
#define     TT_WARMUP_END                   TT_DCCL(2)
#define     TT_TEST_START                   TT_DCCL(3)
#define     TT_TEST_END                     TT_DCCL(4)
// all-reduce (same numbers as the original)
#define     TT_ALLREDUCE_ENTER              TT_DCCL(1001)
#define     TT_ALLREDUCE_MEMCPY             TT_DCCL(1020)
#define     TT_ALLREDUCE_RDH_PREPROCESS     TT_DCCL(1021)
#define     TT_ALLREDUCE_REDUCESCATTER      TT_DCCL(1030)
#define     TT_ALLREDUCE_ALLGATHER          TT_DCCL(1040)
#define     TT_ALLREDUCE_RDH_POSTPROCESS    TT_DCCL(1041)
#define     TT_ALLREDUCE_DONE               TT_DCCL(1100)
// the other entry points (new tags)
#define     TT_REDUCESCATTER_ENTER          TT_DCCL(2001)
#define     TT_REDUCESCATTER_DONE           TT_DCCL(2100)
#define     TT_ALLGATHER_ENTER              TT_DCCL(3001)
#define     TT_ALLGATHER_DONE               TT_DCCL(3100)
#define     TT_BROADCAST_ENTER              TT_DCCL(4001)
#define     TT_BROADCAST_DONE               TT_DCCL(4100)
#define     TT_REDUCE_ENTER                 TT_DCCL(5001)
#define     TT_REDUCE_DONE                  TT_DCCL(5100)
#define     TT_SEND_ENTER                   TT_DCCL(6001)
#define     TT_SEND_DONE                    TT_DCCL(6100)
#define     TT_RECV_ENTER                   TT_DCCL(7001)
#define     TT_RECV_DONE                    TT_DCCL(7100)
// device-side stamps (first CTA in / last CTA out, converted to host time)
#define     TT_DEVICE_KERNEL_BEGIN          TT_DCCL(9001)
#define     TT_DEVICE_KERNEL_END            TT_DCCL(9002)

#define TIMESTAMP(tag,rank,extra)           dccl::Timestamp::log(tag,rank,extra)
#define FLUSH_AND_CLEAR_TIMESTAMP(filename) dccl::Timestamp::flush(filename,true)
#define CLEAR_TIMESTAMP()                   dccl::Timestamp::clear()

#else
#define TIMESTAMP(tag,rank,extra)
#define FLUSH_AND_CLEAR_TIMESTAMP(filename)
#define CLEAR_TIMESTAMP()
#endif//ENABLE_EVALUATION

} // namespace dccl
