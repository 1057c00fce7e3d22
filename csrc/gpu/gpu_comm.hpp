/**
 * Device side of a communicator: symmetric memory, peer mappings, multicast
 * objects and the launchers of the collective kernels.
 *
 * Where the original registers memory with the NIC and posts one RDMA
 * send/recv pair per algorithm step from the host (reference
 * src/core/internal_common.hpp:713-792, dccl.cpp:503-542), this class maps
 * every peer's pool into the local address space once, and each collective is
 * then ONE kernel launch on the caller's stream: all steps, the reduction, the
 * dtype handling and the 1/world scale run inside it, synchronised by flag
 * words in peer memory with bounded waits.
 */
#pragma once
#include <dccl/dccl.hpp>
#include "../bootstrap/bootstrap.hpp"
#include <string>

namespace dccl {

enum Collective { COLL_ALLREDUCE = 0, COLL_REDUCESCATTER, COLL_ALLGATHER, COLL_BROADCAST, COLL_REDUCE, COLL_SENDRECV, COLL_COUNT };

enum GpuAlgo { ALGO_AUTO = 0, ALGO_RING, ALGO_RABENSEIFNER, ALGO_ONESHOT, ALGO_TWOSHOT, ALGO_NVLS, ALGO_LOCAL, ALGO_TWOSHOT_LL, ALGO_COUNT };

const char* algo_name(GpuAlgo a);
/** Returns ALGO_COUNT for an unknown name. */
GpuAlgo parse_algo_name(const char* s);
int parse_collective_name(const char* s);

/** True when p is device memory of some CUDA device (false when CUDA is not usable at all). */
bool is_device_pointer(const void* p, int* device);
/** Number of usable CUDA devices; 0 on a machine without a driver. */
int cuda_device_count();

class GpuComm {
public:
    /** Collective over all ranks of bs: every rank calls it, each with its own device. */
    static GpuComm* create(Bootstrap* bs, int device, std::string* err);
    virtual ~GpuComm() {}

    virtual ncclResult_t all_reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op,
                                    GpuAlgo algo, cudaStream_t stream) = 0;
    virtual ncclResult_t reduce_scatter(const void* send, void* recv, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op,
                                        GpuAlgo algo, cudaStream_t stream) = 0;
    virtual ncclResult_t all_gather(const void* send, void* recv, size_t sendcount, ncclDataType_t dt,
                                    GpuAlgo algo, cudaStream_t stream) = 0;
    virtual ncclResult_t broadcast(const void* send, void* recv, size_t count, ncclDataType_t dt, int root,
                                   GpuAlgo algo, cudaStream_t stream) = 0;
    virtual ncclResult_t reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root,
                                GpuAlgo algo, cudaStream_t stream) = 0;
    virtual ncclResult_t send(const void* buf, size_t bytes, int peer, cudaStream_t stream) = 0;
    virtual ncclResult_t recv(void* buf, size_t bytes, int peer, cudaStream_t stream) = 0;
    virtual void group_start() = 0;
    virtual ncclResult_t group_end() = 0;
    /**
     * The group being recorded has the same `nops` operations on every rank (an all-to-all): its launch may use
     * fewer CTAs per operation so that all of them fit the GPU at once. Only valid when every rank says the same,
     * because both ends of a transfer must split it over the same number of CTAs. Forgotten at the next group end.
     */
    virtual void group_same_shape(int nops) = 0;
    /** dst = src on this device, stream ordered (the own block of all-to-all / gather / scatter). */
    virtual ncclResult_t local_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream) = 0;

    virtual ncclResult_t mem_alloc(void** ptr, size_t size) = 0;
    virtual ncclResult_t mem_free(void* ptr) = 0;
    virtual ncclResult_t register_buffer(void* buf, size_t size) = 0;
    virtual ncclResult_t deregister_buffer(void* buf) = 0;

    /** ncclSuccess, or the error a kernel recorded (timeout on a peer, abort). */
    virtual ncclResult_t async_error(char* msg, size_t msg_len) = 0;
    /** With `DCCL/debug_bounds = 1`: ncclInternalError (and where) when something wrote into the unused parts of
     *  this rank's pool; ncclSuccess otherwise and when guarding is off. Reads 32 KB from the device. */
    virtual ncclResult_t debug_check(char* msg, size_t msg_len) = 0;
    virtual void abort(int failed_rank) = 0;
    /** Wait until every kernel this rank launched has finished (called before peers unmap memory). */
    virtual void quiesce() = 0;
    virtual GpuAlgo last_algo(int coll) const = 0;
    virtual int device() const = 0;
    /** The GPUs of all ranks, the peer-access matrix and the NVLink / multicast facts, as JSON (topology.hpp). */
    virtual std::string topology() const = 0;
    virtual bool has_multicast() const = 0;
    /** Tuning knobs for sweeps: "ctas" (0 = table value), "threads" (128..512), "unroll" (2, 4, 8), ...;
     *  "device_seq" (0 / 1) moves the call sequence number between the host and a device counter, which is
     *  what makes captured launches replayable (collective: every rank switches at the same point). */
    virtual bool set_param(const char* name, int value) = 0;
    /** Kernels launched by this communicator so far. */
    virtual uint64_t launches() const = 0;
    /** True when [p, p + bytes) lies in symmetric memory of this communicator (dcclMemAlloc, or a memory pool served by it). */
    virtual bool is_symmetric(const void* p, size_t bytes) const = 0;
    /** Counters: "launches", "zero_copy_calls", "symmetric_calls" (calls served straight out of / into user memory by the peer kernels). */
    virtual uint64_t stat(const char* name) const = 0;
};

} // namespace dccl
