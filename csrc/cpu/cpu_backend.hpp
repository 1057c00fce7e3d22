/**
 * Host-buffer collectives over POSIX shared memory.
 *
 * This is the host half of the algorithm layer of the original (reference
 * src/core/algorithms.hpp:54-271 and the six algorithm files): ring
 * reduce-scatter / all-gather / all-reduce, recursive-halving reduce-scatter,
 * recursive-doubling all-gather and the Rabenseifner all-reduce with the
 * leader/follower step for world sizes that are not a power of two. The
 * zero-copy RDMA send/recv pair of each step becomes a pair of byte FIFOs in a
 * shared segment; the receiving side reduces straight out of the FIFO, so a
 * step needs no scratchpad. Any element count and any alignment is accepted.
 * Every wait is bounded (DCCL/timeout_ms, default 5000 ms like the original's
 * DCCL_OOB_TIMEOUT_US, reference internal_common.hpp:51-55) and also ends
 * when the group's abort word is set.
 */
#pragma once
#include "../bootstrap/bootstrap.hpp"
#include <vector>

namespace dccl {

enum HostAlgo { HOST_ALGO_RING = 0, HOST_ALGO_RABENSEIFNER = 1 };

class CpuBackend {
public:
    explicit CpuBackend(Bootstrap* bs);

    ncclResult_t all_reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, HostAlgo algo);
    ncclResult_t reduce_scatter(const void* send, void* recv, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op, HostAlgo algo);
    ncclResult_t all_gather(const void* send, void* recv, size_t sendcount, ncclDataType_t dt, HostAlgo algo);
    ncclResult_t broadcast(const void* send, void* recv, size_t count, ncclDataType_t dt, int root);
    ncclResult_t reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root);
    ncclResult_t send(const void* buf, size_t bytes, int peer);
    ncclResult_t recv(void* buf, size_t bytes, int peer);

    /** Between group_start and group_end, send/recv are queued and then progressed together. */
    void group_start() { group_depth_++; }
    ncclResult_t group_end();
    bool in_group() const { return group_depth_ > 0; }

    /* building blocks, public for the unit tests */
    ncclResult_t ring_reduce_scatter(char* buf, size_t count, ncclDataType_t dt, ncclRedOp_t op, int shift);
    ncclResult_t ring_all_gather(char* buf, size_t count, ncclDataType_t dt, int owner_shift);
    ncclResult_t halving_reduce_scatter(char* buf, size_t count, ncclDataType_t dt, ncclRedOp_t op,
                                        int vrank, int vworld, const std::vector<int>& v2r,
                                        std::vector<size_t>* lo_stack, std::vector<size_t>* hi_stack);
    ncclResult_t doubling_all_gather(char* buf, ncclDataType_t dt, int vrank, int vworld, const std::vector<int>& v2r,
                                     const std::vector<size_t>& lo_stack, const std::vector<size_t>& hi_stack);

    uint64_t bytes_sent() const { return bytes_sent_; }

private:
    struct Xfer {
        bool is_send;
        int peer;
        char* buf;
        size_t bytes;      // payload bytes
        size_t padded;     // FIFO bytes (payload rounded up to 16)
        size_t done;       // FIFO bytes moved so far
        bool reduce;
        ncclDataType_t dt;
        ncclRedOp_t op;
    };
    Xfer make_send(int peer, const void* buf, size_t bytes);
    Xfer make_recv(int peer, void* buf, size_t bytes);
    Xfer make_recv_reduce(int peer, void* buf, size_t bytes, ncclDataType_t dt, ncclRedOp_t op);
    bool step(Xfer& x);
    ncclResult_t progress(std::vector<Xfer>& xs);
    ncclResult_t sendrecv(Xfer s, Xfer r);
    ncclResult_t rabenseifner(char* buf, size_t count, ncclDataType_t dt, ncclRedOp_t op);
    char* scratch(size_t bytes, int which);

    Bootstrap* bs_;
    int rank_, world_;
    int timeout_ms_;
    int group_depth_ = 0;
    std::vector<Xfer> group_;
    std::vector<char> scratch_[2];
    uint64_t bytes_sent_ = 0;
};

} // namespace dccl
