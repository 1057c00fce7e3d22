/** The communicator object behind ncclComm_t (counterpart of dcclComm in the
 *  original, reference src/core/internal_common.hpp:126-247). */
#pragma once
#include <dccl/dccl.hpp>
#include "../bootstrap/bootstrap.hpp"
#include "../cpu/cpu_backend.hpp"
#include "../gpu/gpu_comm.hpp"
#include <mutex>
#include <string>

namespace dccl {

struct dcclComm {
    Bootstrap bs;
    CpuBackend* cpu = nullptr;
    GpuComm* gpu = nullptr;
    bool gpu_failed = false;
    std::mutex mu;
    GpuAlgo algo[COLL_COUNT];
    HostAlgo last_host_algo[COLL_COUNT];
    bool last_was_host[COLL_COUNT];
    ncclResult_t host_error = ncclSuccess;
    std::string host_error_msg;
    // counters reported at finalize (log level info)
    uint64_t calls[COLL_COUNT] = {0, 0, 0, 0, 0, 0};
    uint64_t bytes[COLL_COUNT] = {0, 0, 0, 0, 0, 0};
};

/** Bind the device side of the communicator on first use (collective: every rank gets here with its first device call). */
ncclResult_t ensure_gpu(dcclComm* c, int device);

} // namespace dccl
