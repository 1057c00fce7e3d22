/**
 * Smallest client of the library: join, report world size and rank, leave.
 * Same program as the original's example (reference examples/helloworld/main.cpp:7-19);
 * start one process per rank, e.g.
 *   for r in 0 1 2 3; do DCCL_RANK=$r DCCL_WORLD_SIZE=4 ./helloworld & done
 * or from configuration directories (cd cfg/n<r> && helloworld).
 */
#include <dccl/dccl.hpp>
#include <iostream>

using namespace dccl;

int main(int, char**) {
    ncclComm_t comm;
    ncclResult_t ret = ncclCommInit(&comm);
    if (ret != ncclSuccess) {
        std::cerr << "failed to initialize the dccl communicator, error: " << ret << std::endl;
        return 1;
    }
    std::cout << "DCCL communicator initialized: world size = " << dcclGetWorldSize(comm)
              << ", my rank = " << dcclGetMyRank(comm) << std::endl;
    ret = ncclCommFinalize(comm);
    if (ret != ncclSuccess) {
        std::cerr << "failed to finalize the dccl communicator, error: " << ret << std::endl;
        return 1;
    }
    return 0;
}
