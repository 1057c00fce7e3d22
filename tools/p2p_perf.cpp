/**
 * p2p_perf: windowed point-to-point throughput between rank 0 (sender) and
 * rank 1 (receiver).
 *
 * Same options, banner and timestamp tags as the original tool (reference
 * src/application/p2p_perf.cpp:14-22,302-419), whose transport was Derecho's
 * OOB RDMA. Here the transport is this library's ncclSend / ncclRecv: "p2p"
 * (alias "oob") moves GPU buffers with the peer-copy kernels over NVLink, or
 * host buffers through shared memory when no --cuda device is given. A window
 * of --depth messages is issued as one group; the sender logs TT_OOB_SEND per
 * message and TT_OOB_ACKD per completed window. The last window carries 0xFF
 * bytes so the receiver can tell a complete run, as in the original. Ranks
 * other than 0 and 1 only join and leave. Timestamps go to oob.dat.
 */
#include <dccl/dccl.hpp>
#include "tool_common.hpp"
#include <chrono>
#include <cstdlib>
#include <getopt.h>
#include <iostream>
#include <vector>
#ifdef DCCL_WITH_CUDA
#include <cuda_runtime_api.h>
#endif

using namespace dccl;

#define TT_OOB(x)               (2000000 + (x))
#define TT_OOB_WARMUP_START     TT_OOB(1)
#define TT_OOB_WARMUP_END       TT_OOB(2)
#define TT_OOB_TEST_START       TT_OOB(3)
#define TT_OOB_TEST_END         TT_OOB(4)
#define TT_OOB_SEND             TT_OOB(1001)
#define TT_OOB_ACKD             TT_OOB(1002)

static const char* help_string =
    "  -t, --transport NAME  (required) how the messages travel: p2p (the library's send / recv; 'oob' is accepted\n"
    "                        as another spelling)\n"
#ifdef DCCL_WITH_CUDA
    "  -c, --cuda DEV        keep the message pool in device memory of GPU DEV (default: host memory)\n"
#endif
    "  -s, --size BYTES      bytes per message (default 1024)\n"
    "  -d, --depth N         messages in flight before the sender waits for the oldest (default 16)\n"
    "  -w, --warmup SEC      seconds of untimed traffic first (default 1)\n"
    "  -D, --duration SEC    seconds of measured traffic (default 5)\n"
    "  -h, --help            show this text\n";

static void print_help(const char* cmd) {
    std::cout << "Usage: " << cmd << " [options]" << std::endl;
    std::cout << help_string << std::endl;
}

static double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    static struct option long_options[] = {
        {"transport", required_argument, 0, 't'}, {"cuda", required_argument, 0, 'c'}, {"size", required_argument, 0, 's'},
        {"depth", required_argument, 0, 'd'}, {"warmup", required_argument, 0, 'w'}, {"duration", required_argument, 0, 'D'},
        {"help", no_argument, 0, 'h'}, {0, 0, 0, 0}};
    std::string transport;
    int cuda_dev = -1;
    size_t size_byte = 1024, depth = 16;
    double warmup_sec = 1, duration_sec = 5;
    while (true) {
        int idx = 0;
        int c = getopt_long(argc, argv, "t:c:s:d:w:D:h", long_options, &idx);
        if (c == -1) break;
        switch (c) {
        case 't': transport = optarg; break;
        case 'c': cuda_dev = std::stoi(optarg); break;
        case 's': size_byte = std::stoul(optarg); break;
        case 'd': depth = std::stoul(optarg); break;
        case 'w': warmup_sec = std::stod(optarg); break;
        case 'D': duration_sec = std::stod(optarg); break;
        case 'h': print_help(argv[0]); return 0;
        default: break;
        }
    }
    if (transport.empty()) {
        std::cerr << "Error:--transport,-t argument is required." << std::endl;
        print_help(argv[0]);
        return 1;
    }
    if (transport != "oob" && transport != "p2p") {
        std::cerr << "Error: transport must be one of 'p2p' and 'oob'." << std::endl;
        print_help(argv[0]);
        return 2;
    }
    if (depth < 1) depth = 1;
    if (depth > 8) depth = 8;   // one launch carries at most 16 operations
#ifndef DCCL_WITH_CUDA
    cuda_dev = -1;
#endif
    std::cout << "Evaluating transport performance with the following configuration:" << std::endl;
    std::cout << "\ttransport:  " << transport << std::endl;
#ifdef DCCL_WITH_CUDA
    std::cout << "\tcuda dev:   " << cuda_dev << std::endl;
#endif
    std::cout << "\tsize:       " << size_byte << std::endl;
    std::cout << "\tdepth:      " << depth << std::endl;
    std::cout << "\twarmup:     " << warmup_sec << std::endl;
    std::cout << "\tduration:   " << duration_sec << std::endl;

    ncclComm_t comm;
    if (ncclCommInit(&comm) != ncclSuccess) { std::cerr << "failed to initialize the dccl communicator." << std::endl; return 1; }
    const uint32_t rank = dcclGetMyRank(comm), world = dcclGetWorldSize(comm);
    if (world < 2) { std::cerr << "p2p_perf needs at least two ranks." << std::endl; ncclCommFinalize(comm); return 1; }

    // a pool of `depth` message buffers
    char* pool = nullptr;
    cudaStream_t stream = nullptr;
    const size_t pool_bytes = size_byte * depth;
    if (cuda_dev < 0) {
        void* p = nullptr;
        if (posix_memalign(&p, 4096, pool_bytes + 4096)) return 1;
        pool = (char*)p;
        memset(pool, (int)rank, pool_bytes);
    }
#ifdef DCCL_WITH_CUDA
    else {
        if (cudaSetDevice(cuda_dev) != cudaSuccess || cudaMalloc((void**)&pool, pool_bytes + 4096) != cudaSuccess || cudaStreamCreate(&stream) != cudaSuccess) {
            std::cerr << "cannot set up cuda device " << cuda_dev << std::endl;
            return 1;
        }
        cudaMemset(pool, (int)rank, pool_bytes);
    }
#endif
    // a device pool has to exist on every rank before rank 0 and 1 start talking
    dcclRegisterCacheMemory(comm, pool, (pool_bytes + CACHELINE_SIZE - 1) / CACHELINE_SIZE * CACHELINE_SIZE);

    auto fill = [&](int v) {
        if (cuda_dev < 0) memset(pool, v, pool_bytes);
#ifdef DCCL_WITH_CUDA
        else { cudaMemsetAsync(pool, v, pool_bytes, stream); }
#endif
    };
    auto first_byte = [&]() -> int {
        unsigned char b = 0;
        if (cuda_dev < 0) b = (unsigned char)pool[pool_bytes - 1];
#ifdef DCCL_WITH_CUDA
        else { cudaStreamSynchronize(stream); cudaMemcpy(&b, pool + pool_bytes - 1, 1, cudaMemcpyDeviceToHost); }
#endif
        return b;
    };
    auto window = [&](bool sender) -> ncclResult_t {
        dcclGroupStart();
        ncclResult_t r = ncclSuccess;
        for (size_t i = 0; i < depth && r == ncclSuccess; i++) {
            if (sender) { TIMESTAMP(TT_OOB_SEND, rank, i); r = ncclSend(pool + i * size_byte, size_byte, ncclUint8, 1, comm, stream); }
            else r = ncclRecv(pool + i * size_byte, size_byte, ncclUint8, 0, comm, stream);
        }
        ncclResult_t e = dcclGroupEnd();
        if (r == ncclSuccess) r = e;
#ifdef DCCL_WITH_CUDA
        if (cuda_dev >= 0) cudaStreamSynchronize(stream);
#endif
        if (sender) TIMESTAMP(TT_OOB_ACKD, rank, depth);
        return r;
    };

    int rc = 0;
    if (rank == 0) {
        size_t windows = 0;
        for (int phase = 0; phase < 2 && rc == 0; phase++) {
            const double len = phase == 0 ? warmup_sec : duration_sec;
            TIMESTAMP(phase == 0 ? TT_OOB_WARMUP_START : TT_OOB_TEST_START, rank, 0);
            const double t0 = now_s();
            windows = 0;
            while (now_s() - t0 < len) {
                if (window(true) != ncclSuccess) { rc = 2; break; }
                windows++;
            }
            const double dt = now_s() - t0;
            TIMESTAMP(phase == 0 ? TT_OOB_WARMUP_END : TT_OOB_TEST_END, rank, windows);
            if (phase == 1 && rc == 0) {
                const double bytes = (double)windows * (double)depth * (double)size_byte;
                printf("sent %zu messages of %zu bytes in %.3f s: %.3f GB/s, %.2f us per message\n", windows * depth, size_byte, dt,
                       bytes / dt / 1e9, dt / (double)(windows * depth > 0 ? windows * depth : 1) * 1e6);
            }
        }
        // the terminating window
        fill(0xFF);
        if (rc == 0 && window(true) != ncclSuccess) rc = 2;
    } else if (rank == 1) {
        size_t windows = 0;
        while (rc == 0) {
            if (window(false) != ncclSuccess) { rc = 2; break; }
            windows++;
            if (first_byte() == 0xFF) break;
        }
        printf("received %zu windows\n", windows);
    }
    ncclResult_t async = ncclSuccess;
    char msg[200];
    dcclGetLastError(comm, &async, msg, sizeof(msg));
    if (async != ncclSuccess) { std::cerr << "transport error: " << msg << std::endl; rc = 2; }
    dcclDeregisterCacheMemory(comm, pool);
    FLUSH_AND_CLEAR_TIMESTAMP("oob.dat");
    ncclCommFinalize(comm);
    if (cuda_dev < 0) free(pool);
#ifdef DCCL_WITH_CUDA
    else cudaFree(pool);
#endif
    return rc;
}
