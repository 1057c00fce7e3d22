/**
 * nccl_cli: the same workload as dccl_cli, run through stock NVIDIA NCCL.
 *
 * The original ships an MPI twin of its benchmark tool as ground truth and
 * comparator (ompi_cli, reference src/application/cli.cpp:71-116,404-419);
 * on a single NVSwitch box the comparator is NCCL. libnccl is opened at run
 * time with dlopen ($DCCL_NCCL_LIB, then libnccl.so.2 from the loader path),
 * so this library never links against it. The NCCL unique id travels through
 * a host-buffer ncclBroadcast of THIS library, which is also what brings the
 * ranks together. Same options as dccl_cli (GPU buffers only, --gpu is
 * mandatory); timestamps go to nccl_cli.<rank>.tt.
 */
#include <dccl/dccl.hpp>
#include "tool_common.hpp"
#include <chrono>
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <getopt.h>
#include <iostream>

using namespace dccl_tools;

namespace stock {
typedef struct ncclComm* comm_t;
typedef struct { char internal[128]; } uid_t;
typedef int (*GetUniqueId_t)(uid_t*);
typedef int (*CommInitRank_t)(comm_t*, int, uid_t, int);
typedef int (*CommDestroy_t)(comm_t);
typedef int (*AllReduce_t)(const void*, void*, size_t, int, int, comm_t, cudaStream_t);
typedef int (*ReduceScatter_t)(const void*, void*, size_t, int, int, comm_t, cudaStream_t);
typedef int (*AllGather_t)(const void*, void*, size_t, int, comm_t, cudaStream_t);
typedef int (*Broadcast_t)(const void*, void*, size_t, int, int, comm_t, cudaStream_t);
typedef int (*Reduce_t)(const void*, void*, size_t, int, int, int, comm_t, cudaStream_t);
typedef int (*GetVersion_t)(int*);
}

int main(int argc, char** argv) {
    static struct option long_options[] = {
        {"api", required_argument, 0, 'a'}, {"gpu", required_argument, 0, 'g'}, {"warmup", required_argument, 0, 'w'},
        {"repeat", required_argument, 0, 'r'}, {"type", required_argument, 0, 't'}, {"op", required_argument, 0, 'o'},
        {"count", required_argument, 0, 'c'}, {"verify", no_argument, 0, 'v'}, {"init", required_argument, 0, 'i'},
        {"seed", required_argument, 0, 'S'}, {"help", no_argument, 0, 'h'}, {0, 0, 0, 0}};
    std::string api;
    int gpu = -1;
    size_t warmup = 0, repeat = 1000, count = 1024;
    dccl::ncclDataType_t dt = dccl::ncclUint32;
    dccl::ncclRedOp_t op = dccl::ncclSum;
    bool verify = false;
    InitMode init = INIT_BYTES;
    uint64_t seed = 0;
    while (true) {
        int idx = 0;
        int c = getopt_long(argc, argv, "a:g:w:r:t:o:c:vi:S:h", long_options, &idx);
        if (c == -1) break;
        switch (c) {
        case 'a': api = optarg; break;
        case 'g': gpu = !strcmp(optarg, "auto") ? -2 : std::stoi(optarg); break;
        case 'w': warmup = std::stoul(optarg); break;
        case 'r': repeat = std::stoul(optarg); break;
        case 't': dt = parse_type_name(optarg); break;
        case 'o': op = parse_op_name(optarg); break;
        case 'c': count = std::stoul(optarg); break;
        case 'v': verify = true; break;
        case 'i': init = !strcmp(optarg, "uniform") ? INIT_UNIFORM : !strcmp(optarg, "normal") ? INIT_NORMAL : INIT_BYTES; break;
        case 'S': seed = std::stoull(optarg); break;
        default: std::cout << "options: --api --gpu --warmup --repeat --type --op --count --verify --init --seed" << std::endl; return 0;
        }
    }
    if (api.empty() || (gpu < 0 && gpu != -2) || dt == dccl::ncclNumTypes || op == dccl::ncclNumOps) {
        std::cerr << "nccl_cli needs --api, --gpu and valid --type / --op" << std::endl;
        return -1;
    }
    const char* libname = getenv("DCCL_NCCL_LIB");
    void* h = dlopen(libname && *libname ? libname : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) { std::cerr << "cannot open libnccl: " << dlerror() << " (set DCCL_NCCL_LIB)" << std::endl; return 5; }
#define SYM(T, name) stock::T name = (stock::T)dlsym(h, #name); if (!name) { std::cerr << "libnccl lacks " #name << std::endl; return 5; }
    SYM(GetUniqueId_t, ncclGetUniqueId) SYM(CommInitRank_t, ncclCommInitRank) SYM(CommDestroy_t, ncclCommDestroy)
    SYM(AllReduce_t, ncclAllReduce) SYM(ReduceScatter_t, ncclReduceScatter) SYM(AllGather_t, ncclAllGather)
    SYM(Broadcast_t, ncclBroadcast) SYM(Reduce_t, ncclReduce) SYM(GetVersion_t, ncclGetVersion)
#undef SYM
    int version = 0;
    ncclGetVersion(&version);
    std::cout << "nccl api evaluation with the following configuration:" << std::endl;
    std::cout << "\tapi:" << api << "\n\tgpu:" << gpu << "\n\twarmup:" << warmup << "\n\trepeat:" << repeat << "\n\ttype:" << dt
              << "\n\top:" << op << "\n\tcount:" << count << "\n\tnccl:" << version << std::endl;

    // rendezvous through this library's host path
    dccl::ncclComm_t boot;
    if (dccl::ncclCommInit(&boot) != dccl::ncclSuccess) { std::cerr << "failed to initialize the bootstrap communicator." << std::endl; return 1; }
    const int rank = (int)dccl::dcclGetMyRank(boot), world = (int)dccl::dcclGetWorldSize(boot);
    if (gpu == -2) {
        const char* e = getenv("DCCL_LOCAL_DEVICE");
        if (!e || !*e) e = getenv("LOCAL_RANK");
        gpu = e && *e ? atoi(e) : rank;
    }
    if (cudaSetDevice(gpu) != cudaSuccess) { std::cerr << "cudaSetDevice failed" << std::endl; return 4; }
    stock::uid_t id;
    memset(&id, 0, sizeof(id));
    if (rank == 0 && ncclGetUniqueId(&id) != 0) { std::cerr << "ncclGetUniqueId failed" << std::endl; return 1; }
    if (dccl::ncclBroadcast(&id, &id, sizeof(id), dccl::ncclUint8, 0, boot, nullptr) != dccl::ncclSuccess) return 1;
    stock::comm_t comm;
    if (ncclCommInitRank(&comm, world, id, rank) != 0) { std::cerr << "ncclCommInitRank failed" << std::endl; return 1; }

    if ((api == "reduce_scatter" || api == "all_gather") && count % (size_t)world) { std::cerr << "count must be a multiple of the world size" << std::endl; return 1; }
    const size_t es = size_of_type(dt), bytes = count * es, slot = count / (size_t)world, slot_bytes = slot * es;
    std::vector<char> host(bytes);
    fill_buffer(host.data(), count, dt, init, seed + (uint64_t)rank, rank);
    char *sendbuf = nullptr, *recvbuf = nullptr;
    cudaStream_t stream;
    if (cudaMalloc((void**)&sendbuf, bytes + 256) != cudaSuccess || cudaMalloc((void**)&recvbuf, bytes + 256) != cudaSuccess || cudaStreamCreate(&stream) != cudaSuccess) return 4;
    cudaMemcpy(sendbuf, host.data(), bytes, cudaMemcpyHostToDevice);
    cudaMemset(recvbuf, rank, bytes);
    // NCCL's enums share the values of this library's for the types and operators used here
    auto run_once = [&]() -> int {
        if (api == "all_reduce") return ncclAllReduce(sendbuf, verify ? recvbuf : sendbuf, count, dt, op, comm, stream);
        if (api == "reduce_scatter") return ncclReduceScatter(sendbuf, verify ? recvbuf : sendbuf + rank * slot_bytes, slot, dt, op, comm, stream);
        if (api == "all_gather") return ncclAllGather(sendbuf + rank * slot_bytes, verify ? recvbuf : sendbuf, slot, dt, comm, stream);
        if (api == "reduce") return ncclReduce(sendbuf, verify ? recvbuf : sendbuf, count, dt, op, 0, comm, stream);
        if (api == "broadcast") return ncclBroadcast(sendbuf, recvbuf, count, dt, 0, comm, stream);
        return 4;
    };
    std::cout << "warm up..." << std::endl;
    TIMESTAMP(TT_WARMUP_START, rank, 0);
    for (size_t i = 0; i < warmup; i++) if (run_once() != 0) { std::cerr << "API:" << api << " failed" << std::endl; return 2; }
    cudaStreamSynchronize(stream);
    TIMESTAMP(TT_WARMUP_END, rank, 0);
    std::cout << "done." << std::endl << "run test..." << std::endl;
    auto t0 = std::chrono::steady_clock::now();
    TIMESTAMP(TT_TEST_START, rank, 0);
    for (size_t i = 0; i < repeat; i++) {
        TIMESTAMP(TT_ALLREDUCE_ENTER, rank, 0);
        if (run_once() != 0) { std::cerr << "API:" << api << " failed" << std::endl; return 2; }
        TIMESTAMP(TT_ALLREDUCE_DONE, rank, 0);
    }
    cudaStreamSynchronize(stream);
    TIMESTAMP(TT_TEST_END, rank, 0);
    auto t1 = std::chrono::steady_clock::now();
    std::cout << "done." << std::endl;
    if (repeat) {
        double us = std::chrono::duration<double, std::micro>(t1 - t0).count() / (double)repeat, n = world;
        double alg = (double)bytes / (us * 1e-6) / 1e9, f = api == "all_reduce" ? 2 * (n - 1) / n : (api == "reduce_scatter" || api == "all_gather") ? (n - 1) / n : 1.0;
        printf("avg latency: %.2f us   algbw: %.3f GB/s   busbw: %.3f GB/s\n", us, alg, world > 1 ? alg * f : alg);
    }
    int failed = 0;
    if (verify && api == "all_reduce") {
        std::vector<std::vector<char>> all((size_t)world, std::vector<char>(bytes));
        for (int r = 0; r < world; r++) fill_buffer(all[(size_t)r].data(), count, dt, init, seed + (uint64_t)r, r);
        std::vector<char> want(bytes), got(bytes);
        reference_fold(all, count, dt, op, want.data());
        cudaMemcpy(got.data(), recvbuf, bytes, cudaMemcpyDeviceToHost);
        size_t bad = compare_buffers(got.data(), want.data(), count, dt, world, api.c_str());
        if (bad) { std::cerr << "verify: " << bad << " elements differ" << std::endl; failed = 1; }
        else std::cout << "verify: ok (" << count << " elements)" << std::endl;
    }
    std::cout << "flush timestamp..." << std::endl;
    FLUSH_AND_CLEAR_TIMESTAMP("nccl_cli." + std::to_string(rank) + ".tt");
    std::cout << "...done" << std::endl;
    ncclCommDestroy(comm);
    cudaFree(sendbuf);
    cudaFree(recvbuf);
    dccl::ncclCommFinalize(boot);
    return failed ? 3 : 0;
}
