/**
 * dccl_cli: benchmark / validation tool for every API entry point.
 *
 * Same options, defaults, banner, phase lines, exit codes and output files as
 * the original tool (reference src/application/cli.cpp:51-69,190-557):
 * sendbuf is byte-filled with the rank, the test runs in place, --save writes
 * hex dumps, timestamps go to dccl_cli.tt. Operator names are parsed
 * correctly. Additions: bfloat16, --verify (out-of-place run checked against
 * a serial fold of every rank's seeded input), --init / --seed, --algo,
 * --tt-per-rank, --root, and a latency / bandwidth summary line.
 */
#include <dccl/dccl.hpp>
#include "tool_common.hpp"
#include <chrono>
#include <cerrno>
#include <cstdlib>
#include <getopt.h>
#include <iostream>
#include <string>
#include <unistd.h>
#ifdef DCCL_WITH_CUDA
#include <cuda_runtime_api.h>
#endif

using namespace dccl;
using namespace dccl_tools;

static const char* help_string =
    "  -a, --api NAME      (required) the call to run: all_reduce, reduce_scatter, all_gather, broadcast, reduce,\n"
    "                      send, recv; added here: all_to_all, gather, scatter.\n"
    "                      send / recv run between ranks 0 and 1 only; broadcast sends from, and reduce collects at,\n"
    "                      the root rank (--root, 0 by default).\n"
#ifdef DCCL_WITH_CUDA
    "  -g, --gpu DEV       run on device memory of GPU DEV ('auto': the launcher's local device, else the rank);\n"
    "                      without this option the buffers are host memory.\n"
#endif
    "  -w, --warmup N      untimed calls before the measurement (default 0)\n"
    "  -r, --repeat N      timed calls (default 1000)\n"
    "  -t, --type T        element type (default uint32): int8 uint8 int32 uint32 int64 uint64 float16 float32\n"
    "                      float64 bfloat16\n"
    "  -o, --op OP         reduction (default sum): sum prod max min avg\n"
    "  -c, --count N       elements per buffer (default 1024)\n"
    "  -s, --save          dump the buffers before and after the run as hex text files next to the .tt file\n"
    "  -v, --verify        run out of place and compare with a serial fold; exit code 3 when they differ\n"
    "  -i, --init KIND     buffer contents: bytes (every byte = rank, the default), uniform, normal\n"
    "  -S, --seed N        seed of uniform / normal data; rank r draws from seed N + r (default 0)\n"
    "  -A, --algo NAME     force a variant: auto ring rabenseifner oneshot twoshot twoshot_ll nvls\n"
    "  -R, --root RANK     root of broadcast / reduce (default 0)\n"
    "      --tt-per-rank   name the timestamp file dccl_cli.<rank>.tt (for ranks that share a directory)\n"
    "  -h, --help          show this text\n";

static void print_help(const char* cmd) {
    std::cout << "Usage: " << cmd << " [options]" << std::endl;
    std::cout << help_string << std::endl;
}

#ifdef DCCL_WITH_CUDA
#define ASSERTRT(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    std::cerr << "cuda error " << cudaGetErrorString(e_) << " at " << __FILE__ << ":" << __LINE__ << std::endl; return 4; } } while (0)
static int save_cuda_mem(const void* ptr, size_t size, const std::string& fname) {
    std::vector<char> h(size);
    ASSERTRT(cudaMemcpy(h.data(), ptr, size, cudaMemcpyDeviceToHost));
    save_mem(h.data(), size, fname);
    return 0;
}
#endif

int main(int argc, char** argv) {
    static struct option long_options[] = {
        {"api", required_argument, 0, 'a'}, {"gpu", required_argument, 0, 'g'}, {"warmup", required_argument, 0, 'w'},
        {"repeat", required_argument, 0, 'r'}, {"type", required_argument, 0, 't'}, {"op", required_argument, 0, 'o'},
        {"count", required_argument, 0, 'c'}, {"save", no_argument, 0, 's'}, {"help", no_argument, 0, 'h'},
        {"verify", no_argument, 0, 'v'}, {"init", required_argument, 0, 'i'}, {"seed", required_argument, 0, 'S'},
        {"algo", required_argument, 0, 'A'}, {"root", required_argument, 0, 'R'}, {"tt-per-rank", no_argument, 0, 1000},
        {0, 0, 0, 0}};
    std::string api, algo;
    int gpu = -1, root = 0;
    size_t warmup_count = 0, repeat_count = 1000, data_count = 1024;
    ncclDataType_t data_type = ncclUint32;
    ncclRedOp_t operation = ncclSum;
    bool save = false, verify = false, tt_per_rank = false;
    InitMode init = INIT_BYTES;
    uint64_t seed = 0;

    while (true) {
        int idx = 0;
        int c = getopt_long(argc, argv, "a:g:w:r:t:o:c:shvi:S:A:R:", long_options, &idx);
        if (c == -1) break;
        switch (c) {
        case 'a': api = optarg; break;
        case 'g': gpu = !strcmp(optarg, "auto") ? -2 : std::stoi(optarg); break;
        case 'w': warmup_count = std::stoul(optarg); break;
        case 'r': repeat_count = std::stoul(optarg); break;
        case 't':
            data_type = parse_type_name(optarg);
            if (data_type == ncclNumTypes) { std::cerr << "Unknown data type:" << optarg << " falling back to 'uint8'" << std::endl; data_type = ncclUint8; }
            break;
        case 'o':
            operation = parse_op_name(optarg);
            if (operation == ncclNumOps) { std::cerr << "Unknown operation:" << optarg << " falling back to 'sum'" << std::endl; operation = ncclSum; }
            break;
        case 'c': data_count = std::stoul(optarg); break;
        case 's': save = true; break;
        case 'v': verify = true; break;
        case 'i':
            if (!strcmp(optarg, "uniform")) init = INIT_UNIFORM;
            else if (!strcmp(optarg, "normal")) init = INIT_NORMAL;
            else init = INIT_BYTES;
            break;
        case 'S': seed = std::stoull(optarg); break;
        case 'A': algo = optarg; break;
        case 'R': root = std::stoi(optarg); break;
        case 1000: tt_per_rank = true; break;
        case 'h': print_help(argv[0]); return 0;
        default: break;
        }
    }
    if (api.empty()) { print_help(argv[0]); return -1; }
#ifndef DCCL_WITH_CUDA
    if (gpu >= 0) { std::cerr << "this build has no CUDA support; --gpu ignored" << std::endl; gpu = -1; }
#endif

    std::cout << "dccl api evaluation with the following configuration:" << std::endl;
    std::cout << "\tapi:" << api << std::endl;
#ifdef DCCL_WITH_CUDA
    std::cout << "\tgpu:" << gpu << "\t(CPU == -1)" << std::endl;
#endif
    std::cout << "\twarmup:" << warmup_count << std::endl;
    std::cout << "\trepeat:" << repeat_count << std::endl;
    std::cout << "\ttype:" << data_type << std::endl;
    std::cout << "\top:" << operation << std::endl;
    std::cout << "\tcount:" << data_count << std::endl;

    // join the group
    ncclComm_t comm;
    ncclResult_t ret = ncclCommInit(&comm);
    if (ret != ncclSuccess) { std::cerr << "failed to initialize the dccl communicator." << std::endl; return 1; }
    const uint32_t my_rank = dcclGetMyRank(comm), world_size = dcclGetWorldSize(comm);
    if (gpu == -2) {   // --gpu auto: the launcher's local device, else the rank
        const char* e = getenv("DCCL_LOCAL_DEVICE");
        if (!e || !*e) e = getenv("LOCAL_RANK");
        gpu = e && *e ? atoi(e) : (int)my_rank;
    }
    if (!algo.empty()) {
        const char* colls[] = {"allreduce", "reducescatter", "allgather", "broadcast", "reduce"};
        for (const char* c : colls)
            if (dcclSetAlgorithm(comm, c, algo.c_str()) != ncclSuccess) { std::cerr << "unknown algorithm:" << algo << std::endl; ncclCommFinalize(comm); return 1; }
    }
    const bool composed = api == "all_to_all" || api == "gather" || api == "scatter";
    if ((api == "reduce_scatter" || api == "all_gather" || composed) && data_count % world_size) {
        std::cerr << "count must be a multiple of the world size (" << world_size << ") for " << api << std::endl;
        ncclCommFinalize(comm);
        return 1;
    }

    // allocate and fill the buffers
    const size_t data_size = size_of_type(data_type), bytes = data_count * data_size;
    void *raw_send = nullptr, *raw_recv = nullptr, *sendbuf = nullptr, *recvbuf = nullptr;
    cudaStream_t stream = nullptr;
    std::vector<char> host_init(bytes);
    fill_buffer(host_init.data(), data_count, data_type, init, seed + my_rank, (int)my_rank);
    if (gpu < 0) {
        if (posix_memalign(&raw_send, CACHELINE_SIZE, bytes + CACHELINE_SIZE) || posix_memalign(&raw_recv, CACHELINE_SIZE, bytes + CACHELINE_SIZE)) {
            std::cerr << "Failed to allocate " << (bytes + CACHELINE_SIZE) << " bytes" << std::endl;
            std::cerr << "Error:" << std::strerror(errno) << std::endl;
            ncclCommFinalize(comm);
            return 1;
        }
        sendbuf = raw_send; recvbuf = raw_recv;
        memcpy(sendbuf, host_init.data(), bytes);
        memset(recvbuf, (int)(my_rank + 128), bytes);
        if (save) save_mem(sendbuf, bytes, "sendbuf.host.before.txt");
    }
#ifdef DCCL_WITH_CUDA
    else {
        ASSERTRT(cudaSetDevice(gpu));
        ASSERTRT(cudaMalloc(&raw_send, bytes + CUDA_L1_CACHELINE_SIZE));
        ASSERTRT(cudaMalloc(&raw_recv, bytes + CUDA_L1_CACHELINE_SIZE));
        ASSERTRT(cudaStreamCreate(&stream));
        sendbuf = raw_send; recvbuf = raw_recv;   // cudaMalloc returns 256-byte aligned memory
        ASSERTRT(cudaMemcpy(sendbuf, host_init.data(), bytes, cudaMemcpyHostToDevice));
        ASSERTRT(cudaMemset(recvbuf, (int)my_rank, bytes));
        if (save && save_cuda_mem(sendbuf, bytes, "sendbuf.cuda.before.txt")) return 4;
    }
#endif
    // registration wants whole cache lines
    const size_t reg_bytes = (bytes + CACHELINE_SIZE - 1) / CACHELINE_SIZE * CACHELINE_SIZE;
    if (dcclRegisterCacheMemory(comm, sendbuf, reg_bytes) != ncclSuccess) {
        std::cerr << "Failed to register sendbuf@" << sendbuf << "to dccl." << std::endl;
        return 1;
    }
    if (api == "broadcast" || verify || composed) {
        if (dcclRegisterCacheMemory(comm, recvbuf, reg_bytes) != ncclSuccess) {
            std::cerr << "Failed to register recvbuf@" << recvbuf << "to dccl." << std::endl;
            return 1;
        }
    }

    const size_t slot_count = data_count / world_size, slot_bytes = slot_count * data_size;
    auto at = [](void* p, size_t off) { return (void*)((uintptr_t)p + off); };
    auto run_once = [&]() -> ncclResult_t {
        if (api == "all_reduce") return ncclAllReduce(sendbuf, verify ? recvbuf : sendbuf, data_count, data_type, operation, comm, stream);
        if (api == "reduce_scatter")
            return ncclReduceScatter(sendbuf, verify ? recvbuf : at(sendbuf, my_rank * slot_bytes), slot_count, data_type, operation, comm, stream);
        if (api == "all_gather")
            return ncclAllGather(at(sendbuf, my_rank * slot_bytes), verify ? recvbuf : sendbuf, slot_count, data_type, comm, stream);
        if (api == "reduce") return ncclReduce(sendbuf, verify ? recvbuf : sendbuf, data_count, data_type, operation, root, comm, stream);
        if (api == "broadcast") return ncclBroadcast(sendbuf, recvbuf, data_count, data_type, root, comm, stream);
        if (api == "all_to_all") return dcclAllToAll(sendbuf, recvbuf, slot_count, data_type, comm, stream);
        if (api == "gather") return dcclGather(at(sendbuf, my_rank * slot_bytes), recvbuf, slot_count, data_type, root, comm, stream);
        if (api == "scatter") return dcclScatter(sendbuf, recvbuf, slot_count, data_type, root, comm, stream);
        if (api == "send") return my_rank < 2 ? ncclSend(sendbuf, data_count, data_type, 1 - (int)my_rank, comm, stream) : ncclSuccess;
        if (api == "recv") return my_rank < 2 ? ncclRecv(verify ? recvbuf : sendbuf, data_count, data_type, 1 - (int)my_rank, comm, stream) : ncclSuccess;
        return ncclInvalidArgument;
    };
    auto sync = [&]() {
#ifdef DCCL_WITH_CUDA
        if (gpu >= 0) cudaStreamSynchronize(stream);
#endif
    };
    // per-call wall time (meaningful for host buffers, where a call returns when the data is there;
    // for device buffers it is the launch cost and the summary line reports the stream time instead)
    double call_min_us = 1e300, call_max_us = 0.0;
#define RUN_WITH_COUNTER(cnt) \
    for (size_t i_ = 0; i_ < (cnt); i_++) { \
        auto c0_ = std::chrono::steady_clock::now(); \
        ret = run_once(); \
        double d_ = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - c0_).count(); \
        if (d_ < call_min_us) call_min_us = d_; \
        if (d_ > call_max_us) call_max_us = d_; \
        if (ret != ncclSuccess) { \
            std::cerr << "API:" << api << " failed with error:" << ret << std::endl; \
            ncclCommFinalize(comm); \
            if (gpu < 0) { free(raw_send); free(raw_recv); } \
            return 2; \
        } \
    }

    // untimed calls
    std::cout << "warm up..." << std::endl;
    TIMESTAMP(TT_WARMUP_START, my_rank, 0);
    RUN_WITH_COUNTER(warmup_count);
    sync();
    TIMESTAMP(TT_WARMUP_END, my_rank, 0);
    std::cout << "done." << std::endl;

    // the measurement
    std::cout << "run test..." << std::endl;
    call_min_us = 1e300; call_max_us = 0.0;   // forget the warm-up calls
    auto t0 = std::chrono::steady_clock::now();
    TIMESTAMP(TT_TEST_START, my_rank, 0);
    RUN_WITH_COUNTER(repeat_count);
    sync();
    TIMESTAMP(TT_TEST_END, my_rank, 0);
    auto t1 = std::chrono::steady_clock::now();
    std::cout << "done." << std::endl;
    if (repeat_count) {
        double us = std::chrono::duration<double, std::micro>(t1 - t0).count() / (double)repeat_count;
        double n = world_size, alg = (double)bytes / (us * 1e-6) / 1e9, factor = 1.0;
        if (api == "all_reduce") factor = 2.0 * (n - 1) / n;
        else if (api == "reduce_scatter" || api == "all_gather") factor = (n - 1) / n;
        char line[256];
        snprintf(line, sizeof(line), "avg latency: %.2f us   algbw: %.3f GB/s   busbw: %.3f GB/s   algorithm: %s", us, alg,
                 alg * (world_size > 1 ? factor : 1.0),
                 dcclGetLastAlgorithm(comm, api == "all_reduce" ? "allreduce" : api == "reduce_scatter" ? "reducescatter"
                                          : api == "all_gather" ? "allgather" : api == "broadcast" ? "broadcast"
                                          : api == "reduce" ? "reduce" : "sendrecv"));
        std::cout << line << std::endl;
        snprintf(line, sizeof(line), "%s per call: min %.2f us   max %.2f us", gpu < 0 ? "latency" : "launch cost", call_min_us, call_max_us);
        std::cout << line << std::endl;
    }
    {
        ncclResult_t async = ncclSuccess;
        char msg[256];
        dcclGetLastError(comm, &async, msg, sizeof(msg));
        if (async != ncclSuccess) {
            std::cerr << "API:" << api << " failed with error:" << async << " (" << msg << ")" << std::endl;
            ncclCommFinalize(comm);
            return 2;
        }
    }

    // optional check against a serial fold of what every rank put in
    int verify_failed = 0;
    if (verify) {
        std::vector<std::vector<char>> all(world_size, std::vector<char>(bytes));
        for (uint32_t r = 0; r < world_size; r++) fill_buffer(all[r].data(), data_count, data_type, init, seed + r, (int)r);
        std::vector<char> want(bytes), got(bytes);
        size_t check_count = 0, want_off = 0;
        bool have = true;
        if (api == "all_reduce") { reference_fold(all, data_count, data_type, operation, want.data()); check_count = data_count; }
        else if (api == "reduce") { reference_fold(all, data_count, data_type, operation, want.data()); check_count = data_count; have = (int)my_rank == root; }
        else if (api == "reduce_scatter") { reference_fold(all, data_count, data_type, operation, want.data()); check_count = slot_count; want_off = my_rank * slot_bytes; }
        else if (api == "all_gather") { for (uint32_t r = 0; r < world_size; r++) memcpy(want.data() + r * slot_bytes, all[r].data() + r * slot_bytes, slot_bytes); check_count = slot_count * world_size; }
        else if (api == "broadcast") { want = all[root]; check_count = data_count; }
        else if (api == "all_to_all") { for (uint32_t r = 0; r < world_size; r++) memcpy(want.data() + r * slot_bytes, all[r].data() + my_rank * slot_bytes, slot_bytes); check_count = slot_count * world_size; }
        else if (api == "gather") { for (uint32_t r = 0; r < world_size; r++) memcpy(want.data() + r * slot_bytes, all[r].data() + r * slot_bytes, slot_bytes); check_count = slot_count * world_size; have = (int)my_rank == root; }
        else if (api == "scatter") { memcpy(want.data(), all[root].data() + my_rank * slot_bytes, slot_bytes); check_count = slot_count; }
        else if (api == "recv") { if (my_rank < 2) want = all[1 - my_rank]; else have = false; check_count = data_count; }
        else have = false;
        if (have) {
            if (gpu < 0) memcpy(got.data(), recvbuf, check_count * data_size);
#ifdef DCCL_WITH_CUDA
            else ASSERTRT(cudaMemcpy(got.data(), recvbuf, check_count * data_size, cudaMemcpyDeviceToHost));
#endif
            size_t bad = compare_buffers(got.data(), want.data() + want_off, check_count, data_type, (int)world_size, api.c_str());
            if (bad) { std::cerr << "verify: " << bad << " of " << check_count << " elements differ on rank " << my_rank << std::endl; verify_failed = 1; }
            else std::cout << "verify: ok (" << check_count << " elements)" << std::endl;
        }
    }

    if (dcclDeregisterCacheMemory(comm, sendbuf) != ncclSuccess) std::cerr << "Failed to deregister sendbuf@" << sendbuf << "from dccl." << std::endl;
    if (api == "broadcast" || verify || composed)
        if (dcclDeregisterCacheMemory(comm, recvbuf) != ncclSuccess) std::cerr << "Failed to deregister recvbuf@" << recvbuf << "from dccl." << std::endl;
    if (gpu < 0) {
        if (save) { save_mem(recvbuf, bytes, "recvbuf.host.txt"); save_mem(sendbuf, bytes, "sendbuf.host.after.txt"); }
        free(raw_send); free(raw_recv);
    }
#ifdef DCCL_WITH_CUDA
    else {
        if (save) { if (save_cuda_mem(recvbuf, bytes, "recvbuf.cuda.txt") || save_cuda_mem(sendbuf, bytes, "sendbuf.cuda.after.txt")) return 4; }
        ASSERTRT(cudaFree(raw_send));
        ASSERTRT(cudaFree(raw_recv));
    }
#endif

    // write the timestamp log
    std::cout << "flush timestamp..." << std::endl;
    FLUSH_AND_CLEAR_TIMESTAMP(tt_per_rank ? "dccl_cli." + std::to_string(my_rank) + ".tt" : std::string("dccl_cli.tt"));
    std::cout << "...done" << std::endl;

    // leave the group
    ret = ncclCommFinalize(comm);
    if (ret != ncclSuccess) std::cerr << "failed to finalize the dccl communicator." << std::endl;
    return verify_failed ? 3 : 0;
}
