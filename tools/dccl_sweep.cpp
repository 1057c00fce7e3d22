/**
 * dccl_sweep: bus-bandwidth / latency sweep of all-reduce, reduce-scatter and
 * all-gather over message sizes, for this library and for stock NCCL in the
 * same process, with no interpreter in the timed loop.
 *
 * Single-box counterpart of the original's cluster sweep scripts (IMB-MT
 * all-reduce over 4 KB - 1 GB, reference scripts/mpi-benchmarks/run_by_sizes.sh:3-27,
 * and the DCCL-vs-OpenMPI runs of scripts/azure/run_dccl.sh, run_ompi.sh).
 * One process per GPU (DCCL_RANK / DCCL_WORLD_SIZE or torchrun variables).
 * Every point: 5 warm-up calls, then K calls between two CUDA events on the
 * stream, after a host barrier; the time reported is the maximum over ranks.
 * busBW follows nccl-tests: all-reduce algBW*2(n-1)/n, reduce-scatter and
 * all-gather algBW*(n-1)/n, with S the full vector.
 *
 *   --gpu N|auto  --min BYTES --max BYTES --factor F  --type bfloat16|float32|...
 *   --colls all_reduce,reduce_scatter,all_gather  --impls dccl,nccl
 *   --algo NAME (force a variant of this library)  --symmetric (dcclMemAlloc buffers)
 *   --register (ordinary cudaMalloc buffers registered with dcclRegisterCacheMemory)
 *   --param NAME=VALUE (a tuning knob of this library's device side, repeatable: pipe_ctas=96, direct_rs=1, ...)
 *   --nccl-register (the NCCL arm runs on ncclMemAlloc memory registered with ncclCommRegister: NCCL's own
 *                    zero-copy path, the like-for-like partner of --symmetric)
 *   --grid "NAME=V1:V2;NAME2=W1:W2" (the whole sweep once per combination of these parameter values, in one process;
 *                    the combination is appended to the variant column)
 *   --colls also takes broadcast and reduce (root 0; S = the message)
 *   --out FILE (rank 0 writes the rows as JSON)
 */
#include <dccl/dccl.hpp>
#include "tool_common.hpp"
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <getopt.h>
#include <iostream>
#include <sstream>

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
typedef int (*MemAlloc_t)(void**, size_t);
typedef int (*MemFree_t)(void*);
typedef int (*CommRegister_t)(comm_t, void*, size_t, void**);
typedef int (*CommDeregister_t)(comm_t, void*);
}

static std::vector<std::string> split(const std::string& s) {
    std::vector<std::string> out;
    std::stringstream ss(s);
    std::string item;
    while (std::getline(ss, item, ',')) if (!item.empty()) out.push_back(item);
    return out;
}

static size_t parse_size(const char* s) {
    char* end = nullptr;
    unsigned long long v = strtoull(s, &end, 0);
    if (*end == 'k' || *end == 'K') v <<= 10;
    else if (*end == 'm' || *end == 'M') v <<= 20;
    else if (*end == 'g' || *end == 'G') v <<= 30;
    return (size_t)v;
}

int main(int argc, char** argv) {
    static struct option long_options[] = {
        {"gpu", required_argument, 0, 'g'}, {"min", required_argument, 0, 'm'}, {"max", required_argument, 0, 'M'},
        {"factor", required_argument, 0, 'f'}, {"type", required_argument, 0, 't'}, {"colls", required_argument, 0, 'c'},
        {"impls", required_argument, 0, 'i'}, {"algo", required_argument, 0, 'A'}, {"symmetric", no_argument, 0, 's'},
        {"out", required_argument, 0, 'o'}, {"op", required_argument, 0, 'O'}, {"register", no_argument, 0, 'R'},
        {"param", required_argument, 0, 'p'}, {"nccl-register", no_argument, 0, 'N'}, {"grid", required_argument, 0, 'G'}, {0, 0, 0, 0}};
    int gpu = -2;
    size_t minb = 1024, maxb = 1ull << 30, factor = 2;
    dccl::ncclDataType_t dt = dccl::ncclBfloat16;
    dccl::ncclRedOp_t op = dccl::ncclSum;
    std::string colls = "all_reduce,reduce_scatter,all_gather", impls = "dccl,nccl", algo, out;
    bool symmetric = false, registered = false, nccl_registered = false;
    std::vector<std::pair<std::string, int>> params;
    std::vector<std::pair<std::string, std::vector<int>>> grid;
    while (true) {
        int idx = 0;
        int c = getopt_long(argc, argv, "g:m:M:f:t:c:i:A:so:O:Rp:NG:", long_options, &idx);
        if (c == -1) break;
        switch (c) {
        case 'g': gpu = !strcmp(optarg, "auto") ? -2 : atoi(optarg); break;
        case 'm': minb = parse_size(optarg); break;
        case 'M': maxb = parse_size(optarg); break;
        case 'f': factor = (size_t)atoi(optarg); break;
        case 't': dt = parse_type_name(optarg); break;
        case 'c': colls = optarg; break;
        case 'i': impls = optarg; break;
        case 'A': algo = optarg; break;
        case 's': symmetric = true; break;
        case 'R': registered = true; break;
        case 'N': nccl_registered = true; break;
        case 'G': {
            std::stringstream gs(optarg);
            std::string item;
            while (std::getline(gs, item, ';')) {
                const size_t eq = item.find('=');
                if (eq == std::string::npos) { std::cerr << "--grid wants NAME=V1:V2;..." << std::endl; return 1; }
                std::vector<int> vals;
                std::stringstream vs(item.substr(eq + 1));
                std::string v;
                while (std::getline(vs, v, ':')) if (!v.empty()) vals.push_back(atoi(v.c_str()));
                if (vals.empty()) { std::cerr << "--grid: no values for " << item << std::endl; return 1; }
                grid.emplace_back(item.substr(0, eq), vals);
            }
            break;
        }
        case 'p': {
            const char* eq = strchr(optarg, '=');
            if (!eq) { std::cerr << "--param wants NAME=VALUE" << std::endl; return 1; }
            params.emplace_back(std::string(optarg, eq - optarg), atoi(eq + 1));
            break;
        }
        case 'o': out = optarg; break;
        case 'O': op = parse_op_name(optarg); break;
        default: break;
        }
    }
    if (dt == dccl::ncclNumTypes || op == dccl::ncclNumOps || factor < 2) { std::cerr << "bad --type / --op / --factor" << std::endl; return 1; }

    dccl::ncclComm_t comm;
    if (dccl::ncclCommInit(&comm) != dccl::ncclSuccess) { std::cerr << "failed to initialize the dccl communicator." << std::endl; return 1; }
    const int rank = (int)dccl::dcclGetMyRank(comm), world = (int)dccl::dcclGetWorldSize(comm);
    if (gpu == -2) {
        const char* e = getenv("DCCL_LOCAL_DEVICE");
        if (!e || !*e) e = getenv("LOCAL_RANK");
        gpu = e && *e ? atoi(e) : rank;
    }
    if (cudaSetDevice(gpu) != cudaSuccess) { std::cerr << "cudaSetDevice failed" << std::endl; return 4; }
    cudaStream_t stream;
    cudaStreamCreate(&stream);
    const size_t es = size_of_type(dt);

    // buffers: one pair for this library (optionally symmetric), one ordinary pair for NCCL
    char *s_ours = nullptr, *r_ours = nullptr, *s_nccl = nullptr, *r_nccl = nullptr;
    const bool want_dccl = impls.find("dccl") != std::string::npos, want_nccl = impls.find("nccl") != std::string::npos;
    if (want_dccl) {
        // any device call binds the device side; a tiny all-reduce does it collectively
        cudaMalloc((void**)&s_ours, 256);
        if (dccl::ncclAllReduce(s_ours, s_ours, 1, dccl::ncclFloat32, dccl::ncclSum, comm, stream) != dccl::ncclSuccess) return 2;
        cudaStreamSynchronize(stream);
        cudaFree(s_ours);
        if (symmetric && world > 1) {
            if (dccl::dcclMemAlloc(comm, (void**)&s_ours, maxb) != dccl::ncclSuccess || dccl::dcclMemAlloc(comm, (void**)&r_ours, maxb) != dccl::ncclSuccess) return 2;
        } else {
            symmetric = false;
            if (cudaMalloc((void**)&s_ours, maxb) != cudaSuccess || cudaMalloc((void**)&r_ours, maxb) != cudaSuccess) return 4;
            // --register: ordinary allocations that every rank maps (cudaIpc), the zero-copy peer variants can use them
            if (registered && (dccl::dcclRegisterCacheMemory(comm, s_ours, maxb) != dccl::ncclSuccess ||
                               dccl::dcclRegisterCacheMemory(comm, r_ours, maxb) != dccl::ncclSuccess)) return 2;
        }
        cudaMemset(s_ours, 0, maxb);
        for (const auto& kv : params)
            if (dccl::dcclSetParam(comm, kv.first.c_str(), kv.second) != dccl::ncclSuccess) { std::cerr << "unknown parameter " << kv.first << std::endl; return 1; }
        if (!algo.empty())
            for (const char* c : {"allreduce", "reducescatter", "allgather", "broadcast", "reduce"})
                if (dccl::dcclSetAlgorithm(comm, c, algo.c_str()) != dccl::ncclSuccess) { std::cerr << "unknown algorithm" << std::endl; return 1; }
    }
    stock::comm_t ncomm = nullptr;
    stock::AllReduce_t nAllReduce = nullptr;
    stock::ReduceScatter_t nReduceScatter = nullptr;
    stock::AllGather_t nAllGather = nullptr;
    stock::CommDestroy_t nDestroy = nullptr;
    stock::Broadcast_t nBroadcast = nullptr;
    stock::Reduce_t nReduce = nullptr;
    stock::MemFree_t nMemFree = nullptr;
    stock::CommDeregister_t nDeregister = nullptr;
    void *reg_s = nullptr, *reg_r = nullptr;
    if (want_nccl) {
        const char* libname = getenv("DCCL_NCCL_LIB");
        void* h = dlopen(libname && *libname ? libname : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) { std::cerr << "cannot open libnccl: " << dlerror() << " (set DCCL_NCCL_LIB)" << std::endl; return 5; }
        auto getid = (stock::GetUniqueId_t)dlsym(h, "ncclGetUniqueId");
        auto init = (stock::CommInitRank_t)dlsym(h, "ncclCommInitRank");
        nDestroy = (stock::CommDestroy_t)dlsym(h, "ncclCommDestroy");
        nAllReduce = (stock::AllReduce_t)dlsym(h, "ncclAllReduce");
        nReduceScatter = (stock::ReduceScatter_t)dlsym(h, "ncclReduceScatter");
        nAllGather = (stock::AllGather_t)dlsym(h, "ncclAllGather");
        nBroadcast = (stock::Broadcast_t)dlsym(h, "ncclBroadcast");
        nReduce = (stock::Reduce_t)dlsym(h, "ncclReduce");
        auto nMemAlloc = (stock::MemAlloc_t)dlsym(h, "ncclMemAlloc");
        auto nRegister = (stock::CommRegister_t)dlsym(h, "ncclCommRegister");
        nMemFree = (stock::MemFree_t)dlsym(h, "ncclMemFree");
        nDeregister = (stock::CommDeregister_t)dlsym(h, "ncclCommDeregister");
        if (!getid || !init || !nDestroy || !nAllReduce || !nReduceScatter || !nAllGather || !nBroadcast || !nReduce) return 5;
        if (nccl_registered && (!nMemAlloc || !nRegister || !nMemFree || !nDeregister)) { std::cerr << "this libnccl has no ncclMemAlloc / ncclCommRegister" << std::endl; return 5; }
        stock::uid_t id;
        memset(&id, 0, sizeof(id));
        if (rank == 0 && getid(&id) != 0) return 1;
        if (dccl::ncclBroadcast(&id, &id, sizeof(id), dccl::ncclUint8, 0, comm, nullptr) != dccl::ncclSuccess) return 1;
        if (init(&ncomm, world, id, rank) != 0) { std::cerr << "ncclCommInitRank failed" << std::endl; return 1; }
        if (nccl_registered) {
            if (nMemAlloc((void**)&s_nccl, maxb) != 0 || nMemAlloc((void**)&r_nccl, maxb) != 0) { std::cerr << "ncclMemAlloc failed" << std::endl; return 4; }
            if (nRegister(ncomm, s_nccl, maxb, &reg_s) != 0 || nRegister(ncomm, r_nccl, maxb, &reg_r) != 0) { std::cerr << "ncclCommRegister failed" << std::endl; return 4; }
        } else if (cudaMalloc((void**)&s_nccl, maxb) != cudaSuccess || cudaMalloc((void**)&r_nccl, maxb) != cudaSuccess) return 4;
        cudaMemset(s_nccl, 0, maxb);
    }

    auto host_barrier = [&]() { int32_t w = 0; dccl::ncclAllReduce(&w, &w, 1, dccl::ncclInt32, dccl::ncclSum, comm, nullptr); };
    auto host_max = [&](double v) { dccl::ncclAllReduce(&v, &v, 1, dccl::ncclFloat64, dccl::ncclMax, comm, nullptr); return v; };
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    std::ostringstream json;
    json << "{\"n_gpus\": " << world << ", \"dtype\": \"" << name_of_type(dt) << "\", \"symmetric\": " << (symmetric ? "true" : "false") << ", \"rows\": [";
    bool first = true;
    if (rank == 0) printf("%-15s %-5s %12s %10s %10s %10s  %s\n", "collective", "impl", "bytes", "us", "algbw", "busbw", "variant");

    // every combination of the --grid values (one empty combination without --grid)
    std::vector<std::vector<int>> combos(1);
    for (const auto& g : grid) {
        std::vector<std::vector<int>> next;
        for (const auto& c : combos) for (int v : g.second) { auto d = c; d.push_back(v); next.push_back(d); }
        combos.swap(next);
    }
    for (const auto& combo : combos) {
    std::string tag;
    for (size_t k = 0; k < combo.size(); k++) {
        if (want_dccl && dccl::dcclSetParam(comm, grid[k].first.c_str(), combo[k]) != dccl::ncclSuccess) { std::cerr << "bad --grid parameter " << grid[k].first << std::endl; return 1; }
        tag += " " + grid[k].first + "=" + std::to_string(combo[k]);
    }
    for (const std::string& coll : split(colls)) {
        for (const std::string& impl : split(impls)) {
            const bool ours = impl == "dccl";
            if (!ours && &combo != &combos[0]) continue;      // NCCL does not depend on the grid: once
            if ((ours && !want_dccl) || (!ours && !want_nccl)) continue;
            char* sb = ours ? s_ours : s_nccl;
            char* rb = ours ? r_ours : r_nccl;
            for (size_t bytes = minb; bytes <= maxb; bytes *= factor) {
                // S = full vector bytes; per-rank count for reduce-scatter / all-gather
                size_t elems = bytes / es;
                if (elems < (size_t)world) elems = world;
                elems = elems / world * world;
                const size_t per = elems / world, total = elems * es;
                auto call = [&]() -> int {
                    if (coll == "all_reduce") return ours ? (int)dccl::ncclAllReduce(sb, rb, elems, dt, op, comm, stream) : nAllReduce(sb, rb, elems, dt, op, ncomm, stream);
                    if (coll == "reduce_scatter") return ours ? (int)dccl::ncclReduceScatter(sb, rb, per, dt, op, comm, stream) : nReduceScatter(sb, rb, per, dt, op, ncomm, stream);
                    if (coll == "all_gather") return ours ? (int)dccl::ncclAllGather(sb, rb, per, dt, comm, stream) : nAllGather(sb, rb, per, dt, ncomm, stream);
                    if (coll == "broadcast") return ours ? (int)dccl::ncclBroadcast(sb, rb, elems, dt, 0, comm, stream) : nBroadcast(sb, rb, elems, dt, 0, ncomm, stream);
                    if (coll == "reduce") return ours ? (int)dccl::ncclReduce(sb, rb, elems, dt, op, 0, comm, stream) : nReduce(sb, rb, elems, dt, op, 0, ncomm, stream);
                    return 99;
                };
                const int iters = total <= (1u << 20) ? 200 : total <= (64u << 20) ? 40 : 10;
                int rc = 0;
                const unsigned long long zc0 = ours ? dccl::dcclGetStat(comm, "zero_copy_calls") : 0ull;
                for (int i = 0; i < 5 && !rc; i++) rc = call();
                cudaStreamSynchronize(stream);
                host_barrier();
                cudaEventRecord(e0, stream);
                for (int i = 0; i < iters && !rc; i++) rc = call();
                cudaEventRecord(e1, stream);
                cudaStreamSynchronize(stream);
                if (rc) { std::cerr << coll << " (" << impl << ") failed with " << rc << " at " << total << " bytes" << std::endl; return 2; }
                float ms = 0;
                cudaEventElapsedTime(&ms, e0, e1);
                const double us = host_max((double)ms * 1e3 / iters);
                const double n = world, alg = (double)total / (us * 1e-6) / 1e9;
                const double f = world == 1 || coll == "broadcast" || coll == "reduce" ? 1.0 : coll == "all_reduce" ? 2 * (n - 1) / n : (n - 1) / n;
                const char* variant = ours ? dccl::dcclGetLastAlgorithm(comm, coll == "all_reduce" ? "allreduce" : coll == "reduce_scatter" ? "reducescatter"
                                                                              : coll == "all_gather" ? "allgather" : coll.c_str())
                                           : nccl_registered ? "nccl-registered" : "nccl";
                std::string vname(variant);
                if (ours && dccl::dcclGetStat(comm, "zero_copy_calls") > zc0) vname += "+zerocopy";   // served out of / into user memory
                if (ours) vname += tag;
                if (rank == 0) {
                    printf("%-15s %-5s %12zu %10.2f %10.2f %10.2f  %s\n", coll.c_str(), impl.c_str(), total, us, alg, alg * f, vname.c_str());
                    fflush(stdout);
                    json << (first ? "" : ",") << "\n {\"coll\": \"" << coll << "\", \"impl\": \"" << impl << "\", \"bytes\": " << total << ", \"us\": " << us
                         << ", \"algbw_gbs\": " << alg << ", \"busbw_gbs\": " << alg * f << ", \"variant\": \"" << vname << "\"}";
                    first = false;
                }
            }
        }
    }
    }
    json << "\n]}\n";
    if (rank == 0 && !out.empty()) {
        FILE* f = fopen(out.c_str(), "w");
        if (f) { fputs(json.str().c_str(), f); fclose(f); }
    }
    dccl::ncclResult_t async = dccl::ncclSuccess;
    char msg[200];
    dccl::dcclGetLastError(comm, &async, msg, sizeof(msg));
    if (async != dccl::ncclSuccess) std::cerr << "communicator error: " << msg << std::endl;
    if (reg_s) nDeregister(ncomm, reg_s);
    if (reg_r) nDeregister(ncomm, reg_r);
    if (ncomm && nccl_registered) { nMemFree(s_nccl); nMemFree(r_nccl); }
    if (ncomm) nDestroy(ncomm);
    if (symmetric) { dccl::dcclMemFree(comm, s_ours); dccl::dcclMemFree(comm, r_ours); }
    dccl::ncclCommFinalize(comm);
    return async == dccl::ncclSuccess ? 0 : 2;
}
