/**
 * Entry points of the public API (counterpart of reference src/core/dccl.cpp:38-911).
 *
 * Each call checks its arguments, decides host or device from the pointers
 * (like the original, reference dccl.cpp:358-366, not from the stream), picks
 * the algorithm (per-communicator override > DCCL/<collective>_algorithm key >
 * automatic) and hands over to the host backend or to the device communicator.
 * Device calls are stream ordered and return right after the launch; host calls
 * block until done.
 */
#include "comm.hpp"
#include "../core/config.hpp"
#include "../core/log.hpp"
#include "../core/types.hpp"
#include <cstring>
#include <stdexcept>
#include <vector>

namespace dccl {

#define VALIDATE_COMM(c) do { if ((c) == nullptr) throw std::runtime_error("invalid (null) communicator passed to " + std::string(__func__)); } while (0)

const char* dcclGetErrorString(ncclResult_t r) {
    switch (r) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error";
    case ncclSystemError: return "unhandled system error";
    case ncclInternalError: return "internal error";
    case ncclInvalidArgument: return "invalid argument";
    case ncclInvalidUsage: return "invalid usage";
    case ncclRemoteError: return "remote process exited or there was a network error";
    case ncclInProgress: return "operation in progress";
    default: return "unknown result code";
    }
}

uint32_t dcclGetWorldSize(ncclComm_t comm) { VALIDATE_COMM(comm); return (uint32_t)comm->bs.world(); }
uint32_t dcclGetMyRank(ncclComm_t comm) { VALIDATE_COMM(comm); return (uint32_t)comm->bs.rank(); }

/* ---------------- life cycle ---------------- */

static void read_algo_overrides(dcclComm* c) {
    Config& cfg = Config::global();
    const char* keys[COLL_COUNT] = {DCCL_ALLREDUCE_ALGORITHM_CONFSTR, DCCL_REDUCESCATTER_ALGORITHM_CONFSTR,
                                    DCCL_ALLGATHER_ALGORITHM_CONFSTR, "DCCL/broadcast_algorithm", "DCCL/reduce_algorithm", ""};
    std::string all = cfg.get_str("DCCL/algo", "");
    for (int i = 0; i < COLL_COUNT; i++) {
        c->algo[i] = ALGO_AUTO;
        c->last_host_algo[i] = HOST_ALGO_RING;
        c->last_was_host[i] = false;
        std::string v = all;
        if (keys[i][0]) v = cfg.get_str(keys[i], all);
        if (v.empty()) continue;
        GpuAlgo a = parse_algo_name(v.c_str());
        if (a == ALGO_COUNT) dccl_warn("unknown algorithm name '%s' for %s ignored", v.c_str(), keys[i]);
        else c->algo[i] = a;
    }
}

static ncclResult_t finish_init(dcclComm* c, const UniqueIdData& id, int rank, int world, ncclComm_t* out) {
    std::string err;
    int timeout = (int)Config::global().get_int("DCCL/init_timeout_ms", 120000);
    if (!c->bs.init(id, rank, world, timeout, &err)) {
        dccl_error("communicator init failed: %s", err.c_str());
        delete c;
        return ncclSystemError;
    }
    log_set_rank(rank);
    c->cpu = new CpuBackend(&c->bs);
    read_algo_overrides(c);
    c->bs.on_abort([c](int failed) { if (c->gpu) c->gpu->abort(failed); });
    // bind a device right away when the launcher says which one this rank drives
    const char* dev_env = getenv("DCCL_CUDA_DEVICE");
    if (dev_env && *dev_env) {
        std::string gerr;
        c->gpu = GpuComm::create(&c->bs, atoi(dev_env), &gerr);
        if (!c->gpu) { dccl_error("device setup failed: %s", gerr.c_str()); c->gpu_failed = true; }
    }
    dccl_info("communicator ready: rank %d of %d", rank, world);
    *out = c;
    return ncclSuccess;
}

ncclResult_t ncclCommInit(ncclComm_t* comm) {
    if (!comm) return ncclInvalidArgument;
    Config::global().reload();
    BootstrapParams bp;
    std::string err;
    if (!resolve_bootstrap_params(&bp, &err)) { dccl_error("%s", err.c_str()); return ncclInvalidUsage; }
    dccl_debug("bootstrap from %s: rank %d world %d at %s:%d", bp.source.c_str(), bp.rank, bp.world, bp.addr.c_str(), bp.port);
    dcclComm* c = new (std::nothrow) dcclComm();
    if (!c) return ncclSystemError;
    UniqueIdData id;
    memset(&id, 0, sizeof(id));
    if (bp.rank == 0 && bp.world > 1) {
        if (!Bootstrap::create_listener(bp.addr, bp.port, &id, &err)) { dccl_error("%s", err.c_str()); delete c; return ncclSystemError; }
    } else {
        id.port = (uint32_t)bp.port;
        snprintf(id.addr, sizeof(id.addr), "%s", bp.addr.c_str());
    }
    return finish_init(c, id, bp.rank, bp.world, comm);
}

ncclResult_t dcclGetUniqueId(dcclUniqueId* out) {
    if (!out) return ncclInvalidArgument;
    UniqueIdData id;
    std::string err;
    const char* a = getenv("DCCL_MASTER_ADDR");
    if (!Bootstrap::create_listener(a && *a ? a : "127.0.0.1", 0, &id, &err)) { dccl_error("%s", err.c_str()); return ncclSystemError; }
    memset(out, 0, sizeof(*out));
    memcpy(out->internal, &id, sizeof(id));
    return ncclSuccess;
}

ncclResult_t dcclCommInitRank(ncclComm_t* comm, int nranks, dcclUniqueId uid, int rank) {
    if (!comm || nranks < 1 || rank < 0 || rank >= nranks) return ncclInvalidArgument;
    UniqueIdData id;
    memcpy(&id, uid.internal, sizeof(id));
    dcclComm* c = new (std::nothrow) dcclComm();
    if (!c) return ncclSystemError;
    return finish_init(c, id, rank, nranks, comm);
}

ncclResult_t ncclCommFinalize(ncclComm_t comm) {
    VALIDATE_COMM(comm);
    static const char* names[COLL_COUNT] = {"allreduce", "reducescatter", "allgather", "broadcast", "reduce", "sendrecv"};
    for (int i = 0; i < COLL_COUNT; i++)
        if (comm->calls[i]) dccl_info("%s: %llu calls, %llu bytes", names[i], (unsigned long long)comm->calls[i], (unsigned long long)comm->bytes[i]);
    if (comm->gpu) dccl_info("device kernels launched: %llu", (unsigned long long)comm->gpu->launches());
    // everybody arrives here before anybody unmaps peer memory; a failed group skips the wait
    if (comm->gpu) comm->gpu->quiesce();
    if (!comm->bs.aborted()) comm->bs.barrier();
    delete comm->gpu; comm->gpu = nullptr;
    delete comm->cpu; comm->cpu = nullptr;
    comm->bs.shutdown();
    delete comm;
    return ncclSuccess;
}

ncclResult_t dcclCommAbort(ncclComm_t comm) {
    VALIDATE_COMM(comm);
    comm->bs.set_abort(comm->bs.rank(), ncclInternalError);
    if (comm->gpu) comm->gpu->abort(comm->bs.rank());
    return ncclSuccess;
}

ncclResult_t dcclCommShrink(ncclComm_t comm, ncclComm_t* newcomm) {
    VALIDATE_COMM(comm);
    if (!newcomm) return ncclInvalidArgument;
    UniqueIdData id;
    int nr = -1, nw = 0;
    std::string err;
    const int timeout = (int)Config::global().get_int("DCCL/init_timeout_ms", 120000);
    if (!comm->bs.shrink_rendezvous(timeout, &id, &nr, &nw, &err)) {
        dccl_error("dcclCommShrink: %s", err.c_str());
        return ncclInvalidUsage;
    }
    dccl_info("rank %d of %d continues as rank %d of %d", comm->bs.rank(), comm->bs.world(), nr, nw);
    dcclComm* c = new (std::nothrow) dcclComm();
    if (!c) return ncclSystemError;
    return finish_init(c, id, nr, nw, newcomm);
}

ncclResult_t dcclGetLastError(ncclComm_t comm, ncclResult_t* async_error, char* msg, size_t msg_len) {
    VALIDATE_COMM(comm);
    ncclResult_t r = ncclSuccess;
    if (msg && msg_len) msg[0] = 0;
    if (comm->gpu) r = comm->gpu->async_error(msg, msg_len);
    if (r == ncclSuccess && comm->host_error != ncclSuccess) {
        r = comm->host_error;
        if (msg && msg_len) {
            if (comm->bs.aborted()) snprintf(msg, msg_len, "%s (rank %d failed or aborted)", comm->host_error_msg.c_str(), comm->bs.failed_rank());
            else snprintf(msg, msg_len, "%s", comm->host_error_msg.c_str());
        }
    }
    if (r == ncclSuccess && comm->bs.aborted()) {
        r = ncclRemoteError;
        if (msg && msg_len) snprintf(msg, msg_len, "rank %d failed or aborted", comm->bs.failed_rank());
    }
    if (async_error) *async_error = r;
    return ncclSuccess;
}

/* ---------------- helpers ---------------- */

enum Where { ON_HOST, ON_DEVICE, MIXED };

static Where classify(const void* a, const void* b, int* device) {
    int da = -1, db = -1;
    bool ia = a ? is_device_pointer(a, &da) : false;
    bool ib = b ? is_device_pointer(b, &db) : ia;
    if (!a) ia = ib;
    if (ia != ib) return MIXED;
    if (ia) { *device = da >= 0 ? da : db; return ON_DEVICE; }
    return ON_HOST;
}

ncclResult_t ensure_gpu(dcclComm* c, int device) {
    if (c->gpu) return ncclSuccess;
    if (c->gpu_failed) return ncclUnhandledCudaError;
    std::lock_guard<std::mutex> g(c->mu);
    if (c->gpu) return ncclSuccess;
    std::string err;
    c->gpu = GpuComm::create(&c->bs, device, &err);
    if (!c->gpu) { dccl_error("device setup failed: %s", err.c_str()); c->gpu_failed = true; return ncclUnhandledCudaError; }
    return ncclSuccess;
}

static HostAlgo host_algo_for(dcclComm* c, int coll) {
    return c->algo[coll] == ALGO_RABENSEIFNER ? HOST_ALGO_RABENSEIFNER : HOST_ALGO_RING;
}

/** A group that lost a rank or was aborted takes no more work. */
#define HOST_CALL(c, expr) ((c)->bs.aborted() ? ncclRemoteError : (expr))

static ncclResult_t note_host(dcclComm* c, int coll, ncclResult_t r, const char* what) {
    c->last_was_host[coll] = true;
    if (r != ncclSuccess && c->host_error == ncclSuccess) {
        c->host_error = r;
        c->host_error_msg = std::string(what) + " failed on host buffers: " + dcclGetErrorString(r);
    }
    return r;
}

static bool bad_dtype(ncclDataType_t dt) { return (int)dt < 0 || (int)dt >= (int)ncclNumTypes; }
static bool bad_op(ncclRedOp_t op) { return (int)op < 0 || (int)op >= (int)ncclNumOps; }

/* ---------------- memory ---------------- */

ncclResult_t dcclRegisterCacheMemory(ncclComm_t comm, void* buffer, size_t size) {
    VALIDATE_COMM(comm);
    if (!buffer || CACHELINE_OFFSET(buffer) || (size % CACHELINE_SIZE)) {
        dccl_error("dcclRegisterCacheMemory: buffer %p / size %zu is not a multiple of the cache line size (%d)", buffer, size, CACHELINE_SIZE);
        return ncclInvalidArgument;
    }
    int dev = -1;
    if (!is_device_pointer(buffer, &dev)) return ncclSuccess;   // host memory needs no mapping
    ncclResult_t r = ensure_gpu(comm, dev);
    if (r != ncclSuccess) return r;
    return comm->gpu->register_buffer(buffer, size);
}

ncclResult_t dcclDeregisterCacheMemory(ncclComm_t comm, void* buffer, size_t) {
    VALIDATE_COMM(comm);
    int dev = -1;
    if (!buffer) return ncclInvalidArgument;
    if (!is_device_pointer(buffer, &dev) || !comm->gpu) return ncclSuccess;
    return comm->gpu->deregister_buffer(buffer);
}

ncclResult_t dcclMemAlloc(ncclComm_t comm, void** ptr, size_t size) {
    VALIDATE_COMM(comm);
    if (!ptr || !size) return ncclInvalidArgument;
    if (!comm->gpu) {
        dccl_error("dcclMemAlloc needs a bound device: set DCCL_CUDA_DEVICE before ncclCommInit, or make a device call first");
        return ncclInvalidUsage;
    }
    return comm->gpu->mem_alloc(ptr, size);
}

ncclResult_t dcclMemFree(ncclComm_t comm, void* ptr) {
    VALIDATE_COMM(comm);
    if (!comm->gpu) return ncclInvalidUsage;
    return comm->gpu->mem_free(ptr);
}

/* ---------------- collectives ---------------- */

ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t dt, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream) {
    VALIDATE_COMM(comm);
    const uint32_t rank = (uint32_t)comm->bs.rank();
    TIMESTAMP(TT_ALLREDUCE_ENTER, rank, op);
    if (bad_dtype(dt) || bad_op(op) || (count && (!sendbuff || !recvbuff))) return ncclInvalidArgument;
    int dev = -1;
    Where w = classify(sendbuff, recvbuff, &dev);
    if (w == MIXED) {
        dccl_error("ncclAllReduce: sendbuff and recvbuff must both be host or both be device memory");
        return ncclInvalidArgument;
    }
    comm->calls[COLL_ALLREDUCE]++;
    comm->bytes[COLL_ALLREDUCE] += count * size_of_type(dt);
    ncclResult_t r;
    if (w == ON_HOST) {
        HostAlgo ha = host_algo_for(comm, COLL_ALLREDUCE);
        comm->last_host_algo[COLL_ALLREDUCE] = ha;
        r = note_host(comm, COLL_ALLREDUCE, HOST_CALL(comm, comm->cpu->all_reduce(sendbuff, recvbuff, count, dt, op, ha)), "ncclAllReduce");
    } else {
        if ((r = ensure_gpu(comm, dev)) != ncclSuccess) return r;
        comm->last_was_host[COLL_ALLREDUCE] = false;
        r = comm->gpu->all_reduce(sendbuff, recvbuff, count, dt, op, comm->algo[COLL_ALLREDUCE], stream);
    }
    TIMESTAMP(TT_ALLREDUCE_DONE, rank, op);
    return r;
}

ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op,
                               ncclComm_t comm, cudaStream_t stream) {
    VALIDATE_COMM(comm);
    const uint32_t rank = (uint32_t)comm->bs.rank();
    TIMESTAMP(TT_REDUCESCATTER_ENTER, rank, op);
    if (bad_dtype(dt) || bad_op(op) || (recvcount && (!sendbuff || !recvbuff))) return ncclInvalidArgument;
    int dev = -1;
    Where w = classify(sendbuff, recvbuff, &dev);
    if (w == MIXED) return ncclInvalidArgument;
    comm->calls[COLL_REDUCESCATTER]++;
    comm->bytes[COLL_REDUCESCATTER] += recvcount * size_of_type(dt) * comm->bs.world();
    ncclResult_t r;
    if (w == ON_HOST) {
        HostAlgo ha = host_algo_for(comm, COLL_REDUCESCATTER);
        comm->last_host_algo[COLL_REDUCESCATTER] = ha;
        r = note_host(comm, COLL_REDUCESCATTER, HOST_CALL(comm, comm->cpu->reduce_scatter(sendbuff, recvbuff, recvcount, dt, op, ha)), "ncclReduceScatter");
    } else {
        if ((r = ensure_gpu(comm, dev)) != ncclSuccess) return r;
        comm->last_was_host[COLL_REDUCESCATTER] = false;
        r = comm->gpu->reduce_scatter(sendbuff, recvbuff, recvcount, dt, op, comm->algo[COLL_REDUCESCATTER], stream);
    }
    TIMESTAMP(TT_REDUCESCATTER_DONE, rank, op);
    return r;
}

ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t dt,
                           ncclComm_t comm, cudaStream_t stream) {
    VALIDATE_COMM(comm);
    const uint32_t rank = (uint32_t)comm->bs.rank();
    TIMESTAMP(TT_ALLGATHER_ENTER, rank, 0);
    if (bad_dtype(dt) || (sendcount && (!sendbuff || !recvbuff))) return ncclInvalidArgument;
    int dev = -1;
    Where w = classify(sendbuff, recvbuff, &dev);
    if (w == MIXED) return ncclInvalidArgument;
    comm->calls[COLL_ALLGATHER]++;
    comm->bytes[COLL_ALLGATHER] += sendcount * size_of_type(dt) * comm->bs.world();
    ncclResult_t r;
    if (w == ON_HOST) {
        HostAlgo ha = host_algo_for(comm, COLL_ALLGATHER);
        comm->last_host_algo[COLL_ALLGATHER] = ha;
        r = note_host(comm, COLL_ALLGATHER, HOST_CALL(comm, comm->cpu->all_gather(sendbuff, recvbuff, sendcount, dt, ha)), "ncclAllGather");
    } else {
        if ((r = ensure_gpu(comm, dev)) != ncclSuccess) return r;
        comm->last_was_host[COLL_ALLGATHER] = false;
        r = comm->gpu->all_gather(sendbuff, recvbuff, sendcount, dt, comm->algo[COLL_ALLGATHER], stream);
    }
    TIMESTAMP(TT_ALLGATHER_DONE, rank, 0);
    return r;
}

ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t dt, int root,
                           ncclComm_t comm, cudaStream_t stream) {
    VALIDATE_COMM(comm);
    const uint32_t rank = (uint32_t)comm->bs.rank();
    TIMESTAMP(TT_BROADCAST_ENTER, rank, root);
    if (bad_dtype(dt) || root < 0 || root >= comm->bs.world() || (count && !recvbuff)) return ncclInvalidArgument;
    if ((int)rank == root && count && !sendbuff) return ncclInvalidArgument;
    int dev = -1;
    // only the root's sendbuff means anything; classify by what this rank really touches
    Where w = classify((int)rank == root ? sendbuff : recvbuff, recvbuff, &dev);
    if (w == MIXED) return ncclInvalidArgument;
    comm->calls[COLL_BROADCAST]++;
    comm->bytes[COLL_BROADCAST] += count * size_of_type(dt);
    ncclResult_t r;
    if (w == ON_HOST) {
        r = note_host(comm, COLL_BROADCAST, HOST_CALL(comm, comm->cpu->broadcast(sendbuff, recvbuff, count, dt, root)), "ncclBroadcast");
    } else {
        if ((r = ensure_gpu(comm, dev)) != ncclSuccess) return r;
        comm->last_was_host[COLL_BROADCAST] = false;
        r = comm->gpu->broadcast(sendbuff, recvbuff, count, dt, root, comm->algo[COLL_BROADCAST], stream);
    }
    TIMESTAMP(TT_BROADCAST_DONE, rank, root);
    return r;
}

ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t stream) {
    return ncclBroadcast(buff, buff, count, dt, root, comm, stream);
}

ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root,
                        ncclComm_t comm, cudaStream_t stream) {
    VALIDATE_COMM(comm);
    const uint32_t rank = (uint32_t)comm->bs.rank();
    TIMESTAMP(TT_REDUCE_ENTER, rank, op);
    if (bad_dtype(dt) || bad_op(op) || root < 0 || root >= comm->bs.world() || (count && !sendbuff)) return ncclInvalidArgument;
    if ((int)rank == root && count && !recvbuff) return ncclInvalidArgument;
    int dev = -1;
    Where w = classify(sendbuff, (int)rank == root ? recvbuff : sendbuff, &dev);
    if (w == MIXED) return ncclInvalidArgument;
    comm->calls[COLL_REDUCE]++;
    comm->bytes[COLL_REDUCE] += count * size_of_type(dt);
    ncclResult_t r;
    if (w == ON_HOST) {
        r = note_host(comm, COLL_REDUCE, HOST_CALL(comm, comm->cpu->reduce(sendbuff, recvbuff, count, dt, op, root)), "ncclReduce");
    } else {
        if ((r = ensure_gpu(comm, dev)) != ncclSuccess) return r;
        comm->last_was_host[COLL_REDUCE] = false;
        r = comm->gpu->reduce(sendbuff, recvbuff, count, dt, op, root, comm->algo[COLL_REDUCE], stream);
    }
    TIMESTAMP(TT_REDUCE_DONE, rank, op);
    return r;
}

/* ---------------- point to point ---------------- */

static thread_local int t_group_depth = 0;
static thread_local std::vector<dcclComm*> t_group_comms;

static void group_touch(dcclComm* c) {
    for (auto* x : t_group_comms) if (x == c) return;
    t_group_comms.push_back(c);
    c->cpu->group_start();
}

ncclResult_t dcclGroupStart() { t_group_depth++; return ncclSuccess; }

ncclResult_t dcclGroupEnd() {
    if (t_group_depth == 0) return ncclInvalidUsage;
    if (--t_group_depth > 0) return ncclSuccess;
    ncclResult_t r = ncclSuccess;
    for (auto* c : t_group_comms) {
        ncclResult_t a = c->cpu->group_end();
        ncclResult_t b = c->gpu ? c->gpu->group_end() : ncclSuccess;
        if (r == ncclSuccess) r = a != ncclSuccess ? a : b;
    }
    t_group_comms.clear();
    return r;
}

ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t stream) {
    VALIDATE_COMM(comm);
    const int rank = comm->bs.rank();
    TIMESTAMP(TT_SEND_ENTER, rank, peer);
    if (bad_dtype(dt) || peer < 0 || peer >= comm->bs.world() || (count && !sendbuff)) return ncclInvalidArgument;
    if (peer == rank) { dccl_error("ncclSend: cannot send to myself (rank %d)", rank); return ncclInvalidArgument; }
    int dev = -1;
    const size_t bytes = count * size_of_type(dt);
    comm->calls[COLL_SENDRECV]++;
    comm->bytes[COLL_SENDRECV] += bytes;
    ncclResult_t r;
    if (!is_device_pointer(sendbuff, &dev)) {
        if (t_group_depth > 0) group_touch(comm);
        r = note_host(comm, COLL_SENDRECV, HOST_CALL(comm, comm->cpu->send(sendbuff, bytes, peer)), "ncclSend");
    } else {
        if ((r = ensure_gpu(comm, dev)) != ncclSuccess) return r;
        if (t_group_depth > 0) { group_touch(comm); comm->gpu->group_start(); }
        r = comm->gpu->send(sendbuff, bytes, peer, stream);
    }
    TIMESTAMP(TT_SEND_DONE, rank, peer);
    return r;
}

ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t stream) {
    VALIDATE_COMM(comm);
    const int rank = comm->bs.rank();
    TIMESTAMP(TT_RECV_ENTER, rank, peer);
    if (bad_dtype(dt) || peer < 0 || peer >= comm->bs.world() || (count && !recvbuff)) return ncclInvalidArgument;
    if (peer == rank) { dccl_error("ncclRecv: cannot receive from myself (rank %d)", rank); return ncclInvalidArgument; }
    int dev = -1;
    const size_t bytes = count * size_of_type(dt);
    comm->calls[COLL_SENDRECV]++;
    comm->bytes[COLL_SENDRECV] += bytes;
    ncclResult_t r;
    if (!is_device_pointer(recvbuff, &dev)) {
        if (t_group_depth > 0) group_touch(comm);
        r = note_host(comm, COLL_SENDRECV, HOST_CALL(comm, comm->cpu->recv(recvbuff, bytes, peer)), "ncclRecv");
    } else {
        if ((r = ensure_gpu(comm, dev)) != ncclSuccess) return r;
        if (t_group_depth > 0) { group_touch(comm); comm->gpu->group_start(); }
        r = comm->gpu->recv(recvbuff, bytes, peer, stream);
    }
    TIMESTAMP(TT_RECV_DONE, rank, peer);
    return r;
}

ncclResult_t dcclGetTopology(ncclComm_t comm, char* json, size_t len) {
    VALIDATE_COMM(comm);
    if (!json || !len) return ncclInvalidArgument;
    if (!comm->gpu) { json[0] = 0; return ncclInvalidUsage; }
    snprintf(json, len, "%s", comm->gpu->topology().c_str());
    return ncclSuccess;
}

ncclResult_t dcclBarrier(ncclComm_t comm) {
    VALIDATE_COMM(comm);
    if (comm->bs.world() == 1) return ncclSuccess;
    if (!comm->bs.barrier()) {
        comm->host_error = ncclRemoteError;
        comm->host_error_msg = "barrier failed: " + comm->bs.last_error();
        return ncclRemoteError;
    }
    return ncclSuccess;
}

ncclResult_t dcclDebugCheck(ncclComm_t comm) {
    VALIDATE_COMM(comm);
    if (!comm->gpu) return ncclSuccess;
    char msg[200];
    const ncclResult_t r = comm->gpu->debug_check(msg, sizeof(msg));
    if (r != ncclSuccess) {
        dccl_error("%s", msg);
        comm->host_error = r;
        comm->host_error_msg = msg;
    }
    return r;
}

/* ---------------- algorithm control ---------------- */

ncclResult_t dcclSetAlgorithm(ncclComm_t comm, const char* collective, const char* name) {
    VALIDATE_COMM(comm);
    if (!collective || !name) return ncclInvalidArgument;
    int coll = parse_collective_name(collective);
    GpuAlgo a = parse_algo_name(name);
    if (coll < 0 || a == ALGO_COUNT) return ncclInvalidArgument;
    comm->algo[coll] = a;
    return ncclSuccess;
}

ncclResult_t dcclSetParam(ncclComm_t comm, const char* name, int value) {
    VALIDATE_COMM(comm);
    if (!comm->gpu) return ncclInvalidUsage;
    return comm->gpu->set_param(name, value) ? ncclSuccess : ncclInvalidArgument;
}

unsigned long long dcclGetStat(ncclComm_t comm, const char* name) {
    VALIDATE_COMM(comm);
    return comm->gpu ? comm->gpu->stat(name) : 0ull;
}

const char* dcclGetLastAlgorithm(ncclComm_t comm, const char* collective) {
    VALIDATE_COMM(comm);
    int coll = collective ? parse_collective_name(collective) : -1;
    if (coll < 0) return "";
    // a device variant, once one ran, is what tools ask about; host calls report ring / rabenseifner
    if (comm->gpu && comm->gpu->last_algo(coll) != ALGO_AUTO) return algo_name(comm->gpu->last_algo(coll));
    if (comm->last_was_host[coll]) return comm->last_host_algo[coll] == HOST_ALGO_RABENSEIFNER ? "rabenseifner" : "ring";
    return "";
}

} // namespace dccl
