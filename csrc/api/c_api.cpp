/**
 * Flat C symbols over the C++ API, for ctypes / dlopen callers (the Python
 * package binds these). Every function returns the ncclResult_t value as int;
 * C++ exceptions (a null communicator) become ncclInvalidArgument.
 */
#include <atomic>
#include <vector>
#include <dccl/dccl.hpp>
#include "../core/config.hpp"
#include "../core/types.hpp"
#include "../gpu/gpu_comm.hpp"
#ifdef DCCL_WITH_CUDA
#include "../gpu/topology.hpp"
#endif
#include "comm.hpp"
#include "../tuner/tuner.hpp"
#include <cstring>
#include <cstdlib>
#include <sys/mman.h>
#include <unistd.h>

using namespace dccl;

#define GUARD(expr) try { return (int)(expr); } catch (const std::exception&) { return (int)ncclInvalidArgument; }

extern "C" {

int dccl_comm_init(void** comm) { GUARD(ncclCommInit((ncclComm_t*)comm)); }
int dccl_get_unique_id(void* id128) { GUARD(dcclGetUniqueId((dcclUniqueId*)id128)); }
int dccl_comm_init_rank(void** comm, int nranks, const void* id128, int rank) {
    dcclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    GUARD(dcclCommInitRank((ncclComm_t*)comm, nranks, id, rank));
}
int dccl_comm_finalize(void* comm) { GUARD(ncclCommFinalize((ncclComm_t)comm)); }
int dccl_comm_abort(void* comm) { GUARD(dcclCommAbort((ncclComm_t)comm)); }
int dccl_comm_shrink(void* comm, void** newcomm) { GUARD(dcclCommShrink((ncclComm_t)comm, (ncclComm_t*)newcomm)); }
int dccl_world_size(void* comm) { try { return (int)dcclGetWorldSize((ncclComm_t)comm); } catch (...) { return -1; } }
int dccl_rank(void* comm) { try { return (int)dcclGetMyRank((ncclComm_t)comm); } catch (...) { return -1; } }
int dccl_last_error(void* comm, int* code, char* msg, size_t len) {
    ncclResult_t r = ncclSuccess;
    try { dcclGetLastError((ncclComm_t)comm, &r, msg, len); } catch (...) { return (int)ncclInvalidArgument; }
    if (code) *code = (int)r;
    return 0;
}
const char* dccl_error_string(int r) { return dcclGetErrorString((ncclResult_t)r); }

/** Bind this rank to a CUDA device now (collective): the device side is otherwise set up on the first device call. */
int dccl_comm_bind_device(void* comm, int device) {
    dcclComm* c = (dcclComm*)comm;
    if (!c) return (int)ncclInvalidArgument;
    if (c->gpu) return c->gpu->device() == device ? 0 : (int)ncclInvalidUsage;
    std::string err;
    c->gpu = GpuComm::create(&c->bs, device, &err);
    if (!c->gpu) { c->gpu_failed = true; return (int)ncclUnhandledCudaError; }
    return 0;
}
int dccl_has_multicast(void* comm) { dcclComm* c = (dcclComm*)comm; return c && c->gpu && c->gpu->has_multicast() ? 1 : 0; }
unsigned long long dccl_launch_count(void* comm) { dcclComm* c = (dcclComm*)comm; return c && c->gpu ? c->gpu->launches() : 0ull; }
int dccl_is_symmetric(void* comm, const void* p, size_t bytes) { dcclComm* c = (dcclComm*)comm; return c && c->gpu && c->gpu->is_symmetric(p, bytes) ? 1 : 0; }
unsigned long long dccl_comm_stat(void* comm, const char* name) { dcclComm* c = (dcclComm*)comm; return c && c->gpu ? c->gpu->stat(name) : 0ull; }
int dccl_comm_set_param(void* comm, const char* name, int value) { dcclComm* c = (dcclComm*)comm; return c && c->gpu && c->gpu->set_param(name, value) ? 0 : (int)ncclInvalidArgument; }
int dccl_cuda_device_count() { return cuda_device_count(); }
int dccl_barrier(void* comm) { GUARD(dcclBarrier((ncclComm_t)comm)); }
int dccl_debug_check(void* comm) { GUARD(dcclDebugCheck((ncclComm_t)comm)); }
int dccl_topology_json(void* comm, char* out, size_t len) { GUARD(dcclGetTopology((ncclComm_t)comm, out, len)); }
#ifdef DCCL_WITH_CUDA
/** NVLink links per GPU from NVML alone (no CUDA, no communicator): 0 and JSON in `out`, or -1 when NVML cannot be loaded. */
int dccl_nvml_link_report(const char* lib, char* out, size_t len) {
    std::string json, err;
    if (!nvml_link_report(lib, &json, &err)) { if (out && len) snprintf(out, len, "%s", err.c_str()); return -1; }
    if (out && len) snprintf(out, len, "%s", json.c_str());
    return 0;
}
#endif

int dccl_register(void* comm, void* buf, size_t size) { GUARD(dcclRegisterCacheMemory((ncclComm_t)comm, buf, size)); }
int dccl_deregister(void* comm, void* buf) { GUARD(dcclDeregisterCacheMemory((ncclComm_t)comm, buf)); }
int dccl_mem_alloc(void* comm, void** ptr, size_t size) { GUARD(dcclMemAlloc((ncclComm_t)comm, ptr, size)); }
int dccl_mem_free(void* comm, void* ptr) { GUARD(dcclMemFree((ncclComm_t)comm, ptr)); }

int dccl_all_reduce(const void* s, void* r, size_t count, int dt, int op, void* comm, void* stream) {
    GUARD(ncclAllReduce(s, r, count, (ncclDataType_t)dt, (ncclRedOp_t)op, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_reduce_scatter(const void* s, void* r, size_t recvcount, int dt, int op, void* comm, void* stream) {
    GUARD(ncclReduceScatter(s, r, recvcount, (ncclDataType_t)dt, (ncclRedOp_t)op, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_all_gather(const void* s, void* r, size_t sendcount, int dt, void* comm, void* stream) {
    GUARD(ncclAllGather(s, r, sendcount, (ncclDataType_t)dt, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_broadcast(const void* s, void* r, size_t count, int dt, int root, void* comm, void* stream) {
    GUARD(ncclBroadcast(s, r, count, (ncclDataType_t)dt, root, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_reduce(const void* s, void* r, size_t count, int dt, int op, int root, void* comm, void* stream) {
    GUARD(ncclReduce(s, r, count, (ncclDataType_t)dt, (ncclRedOp_t)op, root, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_send(const void* s, size_t count, int dt, int peer, void* comm, void* stream) {
    GUARD(ncclSend(s, count, (ncclDataType_t)dt, peer, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_recv(void* r, size_t count, int dt, int peer, void* comm, void* stream) {
    GUARD(ncclRecv(r, count, (ncclDataType_t)dt, peer, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_all_to_all(const void* s, void* r, size_t count, int dt, void* comm, void* stream) {
    GUARD(dcclAllToAll(s, r, count, (ncclDataType_t)dt, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_all_to_allv(const void* s, const size_t* scounts, const size_t* sdispls, void* r, const size_t* rcounts, const size_t* rdispls,
                     int dt, void* comm, void* stream) {
    GUARD(dcclAllToAllv(s, scounts, sdispls, r, rcounts, rdispls, (ncclDataType_t)dt, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_gather(const void* s, void* r, size_t count, int dt, int root, void* comm, void* stream) {
    GUARD(dcclGather(s, r, count, (ncclDataType_t)dt, root, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_scatter(const void* s, void* r, size_t count, int dt, int root, void* comm, void* stream) {
    GUARD(dcclScatter(s, r, count, (ncclDataType_t)dt, root, (ncclComm_t)comm, (cudaStream_t)stream));
}
int dccl_group_start() { return (int)dcclGroupStart(); }
int dccl_group_end() { return (int)dcclGroupEnd(); }
int dccl_set_algorithm(void* comm, const char* coll, const char* name) { GUARD(dcclSetAlgorithm((ncclComm_t)comm, coll, name)); }
const char* dccl_last_algorithm(void* comm, const char* coll) {
    try { return dcclGetLastAlgorithm((ncclComm_t)comm, coll); } catch (...) { return ""; }
}

/* ---- allocator hook for framework memory pools ----
 * torch.cuda.memory.CUDAPluggableAllocator loads two functions by name from a shared library and torch.cuda.MemPool
 * routes the allocations made inside `use_mem_pool` to them. dccl_pool_alloc serves them with dcclMemAlloc on the
 * communicator bound with dccl_pool_bind, so tensors created there (DDP's gradient buckets, activations that are reduced
 * every step) live in symmetric, multicast-bound memory and collectives on them run zero-copy through the switch, with
 * no change to the code that allocates them. dcclMemAlloc is collective: every rank must make the same allocations in
 * the same order inside the pool (ranks that build the same model do). dccl_pool_free only retires the segment; the
 * memory is unmapped when the communicator is finalized, because the framework may free segments in an order that
 * differs between ranks and a collective free would then hang.
 */
static std::atomic<dcclComm*> g_pool_comm{nullptr};
void dccl_pool_bind(void* comm) { g_pool_comm.store((dcclComm*)comm); }
void* dccl_pool_alloc(ssize_t size, int device, void* stream) {
    (void)device; (void)stream;
    dcclComm* c = g_pool_comm.load();
    void* p = nullptr;
    if (!c || size <= 0 || dcclMemAlloc(c, &p, (size_t)size) != ncclSuccess) return nullptr;
    return p;
}
void dccl_pool_free(void* ptr, ssize_t size, int device, void* stream) { (void)ptr; (void)size; (void)device; (void)stream; }

/**
 * Self test of the exchange board (Bootstrap::fast_allgather): `rounds` all-gathers of a message whose bytes depend on
 * rank and round; the ranks are skewed on purpose (rank r pauses before round k when k % world == r), so that readers
 * meet both a writer that is ahead and one that is behind. Returns 0, or 1 + the round that delivered wrong bytes,
 * or -1 when an exchange failed.
 */
int dccl_selftest_board(void* comm, int rounds) {
    dcclComm* c = (dcclComm*)comm;
    if (!c) return -1;
    Bootstrap& bs = c->bs;
    const int n = bs.world(), r = bs.rank();
    std::vector<unsigned char> mine(kBoardBytes), all((size_t)n * kBoardBytes);
    for (int k = 0; k < rounds; k++) {
        const size_t bytes = 1 + (size_t)(k * 37) % kBoardBytes;
        for (size_t i = 0; i < bytes; i++) mine[i] = (unsigned char)(r * 31 + k * 7 + (int)i);
        if (k % n == r) usleep(200);
        if (!bs.fast_allgather(mine.data(), bytes, all.data())) return -1;
        for (int p = 0; p < n; p++)
            for (size_t i = 0; i < bytes; i++)
                if (all[(size_t)p * bytes + i] != (unsigned char)(p * 31 + k * 7 + (int)i)) return 1 + k;
    }
    return 0;
}

/**
 * Self test of the descriptor plane (what carries the cuMem handles between ranks): every rank puts its rank
 * number into an anonymous memory file, passes the descriptor to every peer and reads what the peers passed.
 * Returns 0, or 1 + the first peer whose file did not arrive or did not hold that peer's rank.
 */
int dccl_selftest_fd_exchange(void* comm) {
    dcclComm* c = (dcclComm*)comm;
    if (!c) return -1;
    Bootstrap& bs = c->bs;
    const int n = bs.world(), r = bs.rank();
    if (n == 1) return 0;
    int fd = memfd_create("dccl-fdtest", 0);
    if (fd < 0) return -2;
    int32_t mine = r;
    if (write(fd, &mine, sizeof(mine)) != (ssize_t)sizeof(mine)) { close(fd); return -2; }
    const uint32_t tag = 0x7e570000u;
    int bad = 0;
    for (int k = 1; k < n && !bad; k++) if (!bs.send_fd((r + k) % n, fd, tag)) bad = 1 + (r + k) % n;
    for (int k = 1; k < n && !bad; k++) {
        const int p = (r + n - k) % n;
        int got = -1;
        int32_t v = -1;
        if (!bs.recv_fd(p, tag, &got, 10000) || pread(got, &v, sizeof(v), 0) != (ssize_t)sizeof(v) || v != p) bad = 1 + p;
        if (got >= 0) close(got);
    }
    close(fd);
    // nobody tears its socket down while a peer still expects a descriptor
    if (!bs.barrier() && !bad) bad = -3;
    return bad;
}

/* timestamps */
void dccl_timestamp_log(unsigned long long tag, unsigned long long rank, unsigned long long extra) { Timestamp::log(tag, rank, extra); }
void dccl_timestamp_flush(const char* filename, int clear) { Timestamp::flush(filename, clear != 0); }
void dccl_timestamp_clear() { Timestamp::clear(); }
unsigned long long dccl_timestamp_size() { return Timestamp::size(); }

/* configuration, for tests */
void dccl_config_reload() { Config::global().reload(); }
void dccl_config_set(const char* key, const char* value) { Config::global().set(key, value); }
int dccl_config_get(const char* key, char* out, size_t len) {
    std::string v;
    if (!Config::global().get(key, &v)) return 0;
    snprintf(out, len, "%s", v.c_str());
    return 1;
}
int dccl_config_parse_world(const char* json) { return Config::world_size_from_layout(json); }

/* variant table, for tests and tools: a process-wide table separate from any communicator */
static Tuner& test_tuner() { static Tuner t; return t; }
int dccl_tuner_load_text(const char* text) { std::string err; return test_tuner().load_text(text, &err); }
int dccl_tuner_choose(const char* coll, int nranks, size_t bytes, int nvls_ok, char* algo_out, size_t len, int* ctas) {
    int c = coll && !strcmp(coll, "allreduce_sym") ? TUNE_ALLREDUCE_SYM : coll && !strcmp(coll, "reducescatter_sym") ? TUNE_REDUCESCATTER_SYM : parse_collective_name(coll);
    if (c < 0) return -1;
    TuneChoice ch = test_tuner().choose(c, nranks, bytes, nvls_ok != 0);
    if (algo_out && len) snprintf(algo_out, len, "%s", algo_name(ch.algo));
    if (ctas) *ctas = ch.ctas;
    return 0;
}

/** The process-wide table in the file format; returns the length of the text (the copy is cut to `len` - 1 characters). */
size_t dccl_tuner_dump(char* out, size_t len) {
    const std::string text = test_tuner().dump();
    if (out && len) snprintf(out, len, "%s", text.c_str());
    return text.size();
}

/** As dccl_tuner_choose, for elements of `esize` bytes (rules bound to an element width come first). */
int dccl_tuner_choose_width(const char* coll, int nranks, size_t bytes, int nvls_ok, int esize, char* algo_out, size_t len, int* ctas) {
    int c = coll && !strcmp(coll, "allreduce_sym") ? TUNE_ALLREDUCE_SYM : coll && !strcmp(coll, "reducescatter_sym") ? TUNE_REDUCESCATTER_SYM : parse_collective_name(coll);
    if (c < 0) return -1;
    TuneChoice ch = test_tuner().choose(c, nranks, bytes, nvls_ok != 0, esize);
    if (algo_out && len) snprintf(algo_out, len, "%s", algo_name(ch.algo));
    if (ctas) *ctas = ch.ctas;
    return 0;
}

/* index arithmetic, exported so unit tests can check it without a communicator */
void dccl_slot_range(size_t count, unsigned n, unsigned i, size_t align, size_t* lo, size_t* hi) { slot_range(count, n, i, align, lo, hi); }
unsigned dccl_reverse_bits(unsigned x, unsigned bits) { return reverse_bits(x, bits); }
unsigned dccl_log_two(unsigned x) { return log_two(x); }
size_t dccl_size_of_type(int dt) { return size_of_type((ncclDataType_t)dt); }
int dccl_parse_type(const char* s) { return (int)parse_type_name(s); }
int dccl_parse_op(const char* s) { return (int)parse_op_name(s); }
float dccl_half_to_float(unsigned short h) { return half_to_float(h); }
unsigned short dccl_float_to_half(float f) { return float_to_half(f); }
float dccl_bf16_to_float(unsigned short h) { return bf16_to_float(h); }
unsigned short dccl_float_to_bf16(float f) { return float_to_bf16(f); }

} // extern "C"
