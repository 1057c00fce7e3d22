/**
 * Implementation of dccl_allreduce_one_device_noalloc (see noalloc_allreduce.h):
 * the two-shot all-reduce kernel with its scratch in a file-scope device array.
 *
 * Host code must not hand the array's NAME to a kernel: on the host that name
 * is only a stand-in symbol, not a device address. The device address is
 * looked up once per device with cudaGetSymbolAddress (with that device
 * current) and passed to the kernel as an ordinary pointer.
 */
#include "noalloc_allreduce.h"
#include "../device/reduce_ops.cuh"
#include "../device/geometry.cuh"
#include <cstdio>
#include <mutex>

namespace dccl {

/* The scratch: flag words and staging of every virtual rank, then one status page. Zero when the
 * module is loaded; shared by all calls on the device; held until the process exits. */
static __device__ __align__(256) unsigned char g_noalloc_scratch[DCCL_NOALLOC_SCRATCH_BYTES];

constexpr int kNoAllocCtas = 4;            // CTAs per virtual rank
constexpr size_t kNoAllocFlagBytes = 16u * 1024u;
constexpr size_t kNoAllocStatusOff = (size_t)DCCL_NOALLOC_MAX_RANKS * DCCL_NOALLOC_RANK_BYTES;

struct NoAllocArgs {
    int nranks;
    int op;
    size_t count;
    const void* in[DCCL_NOALLOC_MAX_RANKS];
    void* out[DCCL_NOALLOC_MAX_RANKS];
    unsigned char* scratch;      // device address of g_noalloc_scratch
    int* user_status;
    unsigned long long timeout_ns;
};

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_noalloc_allreduce(const __grid_constant__ NoAllocArgs a) {
    const int n = a.nranks;
    const int r = blockIdx.x / kNoAllocCtas, bid = blockIdx.x - r * kNoAllocCtas;
    // a communicator view built from the static array: "pool" p is rank p's region of it
    DevComm c;
    c.rank = r;
    c.nranks = n;
    for (int p = 0; p < kMaxPeers; p++) c.pool[p] = reinterpret_cast<char*>(a.scratch) + (size_t)(p < n ? p : 0) * DCCL_NOALLOC_RANK_BYTES;
    c.mc_pool = nullptr;
    c.status = reinterpret_cast<uint32_t*>(a.scratch + kNoAllocStatusOff);
    c.abort_word = c.status + ST_WORDS;      // stays zero: nothing aborts this call from outside
    c.timeout_ns = a.timeout_ns;
    c.stage_bytes = 0;
    const T* send = reinterpret_cast<const T*>(a.in[r]);
    T* recv = reinterpret_cast<T*>(a.out[r]);
    if (n == 1) {   // one rank: the result is the input
        Geometry<T> g1(GEO_WHOLE, a.count, 1, bid, kNoAllocCtas);
        if (recv != send && g1.bhi > g1.blo) copy_range<T>(recv + g1.blo, send + g1.blo, g1.bhi - g1.blo);
        return;
    }
    const Geometry<T> g(GEO_SPLIT, a.count, n, bid, kNoAllocCtas);
    const size_t res_off = g.slot_stride * (size_t)n;
    auto stage_of = [&](int p) { return reinterpret_cast<T*>(c.pool[p] + kNoAllocFlagBytes); };
    auto lo_of = [&](int j) { size_t l = g.len(j); return g.blo < l ? g.blo : l; };
    auto hi_of = [&](int j) { size_t l = g.len(j); return g.bhi < l ? g.bhi : l; };
    const bool avg = a.op == 4;
    bool ok = true;

    // phase 0: push shard p of my input into slot [r] of rank p's staging
    for (int k = 1; k < n; k++) {
        const int p = (r + k) % n;
        const size_t lo = lo_of(p), hi = hi_of(p);
        if (hi > lo) copy_range<T>(stage_of(p) + (size_t)r * g.slot_stride + lo, send + (size_t)p * g.per + lo, hi - lo);
    }
    ok = rank_barrier(c, bid, 1u, 0, 950);
    if (ok) {
        // phase 1: reduce my shard
        const size_t lo = lo_of(r), hi = hi_of(r);
        if (hi > lo) {
            const T* ins[kMaxPeers];
            int k = 0;
            for (int p = 0; p < n; p++) if (p != r) ins[k++] = stage_of(r) + (size_t)p * g.slot_stride + lo;
            reduce_range<T, OP>(stage_of(r) + res_off + lo, recv + (size_t)r * g.per + lo, send + (size_t)r * g.per + lo, ins, k, hi - lo, avg, n);
        }
        ok = rank_barrier(c, bid, 1u, 1, 951);
    }
    if (ok) {
        // phase 2: pull the other result shards
        for (int k = 1; k < n; k++) {
            const int p = (r + k) % n;
            const size_t lo = lo_of(p), hi = hi_of(p);
            if (hi > lo) copy_range<T>(recv + (size_t)p * g.per + lo, stage_of(p) + res_off + lo, hi - lo);
        }
    }
    if (!ok && a.user_status && threadIdx.x == 0) *a.user_status = 1;
}

static std::mutex g_setup_mu;
static unsigned char* g_scratch_addr[64] = {nullptr};   // per device ordinal

} // namespace dccl

using namespace dccl;

extern "C" int dccl_allreduce_one_device_noalloc(int nranks, int dtype, int op, size_t count, const void* const* inputs,
                                                 void* const* outputs, int* device_status, void* stream_v) {
    cudaStream_t stream = (cudaStream_t)stream_v;
    if (nranks < 1 || nranks > DCCL_NOALLOC_MAX_RANKS || dtype < 0 || dtype > 9 || op < 0 || op > 4 || !inputs || !outputs) {
        fprintf(stderr, "dccl_allreduce_one_device_noalloc: bad argument (nranks %d, dtype %d, op %d)\n", nranks, dtype, op);
        return DCCL_NOALLOC_BAD_ARGUMENT;
    }
    static const size_t kSizes[10] = {1, 1, 4, 4, 8, 8, 2, 4, 8, 2};
    const size_t bytes = count * kSizes[dtype];
    if (bytes > DCCL_NOALLOC_MAX_BYTES) {
        fprintf(stderr, "dccl_allreduce_one_device_noalloc: %zu bytes per rank is above the limit of %u bytes of the built-in scratch array\n",
                bytes, (unsigned)DCCL_NOALLOC_MAX_BYTES);
        return DCCL_NOALLOC_TOO_LARGE;
    }
    for (int r = 0; r < nranks; r++)
        if (count && (!inputs[r] || !outputs[r])) {
            fprintf(stderr, "dccl_allreduce_one_device_noalloc: null buffer for rank %d\n", r);
            return DCCL_NOALLOC_BAD_ARGUMENT;
        }
    if (count == 0) return DCCL_NOALLOC_OK;

    // set-up, once per device, with that device current: the device address of the scratch array
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        fprintf(stderr, "dccl_allreduce_one_device_noalloc: cudaGetDevice: %s\n", cudaGetErrorString(e));
        return DCCL_NOALLOC_CUDA_ERROR;
    }
    unsigned char* scratch = nullptr;
    {
        std::lock_guard<std::mutex> g(g_setup_mu);
        if (!g_scratch_addr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                fprintf(stderr, "dccl_allreduce_one_device_noalloc: cudaGetSymbolAddress: %s\n", cudaGetErrorString(e));
                return DCCL_NOALLOC_CUDA_ERROR;
            }
            g_scratch_addr[dev] = (unsigned char*)p;
        }
        scratch = g_scratch_addr[dev];
    }

    // the flag words of every rank and the status page must start from zero; staging need not
    for (int r = 0; r < nranks; r++) {
        e = cudaMemsetAsync(scratch + (size_t)r * DCCL_NOALLOC_RANK_BYTES, 0, kNoAllocFlagBytes, stream);
        if (e != cudaSuccess) break;
    }
    if (e == cudaSuccess) e = cudaMemsetAsync(scratch + kNoAllocStatusOff, 0, 4096, stream);
    if (e == cudaSuccess && device_status) e = cudaMemsetAsync(device_status, 0, sizeof(int), stream);
    if (e != cudaSuccess) {
        fprintf(stderr, "dccl_allreduce_one_device_noalloc: cudaMemsetAsync: %s\n", cudaGetErrorString(e));
        return DCCL_NOALLOC_CUDA_ERROR;
    }

    NoAllocArgs a;
    a.nranks = nranks;
    a.op = op;
    a.count = count;
    for (int r = 0; r < DCCL_NOALLOC_MAX_RANKS; r++) { a.in[r] = r < nranks ? inputs[r] : nullptr; a.out[r] = r < nranks ? outputs[r] : nullptr; }
    a.scratch = scratch;
    a.user_status = device_status;
    a.timeout_ns = 2000000000ull;
    void* params[] = {&a};
    const dim3 grid((unsigned)(nranks * kNoAllocCtas)), block(256);
    e = cudaErrorInvalidValue;
#define CALL(T, OP) e = cudaLaunchCooperativeKernel((const void*)k_noalloc_allreduce<T, OP>, grid, block, params, 0, stream)
    DCCL_DISPATCH_TYPE_OP(dtype, op, CALL)
#undef CALL
    if (e != cudaSuccess) {
        fprintf(stderr, "dccl_allreduce_one_device_noalloc: launch: %s\n", cudaGetErrorString(e));
        cudaGetLastError();
        return DCCL_NOALLOC_CUDA_ERROR;
    }
    return DCCL_NOALLOC_OK;
}
