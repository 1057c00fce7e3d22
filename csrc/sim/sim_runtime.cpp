/**
 * Host simulation of a kernel launch (make SIM=1): every CUDA thread of the grid is an OS thread, a CTA barrier is
 * a counting barrier that forgets threads which have returned (as the hardware does), polling loops yield the
 * processor. All CTAs run at the same time, like the cooperative launch the single-GPU emulation uses, so kernels
 * whose CTAs wait on each other make progress. Nothing here is built into the normal library.
 */
#include <cuda_runtime.h>
#include "../kernels/kernels.hpp"
#include <condition_variable>
#include <mutex>
#include <cstdio>
#include <sched.h>
#include <sys/mman.h>
#include <thread>
#include <vector>

namespace dccl_sim {

thread_local ThreadCtx t_ctx;

namespace {

struct CtaBarrier {
    std::mutex m;
    std::condition_variable cv;
    unsigned members, waiting = 0;
    unsigned long generation = 0;
    explicit CtaBarrier(unsigned n) : members(n) {}
    void wait() {
        std::unique_lock<std::mutex> l(m);
        const unsigned long g = generation;
        if (++waiting == members) { waiting = 0; generation++; cv.notify_all(); return; }
        cv.wait(l, [&] { return generation != g; });
    }
    /** a thread that returned from the kernel no longer takes part */
    void drop() {
        std::unique_lock<std::mutex> l(m);
        members--;
        if (members && waiting == members) { waiting = 0; generation++; cv.notify_all(); }
    }
};

} // namespace

void syncthreads() { static_cast<CtaBarrier*>(t_ctx.cta)->wait(); }

void pause() { sched_yield(); }

namespace {
constexpr int kMaxMaps = 32;
McMap g_maps[kMaxMaps];
std::mutex g_maps_mutex;
}

char* mc_create(size_t size, int n, char* const* mem) {
    void* p = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);   // never dereferenced
    if (p == MAP_FAILED) return nullptr;
    std::lock_guard<std::mutex> l(g_maps_mutex);
    for (McMap& m : g_maps)
        if (!m.base) {
            m.size = size; m.n = n;
            for (int r = 0; r < n; r++) m.mem[r] = mem[r];
            m.base = static_cast<char*>(p);
            return m.base;
        }
    munmap(p, size);
    return nullptr;
}

void mc_destroy(char* base) {
    std::lock_guard<std::mutex> l(g_maps_mutex);
    for (McMap& m : g_maps)
        if (m.base == base && base) { munmap(m.base, m.size); m.base = nullptr; }
}

/** Mappings only change between launches, so the kernels' threads read the table without a lock. */
const McMap* mc_find(const void* p) {
    const char* c = static_cast<const char*>(p);
    for (const McMap& m : g_maps)
        if (m.base && c >= m.base && c < m.base + m.size) return &m;
    fprintf(stderr, "dccl simulation: %p is not a multicast address\n", p);
    abort();
}

void launch(void (*fn)(const void*), const void* arg, unsigned grid, unsigned block) {
    std::vector<CtaBarrier*> bars(grid);
    for (unsigned b = 0; b < grid; b++) bars[b] = new CtaBarrier(block);
    std::vector<std::thread> ts;
    ts.reserve((size_t)grid * block);
    for (unsigned b = 0; b < grid; b++)
        for (unsigned t = 0; t < block; t++)
            ts.emplace_back([=] {
                t_ctx.thread_idx = uint3{t, 0, 0};
                t_ctx.block_idx = uint3{b, 0, 0};
                t_ctx.block_dim = dim3(block);
                t_ctx.grid_dim = dim3(grid);
                t_ctx.cta = bars[b];
                fn(arg);
                bars[b]->drop();
            });
    for (auto& t : ts) t.join();
    for (auto* b : bars) delete b;
}

} // namespace dccl_sim

namespace dccl {

/* The one-rank kernels use the <<< >>> launch syntax and are not part of the simulation. */
cudaError_t launch_local_copy(void* dst, const void* src, size_t bytes, cudaStream_t) { memmove(dst, src, bytes); return cudaSuccess; }
cudaError_t launch_local_reduce(void*, const void*, size_t, ncclDataType_t, ncclRedOp_t, cudaStream_t) { return cudaErrorInvalidValue; }
cudaError_t launch_wait_probe(const DevComm&, cudaStream_t) { return cudaErrorInvalidValue; }

} // namespace dccl
