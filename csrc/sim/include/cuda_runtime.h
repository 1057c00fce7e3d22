/**
 * Stand-in for <cuda_runtime.h> in the host simulation build (make SIM=1): the collective kernels and the
 * single-GPU emulation harness are compiled as ordinary C++ and every CUDA thread becomes an OS thread, so the
 * flag protocol, packet generations, staging geometry and reductions of the non-multimem kernels can be run and
 * checked on a machine without a GPU. Only what those sources use is declared here.
 */
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#define __host__
#define __device__
#define __global__
#define __forceinline__ inline __attribute__((always_inline))
#define __launch_bounds__(...)
#define __grid_constant__
/* One instance per function, shared by ALL simulated CTAs: good enough for the flags the kernels keep in shared
 * memory, which only ever change from "fine" to "failed". */
#define __shared__ static
#define __align__(n) alignas(n)

struct uint2 { unsigned int x, y; };
struct uint3 { unsigned int x, y, z; };
struct alignas(16) uint4 { unsigned int x, y, z, w; };
struct dim3 {
    unsigned int x, y, z;
    dim3(unsigned int x_ = 1, unsigned int y_ = 1, unsigned int z_ = 1) : x(x_), y(y_), z(z_) {}
};
inline uint2 make_uint2(unsigned int x, unsigned int y) { return uint2{x, y}; }
inline uint4 make_uint4(unsigned int x, unsigned int y, unsigned int z, unsigned int w) { return uint4{x, y, z, w}; }

typedef struct CUstream_st* cudaStream_t;
typedef struct CUevent_st* cudaEvent_t;
enum cudaError_t { cudaSuccess = 0, cudaErrorInvalidValue = 1, cudaErrorMemoryAllocation = 2, cudaErrorLaunchFailure = 719 };
typedef cudaError_t cudaError;
enum cudaMemcpyKind { cudaMemcpyHostToHost = 0, cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2, cudaMemcpyDeviceToDevice = 3, cudaMemcpyDefault = 4 };
enum cudaDeviceAttr { cudaDevAttrMultiProcessorCount = 16 };

/* "device memory" is host memory */
inline cudaError_t cudaMalloc(void** p, size_t bytes) { *p = aligned_alloc(256, (bytes + 255) / 256 * 256); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
template <typename T> inline cudaError_t cudaMalloc(T** p, size_t bytes) { return cudaMalloc((void**)p, bytes); }
inline cudaError_t cudaFree(void* p) { free(p); return cudaSuccess; }
inline cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) { memcpy(d, s, n); return cudaSuccess; }
inline cudaError_t cudaMemset(void* d, int v, size_t n) { memset(d, v, n); return cudaSuccess; }
inline cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
inline cudaError_t cudaGetLastError() { return cudaSuccess; }
inline const char* cudaGetErrorString(cudaError_t e) { return e == cudaSuccess ? "no error" : "simulated CUDA error"; }
inline cudaError_t cudaGetDevice(int* d) { *d = 0; return cudaSuccess; }
inline cudaError_t cudaDeviceGetAttribute(int* v, cudaDeviceAttr, int) { *v = 8; return cudaSuccess; }
inline cudaError_t cudaEventCreate(cudaEvent_t* e) { *e = nullptr; return cudaSuccess; }
inline cudaError_t cudaEventDestroy(cudaEvent_t) { return cudaSuccess; }
inline cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t = nullptr) { return cudaSuccess; }
inline cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t, cudaEvent_t) { *ms = 0.f; return cudaSuccess; }

namespace dccl_sim {

/** What a simulated CUDA thread knows about itself. */
struct ThreadCtx {
    uint3 thread_idx, block_idx;
    dim3 block_dim, grid_dim;
    void* cta;             // barrier of the CTA
};
extern thread_local ThreadCtx t_ctx;
void syncthreads();
void pause();              // called from polling loops: lets the other simulated threads run
/** Run fn(arg) once per simulated thread of a grid x block launch; returns when all of them have returned. */
void launch(void (*fn)(const void*), const void* arg, unsigned grid, unsigned block);

/** A simulated multicast mapping: addresses [base, base + size) stand for the same offsets in n memories. */
struct McMap { char* base; size_t size; int n; char* mem[8]; };
/** Reserve an inaccessible address range of `size` bytes that stands for mem[0..n) and return its base. */
char* mc_create(size_t size, int n, char* const* mem);
void mc_destroy(char* base);
const McMap* mc_find(const void* p);

} // namespace dccl_sim

#define threadIdx (::dccl_sim::t_ctx.thread_idx)
#define blockIdx (::dccl_sim::t_ctx.block_idx)
#define blockDim (::dccl_sim::t_ctx.block_dim)
#define gridDim (::dccl_sim::t_ctx.grid_dim)

inline void __syncthreads() { ::dccl_sim::syncthreads(); }
inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
inline void __threadfence_system() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
inline unsigned int atomicAdd(unsigned int* p, unsigned int v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
