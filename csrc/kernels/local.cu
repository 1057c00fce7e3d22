/**
 * Single-GPU kernels: copy, pairwise reduce (the operation of the original's
 * only kernel, reference src/core/reduce.cu:9-38, as a vectorised, operator-
 * templated grid), and the bounded-wait self test.
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"

namespace dccl {

static int g_sm_count = 0;
static int sm_count() {
    if (!g_sm_count) {
        int dev = 0, n = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        g_sm_count = n > 0 ? n : 148;
    }
    return g_sm_count;
}

__global__ void __launch_bounds__(512) k_local_copy(char* __restrict__ dst, const char* __restrict__ src, size_t bytes) {
    // each CTA takes one contiguous, 16-byte aligned piece
    const size_t per = ((bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
    const size_t lo = per * blockIdx.x;
    if (lo >= bytes) return;
    const size_t n = bytes - lo < per ? bytes - lo : per;
    copy_bytes(dst + lo, src + lo, n);
}

/**
 * acc[i] = op(acc[i], in[i]). Three streams of HBM traffic and nothing else, so what matters is bytes in flight:
 * every thread keeps kLocalU 16-byte vectors of each operand outstanding (128 KB per SM with two resident CTAs),
 * each CTA on one contiguous piece.
 */
constexpr int kLocalU = 4;
template <typename T, int OP>
__global__ void __launch_bounds__(512) k_local_reduce(T* acc, const T* __restrict__ in, size_t count, int avg) {
    using A = typename Traits<T>::Acc;
    constexpr size_t VE = 16 / sizeof(T);
    constexpr int N = Vec16<T>::N;
    const size_t per = ((count + gridDim.x - 1) / gridDim.x + VE - 1) / VE * VE;
    const size_t lo = per * blockIdx.x;
    if (lo >= count) return;
    const size_t n = count - lo < per ? count - lo : per;
    T* a = acc + lo;
    const T* b = in + lo;
    size_t done = 0;
    if (aligned16(a) && aligned16(b)) {
        const size_t nv = n / N, tid = threadIdx.x, nt = blockDim.x;
        size_t i = tid;
        for (; i + (size_t)(kLocalU - 1) * nt < nv; i += (size_t)kLocalU * nt) {
            Vec16<T> x[kLocalU], y[kLocalU];
#pragma unroll
            for (int u = 0; u < kLocalU; u++) { x[u] = ld_vec<T>(a + (i + (size_t)u * nt) * N); y[u] = ld_vec<T>(b + (i + (size_t)u * nt) * N); }
#pragma unroll
            for (int u = 0; u < kLocalU; u++) {
#pragma unroll
                for (int e = 0; e < N; e++) x[u].e[e] = Traits<T>::down(op_apply<OP, A>(Traits<T>::up(x[u].e[e]), Traits<T>::up(y[u].e[e])));
                st_vec<T>(a + (i + (size_t)u * nt) * N, x[u]);
            }
        }
        for (; i < nv; i += nt) {
            Vec16<T> x = ld_vec<T>(a + i * N), y = ld_vec<T>(b + i * N);
#pragma unroll
            for (int e = 0; e < N; e++) x.e[e] = Traits<T>::down(op_apply<OP, A>(Traits<T>::up(x.e[e]), Traits<T>::up(y.e[e])));
            st_vec<T>(a + i * N, x);
        }
        done = nv * N;
    }
    // ragged end, or operands that are not 16-byte aligned
    const T* ins[1] = {b + done};
    if (n > done) reduce_range<T, OP>(a + done, nullptr, a + done, ins, 1, n - done, avg != 0, 2);
}

cudaError_t launch_local_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
    if (!bytes || dst == src) return cudaSuccess;
    // one CTA per SM, two when the message is large enough to keep them busy
    size_t want = (bytes + (64u << 10) - 1) / (64u << 10);
    int grid = (int)(want < (size_t)(2 * sm_count()) ? want : (size_t)(2 * sm_count()));
    if (grid < 1) grid = 1;
    k_local_copy<<<grid, 512, 0, stream>>>((char*)dst, (const char*)src, bytes);
    return cudaGetLastError();
}

cudaError_t launch_local_reduce(void* acc, const void* in, size_t count, ncclDataType_t dt, ncclRedOp_t op, cudaStream_t stream) {
    if (!count) return cudaSuccess;
    const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                      : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
    size_t want = (count * es + (64u << 10) - 1) / (64u << 10);
    int grid = (int)(want < (size_t)(2 * sm_count()) ? want : (size_t)(2 * sm_count()));   // two resident CTAs per SM: one wave
    if (grid < 1) grid = 1;
    const int avg = 0;   // a pairwise fold has no world size: ncclAvg accumulates like ncclSum here
#define CALL(T, OP) k_local_reduce<T, OP><<<grid, 512, 0, stream>>>((T*)acc, (const T*)in, count, avg)
    DCCL_DISPATCH_TYPE_OP((int)dt, (int)op, CALL)
#undef CALL
    return cudaGetLastError();
}

/** Waits for a flag value that nothing ever writes; must return through the timeout path. */
__global__ void k_wait_probe(const __grid_constant__ DevComm c) {
    if (threadIdx.x == 0) {
        uint32_t* slot = flag_slot(c.pool[c.rank], kMaxCtas - 1, kMaxPeers - 1);
        const uint32_t never = ld_volatile_u32(slot) + 0x40000000u;
        wait_flag_ge(c, slot, never, kMaxPeers - 1, 900, 0);
    }
}

cudaError_t launch_wait_probe(const DevComm& c, cudaStream_t stream) {
    void* params[] = {const_cast<DevComm*>(&c)};
    return cudaLaunchKernel((const void*)k_wait_probe, dim3(1), dim3(32), params, 0, stream);
}

} // namespace dccl
