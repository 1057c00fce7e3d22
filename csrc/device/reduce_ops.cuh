/**
 * Element types, reduction operators and CTA-cooperative range routines.
 *
 * The original has one scalar kernel, recv[i] = op(recv[i], send[i]), with the
 * operator switch inside the loop, no bf16, Avg treated as Sum and Prod
 * squaring the destination (reference src/core/reduce.cu:9-38). Here every
 * operator is a compile-time functor, 16-bit floats accumulate in fp32 over
 * all sources before one rounding, Avg is Sum followed by a fused scale, and
 * accesses are 16-byte vectors whenever the pointers allow it (a scalar loop
 * takes unaligned buffers and tails, so any pointer and any count is legal).
 */
#pragma once
#include "prims.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <type_traits>

namespace dccl {

enum { OP_SUM = 0, OP_PROD = 1, OP_MAX = 2, OP_MIN = 3 };   // ncclAvg runs as OP_SUM plus a final scale

template <typename T> struct Traits { using Acc = T; static __device__ __forceinline__ Acc up(T v) { return v; } static __device__ __forceinline__ T down(Acc a) { return a; } };
template <> struct Traits<__half> {
    using Acc = float;
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float a) { return __float2half_rn(a); }
};
template <> struct Traits<__nv_bfloat16> {
    using Acc = float;
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float a) { return __float2bfloat16_rn(a); }
};

/**
 * One step of the fold. Floating-point max / min follow IEEE maxNum / minNum, like fmaxf / fminf, NCCL's float kernels
 * and the switch's multimem.ld_reduce.max/min: when one operand is NaN the other is returned, so the result does not
 * depend on the order in which the ranks' values meet and is NaN only when every rank's value is.
 */
template <int OP, typename A> __device__ __forceinline__ A op_apply(A a, A b) {
    if constexpr (OP == OP_SUM) return a + b;
    else if constexpr (OP == OP_PROD) return a * b;
    else if constexpr (OP == OP_MAX) {
        if constexpr (std::is_floating_point<A>::value) return (a < b || a != a) ? b : a;
        else return a < b ? b : a;
    } else {
        if constexpr (std::is_floating_point<A>::value) return (b < a || a != a) ? b : a;
        else return b < a ? b : a;
    }
}

/** Final step of ncclAvg on an accumulated sum: floats scale by 1/n, integers divide. */
template <typename A> __device__ __forceinline__ A avg_finish(A a, int n) {
    if constexpr (std::is_floating_point<A>::value) return a * (A(1) / (A)n);
    else return (A)(a / (A)n);
}

template <typename T> struct alignas(16) Vec16 {
    static constexpr int N = 16 / (int)sizeof(T);
    T e[N];
};

template <typename T> __device__ __forceinline__ Vec16<T> ld_vec(const void* p) {
    Vec16<T> v;
    *reinterpret_cast<uint4*>(&v) = *reinterpret_cast<const uint4*>(p);
    return v;
}
template <typename T> __device__ __forceinline__ void st_vec(void* p, const Vec16<T>& v) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&v);
}

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kUnroll = 8;   // 16-byte vectors in flight per thread in the copy loops

/**
 * dst[0..bytes) = src[0..bytes), all threads of the CTA cooperate. When source and
 * destination are misaligned by the same amount the head is peeled and the body moves
 * 16 bytes per access; otherwise 4-byte words or single bytes are used.
 */
__device__ __forceinline__ void copy_bytes(char* dst, const char* src, size_t bytes) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const uintptr_t d = reinterpret_cast<uintptr_t>(dst), s = reinterpret_cast<uintptr_t>(src);
    if (((d ^ s) & 15u) == 0) {
        size_t head = (16u - (d & 15u)) & 15u;
        if (head > bytes) head = bytes;
        for (size_t j = tid; j < head; j += nt) dst[j] = src[j];
        const size_t nv = (bytes - head) / 16;
        const uint4* sv = reinterpret_cast<const uint4*>(src + head);
        uint4* dv = reinterpret_cast<uint4*>(dst + head);
        size_t i = tid;
        for (; i + (size_t)(kUnroll - 1) * nt < nv; i += (size_t)kUnroll * nt) {
            uint4 v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) v[u] = sv[i + (size_t)u * nt];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) dv[i + (size_t)u * nt] = v[u];
        }
        for (; i < nv; i += nt) dv[i] = sv[i];
        for (size_t j = head + nv * 16 + tid; j < bytes; j += nt) dst[j] = src[j];
    } else if (((d | s) & 3u) == 0) {
        const size_t nw = bytes / 4;
        const uint32_t* sw = reinterpret_cast<const uint32_t*>(src);
        uint32_t* dw = reinterpret_cast<uint32_t*>(dst);
        for (size_t i = tid; i < nw; i += nt) dw[i] = sw[i];
        for (size_t j = nw * 4 + tid; j < bytes; j += nt) dst[j] = src[j];
    } else {
        for (size_t j = tid; j < bytes; j += nt) dst[j] = src[j];
    }
}

template <typename T>
__device__ __forceinline__ void copy_range(T* dst, const T* src, size_t n) {
    copy_bytes(reinterpret_cast<char*>(dst), reinterpret_cast<const char*>(src), n * sizeof(T));
}

/**
 * out[i] = finish(op(own[i], in_0[i], ..., in_{k-1}[i])) for i in [0,n), with up to two
 * destinations. `ins` are k additional sources (staging slots or peer buffers). The pointers carry no
 * __restrict__: an in-place call passes the same buffer as `own` and as a destination, and every thread reads the
 * vector it is about to overwrite before it writes it. Buffers that overlap only partly are not supported.
 */
template <typename T, int OP>
__device__ __forceinline__ void reduce_range(T* out0, T* out1, const T* own, const T* const* ins, int k, size_t n, bool avg, int world) {
    using A = typename Traits<T>::Acc;
    constexpr int N = Vec16<T>::N;
    const int tid = threadIdx.x, nt = blockDim.x;
    bool vec = aligned16(own) && aligned16(out0) && (out1 == nullptr || aligned16(out1));
    for (int s = 0; s < k; s++) vec = vec && aligned16(ins[s]);
    size_t done = 0;
    if (vec) {
        const size_t nv = n / N;
        for (size_t i = tid; i < nv; i += nt) {
            Vec16<T> v[kMaxPeers];
            v[0] = ld_vec<T>(own + i * N);
#pragma unroll
            for (int s = 0; s < kMaxPeers - 1; s++) if (s < k) v[s + 1] = ld_vec<T>(ins[s] + i * N);
            A acc[N];
#pragma unroll
            for (int e = 0; e < N; e++) acc[e] = Traits<T>::up(v[0].e[e]);
#pragma unroll
            for (int s = 0; s < kMaxPeers - 1; s++) {
                if (s < k) {
#pragma unroll
                    for (int e = 0; e < N; e++) acc[e] = op_apply<OP, A>(acc[e], Traits<T>::up(v[s + 1].e[e]));
                }
            }
            Vec16<T> r;
#pragma unroll
            for (int e = 0; e < N; e++) r.e[e] = Traits<T>::down(avg ? avg_finish<A>(acc[e], world) : acc[e]);
            st_vec<T>(out0 + i * N, r);
            if (out1) st_vec<T>(out1 + i * N, r);
        }
        done = nv * N;
    }
    for (size_t j = done + tid; j < n; j += nt) {
        A acc = Traits<T>::up(own[j]);
        for (int s = 0; s < k; s++) acc = op_apply<OP, A>(acc, Traits<T>::up(ins[s][j]));
        T r = Traits<T>::down(avg ? avg_finish<A>(acc, world) : acc);
        out0[j] = r;
        if (out1) out1[j] = r;
    }
}

/** Call f.template operator()<T, OP>() for the run-time (dtype, op) pair. */
#define DCCL_DISPATCH_OP(T, op, CALL)                                    \
    switch (op) {                                                        \
    case 0: case 4: { constexpr int OP = OP_SUM; CALL(T, OP); } break;   \
    case 1: { constexpr int OP = OP_PROD; CALL(T, OP); } break;          \
    case 2: { constexpr int OP = OP_MAX; CALL(T, OP); } break;           \
    default: { constexpr int OP = OP_MIN; CALL(T, OP); } break;          \
    }

#define DCCL_DISPATCH_TYPE_OP(dt, op, CALL)                                   \
    switch (dt) {                                                             \
    case 0: DCCL_DISPATCH_OP(int8_t, op, CALL) break;                         \
    case 1: DCCL_DISPATCH_OP(uint8_t, op, CALL) break;                        \
    case 2: DCCL_DISPATCH_OP(int32_t, op, CALL) break;                        \
    case 3: DCCL_DISPATCH_OP(uint32_t, op, CALL) break;                       \
    case 4: DCCL_DISPATCH_OP(long long, op, CALL) break;                      \
    case 5: DCCL_DISPATCH_OP(unsigned long long, op, CALL) break;             \
    case 6: DCCL_DISPATCH_OP(__half, op, CALL) break;                         \
    case 7: DCCL_DISPATCH_OP(float, op, CALL) break;                          \
    case 8: DCCL_DISPATCH_OP(double, op, CALL) break;                         \
    case 9: DCCL_DISPATCH_OP(__nv_bfloat16, op, CALL) break;                  \
    default: break;                                                           \
    }

} // namespace dccl
