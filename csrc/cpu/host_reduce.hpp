/**
 * Host-side element-wise reduction: acc[i] = op(acc[i], in[i]).
 *
 * Replaces do_host_reduce<DT> of the original (reference
 * src/core/internal_common.hpp:496-586). That version split the range into an
 * unaligned head, cache-line packs and a tail and was only right for aligned
 * destinations; here a plain loop over any pointer is left to the compiler's
 * vectoriser, so every alignment and every count is handled the same way.
 * fp16 and bf16 are reduced through float. ncclAvg accumulates like ncclSum;
 * the owner of a finished slice calls host_finish_avg() once.
 */
#pragma once
#include "../core/types.hpp"

namespace dccl {

template <typename T> struct HostSum  { static inline T f(T a, T b) { return (T)(a + b); } };
template <typename T> struct HostProd { static inline T f(T a, T b) { return (T)(a * b); } };
// max / min of floats: the other operand when one is NaN (a != a), like fmax / fmin and the device kernels
template <typename T> struct HostMax  { static inline T f(T a, T b) { return (a < b || a != a) ? b : a; } };
template <typename T> struct HostMin  { static inline T f(T a, T b) { return (b < a || a != a) ? b : a; } };

template <typename T, template <typename> class OP>
static inline void host_reduce_loop(T* __restrict__ acc, const T* __restrict__ in, size_t n) {
    for (size_t i = 0; i < n; i++) acc[i] = OP<T>::f(acc[i], in[i]);
}

template <typename T>
static inline ncclResult_t host_reduce_typed(T* acc, const T* in, size_t n, ncclRedOp_t op) {
    switch (op) {
    case ncclSum: case ncclAvg: host_reduce_loop<T, HostSum>(acc, in, n); return ncclSuccess;
    case ncclProd: host_reduce_loop<T, HostProd>(acc, in, n); return ncclSuccess;
    case ncclMax: host_reduce_loop<T, HostMax>(acc, in, n); return ncclSuccess;
    case ncclMin: host_reduce_loop<T, HostMin>(acc, in, n); return ncclSuccess;
    default: return ncclInvalidArgument;
    }
}

template <float (*TO)(uint16_t), uint16_t (*FROM)(float)>
static inline ncclResult_t host_reduce_16(uint16_t* acc, const uint16_t* in, size_t n, ncclRedOp_t op) {
    switch (op) {
    case ncclSum: case ncclAvg: for (size_t i = 0; i < n; i++) acc[i] = FROM(TO(acc[i]) + TO(in[i])); return ncclSuccess;
    case ncclProd: for (size_t i = 0; i < n; i++) acc[i] = FROM(TO(acc[i]) * TO(in[i])); return ncclSuccess;
    case ncclMax: for (size_t i = 0; i < n; i++) { float a = TO(acc[i]), b = TO(in[i]); acc[i] = FROM((a < b || a != a) ? b : a); } return ncclSuccess;
    case ncclMin: for (size_t i = 0; i < n; i++) { float a = TO(acc[i]), b = TO(in[i]); acc[i] = FROM((b < a || a != a) ? b : a); } return ncclSuccess;
    default: return ncclInvalidArgument;
    }
}

/** acc[i] = op(acc[i], in[i]) for n elements of type dt. */
inline ncclResult_t host_reduce(void* acc, const void* in, size_t n, ncclDataType_t dt, ncclRedOp_t op) {
    switch (dt) {
    case ncclInt8:    return host_reduce_typed<int8_t>((int8_t*)acc, (const int8_t*)in, n, op);
    case ncclUint8:   return host_reduce_typed<uint8_t>((uint8_t*)acc, (const uint8_t*)in, n, op);
    case ncclInt32:   return host_reduce_typed<int32_t>((int32_t*)acc, (const int32_t*)in, n, op);
    case ncclUint32:  return host_reduce_typed<uint32_t>((uint32_t*)acc, (const uint32_t*)in, n, op);
    case ncclInt64:   return host_reduce_typed<int64_t>((int64_t*)acc, (const int64_t*)in, n, op);
    case ncclUint64:  return host_reduce_typed<uint64_t>((uint64_t*)acc, (const uint64_t*)in, n, op);
    case ncclFloat32: return host_reduce_typed<float>((float*)acc, (const float*)in, n, op);
    case ncclFloat64: return host_reduce_typed<double>((double*)acc, (const double*)in, n, op);
    case ncclFloat16: return host_reduce_16<half_to_float, float_to_half>((uint16_t*)acc, (const uint16_t*)in, n, op);
    case ncclBfloat16: return host_reduce_16<bf16_to_float, float_to_bf16>((uint16_t*)acc, (const uint16_t*)in, n, op);
    default: return ncclInvalidArgument;
    }
}

/** Turn a finished sum over `world` ranks into the average (floats: times 1/world; integers: C++ division). */
inline void host_finish_avg(void* acc, size_t n, ncclDataType_t dt, uint32_t world) {
    switch (dt) {
    case ncclInt8:    { auto* p = (int8_t*)acc;   for (size_t i = 0; i < n; i++) p[i] = (int8_t)(p[i] / (int)world); break; }
    case ncclUint8:   { auto* p = (uint8_t*)acc;  for (size_t i = 0; i < n; i++) p[i] = (uint8_t)(p[i] / world); break; }
    case ncclInt32:   { auto* p = (int32_t*)acc;  for (size_t i = 0; i < n; i++) p[i] = p[i] / (int32_t)world; break; }
    case ncclUint32:  { auto* p = (uint32_t*)acc; for (size_t i = 0; i < n; i++) p[i] = p[i] / world; break; }
    case ncclInt64:   { auto* p = (int64_t*)acc;  for (size_t i = 0; i < n; i++) p[i] = p[i] / (int64_t)world; break; }
    case ncclUint64:  { auto* p = (uint64_t*)acc; for (size_t i = 0; i < n; i++) p[i] = p[i] / world; break; }
    case ncclFloat32: { auto* p = (float*)acc;  float s = 1.0f / (float)world; for (size_t i = 0; i < n; i++) p[i] *= s; break; }
    case ncclFloat64: { auto* p = (double*)acc; double s = 1.0 / (double)world; for (size_t i = 0; i < n; i++) p[i] *= s; break; }
    case ncclFloat16: { auto* p = (uint16_t*)acc; float s = 1.0f / (float)world; for (size_t i = 0; i < n; i++) p[i] = float_to_half(half_to_float(p[i]) * s); break; }
    case ncclBfloat16: { auto* p = (uint16_t*)acc; float s = 1.0f / (float)world; for (size_t i = 0; i < n; i++) p[i] = float_to_bf16(bf16_to_float(p[i]) * s); break; }
    default: break;
    }
}

} // namespace dccl
