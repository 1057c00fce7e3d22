/**
 * multimem.* wrappers: loads that return op(all ranks' copies) of a 16-byte vector
 * from a multicast address (reduced inside the NVSwitch) and stores that write a
 * vector to every rank, plus CTA-cooperative passes built from them. Shared by the
 * switch (NVLS) kernels. Forms accepted by the sm_100a assembler: add on f32 (v4),
 * add/min/max on bf16x2 and f16x2 (v4, fp32 accumulation for add), add on f64,
 * add/min/max on 32-bit integers, add on u64, min/max on 64-bit integers (scalar).
 */
#pragma once
#include "reduce_ops.cuh"

namespace dccl {

/* ---- 16-byte multimem accessors ---- */

#ifdef DCCL_HOST_SIM
/* Host simulation (make SIM=1): a multicast address is an address inside a reserved, inaccessible range that stands for
 * the same offset in every rank's memory; a reducing load folds the ranks' copies (16-bit floats in fp32 with one
 * rounding, as the switch does with .acc::f32), a store writes all of them. */
template <typename T, int OP> __device__ __forceinline__ uint4 mm_ld_reduce16(const char* mc) {
    using A = typename Traits<T>::Acc;
    constexpr int N = Vec16<T>::N;
    const ::dccl_sim::McMap* m = ::dccl_sim::mc_find(mc);
    const size_t off = (size_t)(mc - m->base);
    A acc[N];
    for (int r = 0; r < m->n; r++) {
        const Vec16<T> v = ld_vec<T>(m->mem[r] + off);
        for (int e = 0; e < N; e++) acc[e] = r == 0 ? Traits<T>::up(v.e[e]) : op_apply<OP, A>(acc[e], Traits<T>::up(v.e[e]));
    }
    Vec16<T> out;
    for (int e = 0; e < N; e++) out.e[e] = Traits<T>::down(acc[e]);
    return *reinterpret_cast<uint4*>(&out);
}
__device__ __forceinline__ void mm_st16(void* mc, uint4 v) {
    const ::dccl_sim::McMap* m = ::dccl_sim::mc_find(mc);
    const size_t off = (size_t)(static_cast<char*>(mc) - m->base);
    for (int r = 0; r < m->n; r++) *reinterpret_cast<uint4*>(m->mem[r] + off) = v;
}
#else

#define MM_LDRED_V4(NAME, INSTR)                                                                             \
    __device__ __forceinline__ uint4 NAME(const void* mc) {                                                  \
        uint4 v;                                                                                             \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " {%0,%1,%2,%3}, [%4];"                  \
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                     \
        return v;                                                                                            \
    }
MM_LDRED_V4(mm_add_f32x4, "add.v4.f32")
MM_LDRED_V4(mm_add_bf16x8, "add.acc::f32.v4.bf16x2")
MM_LDRED_V4(mm_min_bf16x8, "min.v4.bf16x2")
MM_LDRED_V4(mm_max_bf16x8, "max.v4.bf16x2")
MM_LDRED_V4(mm_add_f16x8, "add.acc::f32.v4.f16x2")
MM_LDRED_V4(mm_min_f16x8, "min.v4.f16x2")
MM_LDRED_V4(mm_max_f16x8, "max.v4.f16x2")
#undef MM_LDRED_V4

#define MM_LDRED_32(NAME, INSTR)                                                                             \
    __device__ __forceinline__ uint32_t NAME(const void* mc) {                                               \
        uint32_t v;                                                                                          \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v) : "l"(mc) : "memory"); \
        return v;                                                                                            \
    }
#define MM_LDRED_64(NAME, INSTR)                                                                             \
    __device__ __forceinline__ unsigned long long NAME(const void* mc) {                                     \
        unsigned long long v;                                                                                \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=l"(v) : "l"(mc) : "memory"); \
        return v;                                                                                            \
    }
MM_LDRED_32(mm_add_s32, "add.s32") MM_LDRED_32(mm_min_s32, "min.s32") MM_LDRED_32(mm_max_s32, "max.s32")
MM_LDRED_32(mm_add_u32, "add.u32") MM_LDRED_32(mm_min_u32, "min.u32") MM_LDRED_32(mm_max_u32, "max.u32")
MM_LDRED_64(mm_add_u64, "add.u64") MM_LDRED_64(mm_min_s64, "min.s64") MM_LDRED_64(mm_max_s64, "max.s64")
MM_LDRED_64(mm_min_u64, "min.u64") MM_LDRED_64(mm_max_u64, "max.u64")
#undef MM_LDRED_32
#undef MM_LDRED_64

__device__ __forceinline__ unsigned long long mm_add_f64(const void* mc) {
    unsigned long long v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f64 %0, [%1];" : "=l"(v) : "l"(mc) : "memory");
    return v;
}

__device__ __forceinline__ void mm_st16(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

/** op over all ranks of the 16 bytes at multicast address mc. */
template <typename T, int OP> __device__ __forceinline__ uint4 mm_ld_reduce16(const char* mc) {
    if constexpr (std::is_same<T, float>::value) return mm_add_f32x4(mc);
    else if constexpr (std::is_same<T, __nv_bfloat16>::value) return OP == OP_SUM ? mm_add_bf16x8(mc) : OP == OP_MAX ? mm_max_bf16x8(mc) : mm_min_bf16x8(mc);
    else if constexpr (std::is_same<T, __half>::value) return OP == OP_SUM ? mm_add_f16x8(mc) : OP == OP_MAX ? mm_max_f16x8(mc) : mm_min_f16x8(mc);
    else if constexpr (std::is_same<T, int32_t>::value) {
        uint4 v;
        v.x = OP == OP_SUM ? mm_add_s32(mc) : OP == OP_MAX ? mm_max_s32(mc) : mm_min_s32(mc);
        v.y = OP == OP_SUM ? mm_add_s32(mc + 4) : OP == OP_MAX ? mm_max_s32(mc + 4) : mm_min_s32(mc + 4);
        v.z = OP == OP_SUM ? mm_add_s32(mc + 8) : OP == OP_MAX ? mm_max_s32(mc + 8) : mm_min_s32(mc + 8);
        v.w = OP == OP_SUM ? mm_add_s32(mc + 12) : OP == OP_MAX ? mm_max_s32(mc + 12) : mm_min_s32(mc + 12);
        return v;
    } else if constexpr (std::is_same<T, uint32_t>::value) {
        uint4 v;
        v.x = OP == OP_SUM ? mm_add_u32(mc) : OP == OP_MAX ? mm_max_u32(mc) : mm_min_u32(mc);
        v.y = OP == OP_SUM ? mm_add_u32(mc + 4) : OP == OP_MAX ? mm_max_u32(mc + 4) : mm_min_u32(mc + 4);
        v.z = OP == OP_SUM ? mm_add_u32(mc + 8) : OP == OP_MAX ? mm_max_u32(mc + 8) : mm_min_u32(mc + 8);
        v.w = OP == OP_SUM ? mm_add_u32(mc + 12) : OP == OP_MAX ? mm_max_u32(mc + 12) : mm_min_u32(mc + 12);
        return v;
    } else {
        unsigned long long lo, hi;
        if constexpr (std::is_same<T, double>::value) { lo = mm_add_f64(mc); hi = mm_add_f64(mc + 8); }
        else if constexpr (std::is_same<T, long long>::value) {
            lo = OP == OP_SUM ? mm_add_u64(mc) : OP == OP_MAX ? mm_max_s64(mc) : mm_min_s64(mc);
            hi = OP == OP_SUM ? mm_add_u64(mc + 8) : OP == OP_MAX ? mm_max_s64(mc + 8) : mm_min_s64(mc + 8);
        } else {
            lo = OP == OP_SUM ? mm_add_u64(mc) : OP == OP_MAX ? mm_max_u64(mc) : mm_min_u64(mc);
            hi = OP == OP_SUM ? mm_add_u64(mc + 8) : OP == OP_MAX ? mm_max_u64(mc + 8) : mm_min_u64(mc + 8);
        }
        return make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
    }
}

#endif   // DCCL_HOST_SIM

/** Scale a reduced vector by 1/world (ncclAvg). */
template <typename T> __device__ __forceinline__ uint4 avg16(uint4 raw, int world) {
    using A = typename Traits<T>::Acc;
    Vec16<T> v = *reinterpret_cast<Vec16<T>*>(&raw);
#pragma unroll
    for (int e = 0; e < Vec16<T>::N; e++) v.e[e] = Traits<T>::down(avg_finish<A>(Traits<T>::up(v.e[e]), world));
    return *reinterpret_cast<uint4*>(&v);
}


/**
 * For every 16-byte vector i in [0,nv): out = finish(ld_reduce(src_mc + 16 i)), then
 * multimem.st to dst_mc and / or a plain store to dst_local (either may be null).
 * `valid_bytes` limits the plain store of the last vector (local destinations only).
 */
template <typename T, int OP, int kNvUnroll>
__device__ __forceinline__ void nvls_pass_u(const char* src_mc, char* dst_mc, char* dst_local, size_t nv, size_t valid_bytes, bool avg, int world) {
    const int tid = threadIdx.x, nt = blockDim.x;
    size_t i = tid;
    const size_t full = dst_local ? valid_bytes / 16 : nv;   // vectors that can be stored whole
    for (; i + (size_t)(kNvUnroll - 1) * nt < full; i += (size_t)kNvUnroll * nt) {
        uint4 v[kNvUnroll];
#pragma unroll
        for (int u = 0; u < kNvUnroll; u++) v[u] = mm_ld_reduce16<T, OP>(src_mc + (i + (size_t)u * nt) * 16);
#pragma unroll
        for (int u = 0; u < kNvUnroll; u++) {
            if (avg) v[u] = avg16<T>(v[u], world);
            if (dst_mc) mm_st16(dst_mc + (i + (size_t)u * nt) * 16, v[u]);
            if (dst_local) *reinterpret_cast<uint4*>(dst_local + (i + (size_t)u * nt) * 16) = v[u];
        }
    }
    for (; i < nv; i += nt) {
        uint4 v = mm_ld_reduce16<T, OP>(src_mc + i * 16);
        if (avg) v = avg16<T>(v, world);
        if (dst_mc) mm_st16(dst_mc + i * 16, v);
        if (dst_local) {
            if (i < full) *reinterpret_cast<uint4*>(dst_local + i * 16) = v;
            else {  // ragged end of a local destination: store only the bytes that belong to the message
                const unsigned char* b = reinterpret_cast<const unsigned char*>(&v);
                for (size_t k = 0; k < valid_bytes - i * 16; k++) dst_local[i * 16 + k] = (char)b[k];
            }
        }
    }
}

template <typename T, int OP>
__device__ __forceinline__ void nvls_pass(const char* src_mc, char* dst_mc, char* dst_local, size_t nv, size_t valid_bytes, bool avg, int world, int unroll = 4) {
    if (unroll >= 8) nvls_pass_u<T, OP, 8>(src_mc, dst_mc, dst_local, nv, valid_bytes, avg, world);
    else if (unroll >= 4) nvls_pass_u<T, OP, 4>(src_mc, dst_mc, dst_local, nv, valid_bytes, avg, world);
    else nvls_pass_u<T, OP, 2>(src_mc, dst_mc, dst_local, nv, valid_bytes, avg, world);
}

/** multimem.st of nv vectors read from local memory (src must be 16-byte aligned). */
__device__ __forceinline__ void nvls_push(char* dst_mc, const char* src, size_t nv) {
    constexpr int kNvUnroll = 4;
    const int tid = threadIdx.x, nt = blockDim.x;
    size_t i = tid;
    for (; i + (size_t)(kNvUnroll - 1) * nt < nv; i += (size_t)kNvUnroll * nt) {
        uint4 v[kNvUnroll];
#pragma unroll
        for (int u = 0; u < kNvUnroll; u++) v[u] = *reinterpret_cast<const uint4*>(src + (i + (size_t)u * nt) * 16);
#pragma unroll
        for (int u = 0; u < kNvUnroll; u++) mm_st16(dst_mc + (i + (size_t)u * nt) * 16, v[u]);
    }
    for (; i < nv; i += nt) mm_st16(dst_mc + i * 16, *reinterpret_cast<const uint4*>(src + i * 16));
}

} // namespace dccl
