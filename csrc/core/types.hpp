/**
 * Data-type and operator tables shared by the host and device sides.
 * Counterpart of size_of_type / ON_DCCL_DATATYPE in the original
 * (reference src/core/internal_common.hpp:314-413), but table driven and with
 * bfloat16 and fp16 present on both sides.
 */
#pragma once
#include <dccl/dccl.hpp>
#include <cstring>
#include <cstdint>

namespace dccl {

inline size_t size_of_type(ncclDataType_t t) {
    switch (t) {
    case ncclInt8: case ncclUint8: return 1;
    case ncclFloat16: case ncclBfloat16: return 2;
    case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
    case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
    default: return 0;
    }
}

inline const char* name_of_type(ncclDataType_t t) {
    static const char* n[] = {"int8","uint8","int32","uint32","int64","uint64",
                              "float16","float32","float64","bfloat16"};
    return (int)t >= 0 && (int)t < ncclNumTypes ? n[(int)t] : "?";
}

inline const char* name_of_op(ncclRedOp_t o) {
    static const char* n[] = {"sum","prod","max","min","avg"};
    return (int)o >= 0 && (int)o < ncclNumOps ? n[(int)o] : "?";
}

/** Parse a type name as the command-line tools spell it; returns ncclNumTypes when unknown. */
inline ncclDataType_t parse_type_name(const char* s) {
    for (int i = 0; i < ncclNumTypes; i++)
        if (std::strcmp(s, name_of_type((ncclDataType_t)i)) == 0) return (ncclDataType_t)i;
    if (!std::strcmp(s, "bf16")) return ncclBfloat16;
    if (!std::strcmp(s, "fp16") || !std::strcmp(s, "half")) return ncclFloat16;
    if (!std::strcmp(s, "fp32") || !std::strcmp(s, "float")) return ncclFloat32;
    if (!std::strcmp(s, "fp64") || !std::strcmp(s, "double")) return ncclFloat64;
    return ncclNumTypes;
}

/** Parse an operator name; returns ncclNumOps when unknown. */
inline ncclRedOp_t parse_op_name(const char* s) {
    for (int i = 0; i < ncclNumOps; i++)
        if (std::strcmp(s, name_of_op((ncclRedOp_t)i)) == 0) return (ncclRedOp_t)i;
    return ncclNumOps;
}

inline bool is_float_type(ncclDataType_t t) {
    return t == ncclFloat16 || t == ncclFloat32 || t == ncclFloat64 || t == ncclBfloat16;
}

/* ---- software half / bfloat16 conversion for the host backend ---- */
inline float bf16_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f;
}
inline uint16_t float_to_bf16(float f) {
    uint32_t u; std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);                                           // round to nearest even
    return (uint16_t)(u >> 16);
}
inline float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {  // subnormal: normalise
            int e = -1; do { e++; man <<= 1; } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112u) << 23) | (man << 13);
    float f; std::memcpy(&f, &u, 4); return f;
}
inline uint16_t float_to_half(float f) {
    uint32_t u; std::memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    int32_t exp = (int32_t)((u >> 23) & 0xffu) - 127 + 15;
    uint32_t man = u & 0x7fffffu;
    if (((u >> 23) & 0xffu) == 0xffu) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u | (man >> 13) : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half = man >> shift, rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13), rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

inline bool is_power_of_two(uint32_t x) { return x && !(x & (x - 1)); }

/** floor(log2(x)) for x >= 1. */
inline uint32_t log_two(uint32_t x) { uint32_t e = 0; while (x >>= 1) e++; return e; }

/** Reverse the low `bits` bits of x (owner of a slice after recursive halving). */
inline uint32_t reverse_bits(uint32_t x, uint32_t bits) {
    uint32_t r = 0;
    for (uint32_t i = 0; i < bits; i++) if (x & (1u << i)) r |= 1u << (bits - 1 - i);
    return r;
}

/** Element range [lo,hi) of slot `i` when `count` elements are split over `n` slots.
 *  Slot boundaries are rounded to `align` elements so that vector accesses stay
 *  aligned; the last slot takes the remainder. Works for any count (the original
 *  required count % world == 0, reference all_reduce_ring.cpp:51-55). */
inline void slot_range(size_t count, uint32_t n, uint32_t i, size_t align, size_t* lo, size_t* hi) {
    size_t per = (count + n - 1) / n;
    if (align > 1) per = (per + align - 1) / align * align;
    size_t l = per * i, h = per * (i + 1);
    if (l > count) l = count;
    if (h > count) h = count;
    *lo = l; *hi = h;
}

} // namespace dccl
