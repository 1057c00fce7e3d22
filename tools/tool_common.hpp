/**
 * Shared pieces of the command-line tools: hex dump in the layout of the
 * original's save_mem (reference src/application/utils.cpp:6-33: 32 bytes per
 * line, "0x%08x: " offsets, double space every 8 bytes), seeded buffer
 * initialisation and a serial reference fold for --verify.
 */
#pragma once
#include <dccl/dccl.hpp>
#include "../csrc/core/types.hpp"
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace dccl_tools {
using namespace dccl;

inline void save_mem(const void* ptr, size_t size, const std::string& fname) {
    FILE* f = fopen(fname.c_str(), "w");
    if (!f) return;
    const uint8_t* p = (const uint8_t*)ptr;
    for (size_t off = 0; off < size;) {
        if (off % 32 == 0) fprintf(f, "0x%08zx: ", off);
        fprintf(f, "%02x", p[off]);
        off++;
        if (off % 32 == 0) fputc('\n', f);
        else if (off % 8 == 0) fputs("  ", f);
        else fputc(' ', f);
    }
    fclose(f);
}

struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0xD1B54A32D192ED03ull) {}
    uint64_t next() { uint64_t z = (s += 0x9E3779B97F4A7C15ull); z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31); }
    double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }          // [0,1)
    double normal() { double u = uniform(), v = uniform(); if (u < 1e-300) u = 1e-300; return std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586 * v); }
};

enum InitMode { INIT_BYTES, INIT_UNIFORM, INIT_NORMAL };

inline void store_value(void* buf, size_t i, ncclDataType_t dt, double v) {
    switch (dt) {
    case ncclInt8: ((int8_t*)buf)[i] = (int8_t)v; break;
    case ncclUint8: ((uint8_t*)buf)[i] = (uint8_t)v; break;
    case ncclInt32: ((int32_t*)buf)[i] = (int32_t)v; break;
    case ncclUint32: ((uint32_t*)buf)[i] = (uint32_t)v; break;
    case ncclInt64: ((int64_t*)buf)[i] = (int64_t)v; break;
    case ncclUint64: ((uint64_t*)buf)[i] = (uint64_t)v; break;
    case ncclFloat16: ((uint16_t*)buf)[i] = float_to_half((float)v); break;
    case ncclBfloat16: ((uint16_t*)buf)[i] = float_to_bf16((float)v); break;
    case ncclFloat32: ((float*)buf)[i] = (float)v; break;
    case ncclFloat64: ((double*)buf)[i] = v; break;
    default: break;
    }
}

inline double load_value(const void* buf, size_t i, ncclDataType_t dt) {
    switch (dt) {
    case ncclInt8: return ((const int8_t*)buf)[i];
    case ncclUint8: return ((const uint8_t*)buf)[i];
    case ncclInt32: return ((const int32_t*)buf)[i];
    case ncclUint32: return ((const uint32_t*)buf)[i];
    case ncclInt64: return (double)((const int64_t*)buf)[i];
    case ncclUint64: return (double)((const uint64_t*)buf)[i];
    case ncclFloat16: return half_to_float(((const uint16_t*)buf)[i]);
    case ncclBfloat16: return bf16_to_float(((const uint16_t*)buf)[i]);
    case ncclFloat32: return ((const float*)buf)[i];
    case ncclFloat64: return ((const double*)buf)[i];
    default: return 0;
    }
}

/** Fill `count` elements the way rank `rank` does: bytes = memset(rank) like the original;
 *  uniform = U[-1,1] for floats / U[-1000,1000] for integers (unsigned: [0,1000]); normal = N(0,1). */
inline void fill_buffer(void* buf, size_t count, ncclDataType_t dt, InitMode mode, uint64_t seed, int rank) {
    if (mode == INIT_BYTES) { memset(buf, rank, count * size_of_type(dt)); return; }
    Rng rng(seed);
    const bool flt = is_float_type(dt);
    const bool uns = dt == ncclUint8 || dt == ncclUint32 || dt == ncclUint64;
    const bool tiny = dt == ncclInt8 || dt == ncclUint8;
    for (size_t i = 0; i < count; i++) {
        double v;
        if (flt) v = mode == INIT_UNIFORM ? rng.uniform() * 2.0 - 1.0 : rng.normal();
        else {
            double span = tiny ? 12.0 : 1000.0;
            v = std::floor(uns ? rng.uniform() * (span + 1) : rng.uniform() * (2 * span + 1) - span);
        }
        store_value(buf, i, dt, v);
    }
}

/** Serial fold of per-rank inputs (element i of every rank) the way the API defines the result. */
inline void reference_fold(const std::vector<std::vector<char>>& in, size_t count, ncclDataType_t dt, ncclRedOp_t op, void* out) {
    const size_t n = in.size();
    const bool flt = is_float_type(dt);
    for (size_t i = 0; i < count; i++) {
        if (flt) {
            double acc = load_value(in[0].data(), i, dt);
            for (size_t r = 1; r < n; r++) {
                double v = load_value(in[r].data(), i, dt);
                switch (op) {
                case ncclSum: case ncclAvg: acc += v; break;
                case ncclProd: acc *= v; break;
                case ncclMax: acc = acc < v ? v : acc; break;
                case ncclMin: acc = v < acc ? v : acc; break;
                default: break;
                }
            }
            if (op == ncclAvg) acc /= (double)n;
            store_value(out, i, dt, acc);
        } else {
            // integers: wrap-around arithmetic in the element width, division for avg
            const bool uns = dt == ncclUint8 || dt == ncclUint32 || dt == ncclUint64;
            const size_t es = size_of_type(dt);
            auto ld = [&](size_t r) -> uint64_t {
                uint64_t u = 0; memcpy(&u, in[r].data() + i * es, es);
                if (!uns && es < 8 && (u >> (8 * es - 1))) u |= ~0ull << (8 * es);   // sign extend
                return u;
            };
            auto wrap = [&](uint64_t u) -> uint64_t {
                if (es == 8) return u;
                u &= (1ull << (8 * es)) - 1;
                if (!uns && (u >> (8 * es - 1))) u |= ~0ull << (8 * es);
                return u;
            };
            uint64_t acc = ld(0);
            for (size_t r = 1; r < n; r++) {
                uint64_t v = ld(r);
                switch (op) {
                case ncclSum: case ncclAvg: acc = wrap(acc + v); break;
                case ncclProd: acc = wrap(acc * v); break;
                case ncclMax: acc = uns ? (acc < v ? v : acc) : ((int64_t)acc < (int64_t)v ? v : acc); break;
                case ncclMin: acc = uns ? (v < acc ? v : acc) : ((int64_t)v < (int64_t)acc ? v : acc); break;
                default: break;
                }
            }
            if (op == ncclAvg) acc = uns ? acc / n : (uint64_t)((int64_t)acc / (int64_t)n);
            memcpy((char*)out + i * es, &acc, es);
        }
    }
}

/** Compare got with want; returns the number of mismatches and prints the first few. */
inline size_t compare_buffers(const void* got, const void* want, size_t count, ncclDataType_t dt, int world, const char* what) {
    size_t bad = 0;
    double rtol, atol;
    switch (dt) {
    case ncclFloat32: rtol = 1e-5; atol = 1e-6 * world; break;
    case ncclFloat64: rtol = 1e-12; atol = 1e-13 * world; break;
    case ncclFloat16: rtol = 4e-3; atol = 4e-3 * world; break;
    case ncclBfloat16: rtol = 2e-2; atol = 2e-2 * world; break;
    default: rtol = 0; atol = 0; break;
    }
    for (size_t i = 0; i < count; i++) {
        double g = load_value(got, i, dt), w = load_value(want, i, dt);
        bool ok = is_float_type(dt) ? (std::fabs(g - w) <= atol + rtol * std::fabs(w) || (std::isnan(g) && std::isnan(w)))
                                    : memcmp((const char*)got + i * size_of_type(dt), (const char*)want + i * size_of_type(dt), size_of_type(dt)) == 0;
        if (!ok && bad++ < 5) fprintf(stderr, "verify %s: element %zu is %.9g, expected %.9g\n", what, i, g, w);
    }
    return bad;
}

} // namespace dccl_tools
