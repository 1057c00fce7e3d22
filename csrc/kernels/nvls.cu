/**
 * Collectives that reduce and replicate inside the NVSwitch (NVLS):
 * multimem.ld_reduce returns op(all ranks' copies) of a 16-byte vector in one
 * load from the multicast address, multimem.st writes a vector to every rank.
 *
 *   all-reduce      each rank owns 1/n of the vector: ld_reduce its shard, apply
 *                   the 1/world scale of ncclAvg, multimem.st the result to all
 *   reduce-scatter  ld_reduce the own shard straight into the receive buffer
 *   all-gather      multimem.st the own slot to every rank
 *   broadcast       the root multimem.st's the message
 *   reduce          the root ld_reduce's the message
 *
 * This is the switch-side counterpart of the original's ordered multicast plus
 * host reduction (reference src/core/dccl.cpp:701-846); per GPU the links carry
 * about (1 + 1/n) S instead of 2 (n-1)/n S for an all-reduce of S bytes.
 *
 * Two buffer modes. "staged": user buffers are ordinary device memory; the
 * kernel copies the input into the multicast-bound staging half (local HBM
 * traffic only), and copies the result out after the switch pass.
 * "symmetric": the user buffers themselves live in multicast-bound symmetric
 * memory (dcclMemAlloc), the kernel touches them directly and nothing is
 * copied; a leading barrier makes sure every peer has reached the call and a
 * trailing one that nobody still reads a buffer when the call returns.
 *
 * Supported by the hardware instruction, checked by nvls_supports(): sum / avg
 * on fp32, fp64, fp16, bf16 (16-bit types accumulate in fp32), min / max on
 * fp16, bf16, and sum / avg / min / max on 32- and 64-bit integers. Everything
 * else (prod, 8-bit types, fp32/fp64 min/max) is served by the peer-to-peer
 * variants.
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"
#include "../device/geometry.cuh"
#include "../device/multimem.cuh"

namespace dccl {

template <typename T, int OP>
__device__ __forceinline__ void nvls_body(const CollArgs& a, const Ctx& x) {
    constexpr size_t ES = sizeof(T);
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank, mode = a.mode;
    const T* send = reinterpret_cast<const T*>(x.io->send);
    T* recv = reinterpret_cast<T*>(x.io->recv);
    const bool slots = mode == NV_REDUCESCATTER || mode == NV_ALLGATHER;
    const Geometry<T> g(slots ? GEO_SLOTS : GEO_SPLIT, a.count, n, x.bid, x.nb);
    const size_t stride = slots ? a.stride : g.per;
    const bool avg = a.op == (int)ncclAvg;
    const size_t stage_off = kStageOff + (size_t)x.parity * c.stage_bytes;
    T* my_stage = reinterpret_cast<T*>(c.pool[r] + stage_off);
    char* mc_stage = c.mc_pool + stage_off;
    if (!a.symmetric && !stage_extent_ok<T>(c, (size_t)n * g.slot_stride, 1907)) return;   // one slot per rank
    auto lo_of = [&](int j) { size_t l = g.len(j); return g.blo < l ? g.blo : l; };
    auto hi_of = [&](int j) { size_t l = g.len(j); return g.bhi < l ? g.bhi : l; };
    auto vecs = [&](size_t elems) { return (elems * ES + 15) / 16; };

    if (a.symmetric) {
        /* ---- user buffers are multicast-bound: no copies ---- */
        const char* send_mc = x.io->send_mc;
        char* recv_mc = x.io->recv_mc;
        if (!rank_barrier(c, x.bid, x.seq, 0, 400 + mode)) return;
        if (mode == NV_ALLREDUCE) {
            const size_t lo = lo_of(r), hi = hi_of(r);
            if (hi > lo) nvls_pass<T, OP>(send_mc + ((size_t)r * stride + lo) * ES, recv_mc + ((size_t)r * stride + lo) * ES, nullptr, vecs(hi - lo), 0, avg, n, a.unroll);
        } else if (mode == NV_REDUCESCATTER) {
            const size_t lo = lo_of(r), hi = hi_of(r);
            if (hi > lo) nvls_pass<T, OP>(send_mc + ((size_t)r * stride + lo) * ES, nullptr, reinterpret_cast<char*>(recv + lo), vecs(hi - lo), (hi - lo) * ES, avg, n);
        } else if (mode == NV_ALLGATHER) {
            const size_t lo = lo_of(r), hi = hi_of(r);
            if (hi > lo) {
                if (aligned16(send + lo)) nvls_push(recv_mc + ((size_t)r * stride + lo) * ES, reinterpret_cast<const char*>(send + lo), vecs(hi - lo));
                else {
                    // a source that is not 16-byte aligned (only this rank knows): through the own slot of the receive
                    // buffer, which is, then from there to every rank
                    T* own = recv + (size_t)r * stride + lo;
                    copy_range<T>(own, send + lo, hi - lo);
                    __syncthreads();
                    nvls_push(recv_mc + ((size_t)r * stride + lo) * ES, reinterpret_cast<const char*>(own), vecs(hi - lo));
                }
            }
        } else if (mode == NV_BROADCAST) {
            if (r == a.root)
                for (int j = 0; j < n; j++) {
                    const size_t lo = lo_of(j), hi = hi_of(j);
                    if (hi > lo) nvls_push(recv_mc + ((size_t)j * stride + lo) * ES, reinterpret_cast<const char*>(send + (size_t)j * stride + lo), vecs(hi - lo));
                }
        } else {  // NV_REDUCE
            if (r == a.root)
                for (int j = 0; j < n; j++) {
                    const size_t lo = lo_of(j), hi = hi_of(j);
                    if (hi > lo) nvls_pass<T, OP>(send_mc + ((size_t)j * stride + lo) * ES, nullptr, reinterpret_cast<char*>(recv + (size_t)j * stride + lo), vecs(hi - lo), (hi - lo) * ES, avg, n);
                }
        }
        rank_barrier(c, x.bid, x.seq, 1, 450 + mode);
        return;
    }

    /* ---- staged: copy in (local), switch pass, copy out (local) ---- */
    if (mode == NV_ALLREDUCE || mode == NV_REDUCESCATTER || mode == NV_REDUCE) {
        for (int j = 0; j < n; j++) {
            const size_t lo = lo_of(j), hi = hi_of(j);
            if (hi > lo) copy_range<T>(my_stage + (size_t)j * g.slot_stride + lo, send + (size_t)j * stride + lo, hi - lo);
        }
    } else if (mode == NV_ALLGATHER) {
        // own slot: through a local copy when the source is not 16-byte aligned, else straight to all ranks
        const size_t lo = lo_of(r), hi = hi_of(r);
        if (hi > lo) {
            if (aligned16(send + lo)) nvls_push(mc_stage + ((size_t)r * g.slot_stride + lo) * ES, reinterpret_cast<const char*>(send + lo), vecs(hi - lo));
            else {
                copy_range<T>(my_stage + (size_t)r * g.slot_stride + lo, send + lo, hi - lo);
                __syncthreads();
                nvls_push(mc_stage + ((size_t)r * g.slot_stride + lo) * ES, reinterpret_cast<const char*>(my_stage + (size_t)r * g.slot_stride + lo), vecs(hi - lo));
            }
        }
    } else {  // NV_BROADCAST
        if (r == a.root)
            for (int j = 0; j < n; j++) {
                const size_t lo = lo_of(j), hi = hi_of(j);
                if (hi <= lo) continue;
                const T* src = send + (size_t)j * stride + lo;
                if (aligned16(src)) nvls_push(mc_stage + ((size_t)j * g.slot_stride + lo) * ES, reinterpret_cast<const char*>(src), vecs(hi - lo));
                else {
                    copy_range<T>(my_stage + (size_t)j * g.slot_stride + lo, src, hi - lo);
                    __syncthreads();
                    nvls_push(mc_stage + ((size_t)j * g.slot_stride + lo) * ES, reinterpret_cast<const char*>(my_stage + (size_t)j * g.slot_stride + lo), vecs(hi - lo));
                }
            }
    }
    if (!rank_barrier(c, x.bid, x.seq, 0, 500 + mode)) return;

    if (mode == NV_ALLREDUCE) {
        const size_t lo = lo_of(r), hi = hi_of(r);
        if (hi > lo) {
            const size_t off = ((size_t)r * g.slot_stride + lo) * ES;
            nvls_pass<T, OP>(mc_stage + off, mc_stage + off, nullptr, vecs(hi - lo), 0, avg, n, a.unroll);
        }
        if (!rank_barrier(c, x.bid, x.seq, 1, 550 + mode)) return;
    } else if (mode == NV_REDUCESCATTER) {
        const size_t lo = lo_of(r), hi = hi_of(r);
        if (hi > lo) {
            char* dst = reinterpret_cast<char*>(recv + lo);
            if (aligned16(dst)) nvls_pass<T, OP>(mc_stage + ((size_t)r * g.slot_stride + lo) * ES, nullptr, dst, vecs(hi - lo), (hi - lo) * ES, avg, n);
            else {  // unaligned output: reduce into the own staging slot, then copy
                char* tmp = reinterpret_cast<char*>(my_stage + (size_t)r * g.slot_stride + lo);
                // peers only read this slot through the switch during their own pass over THEIR shard, never this one
                nvls_pass<T, OP>(mc_stage + ((size_t)r * g.slot_stride + lo) * ES, nullptr, tmp, vecs(hi - lo), vecs(hi - lo) * 16, avg, n);
                __syncthreads();
                copy_range<T>(recv + lo, reinterpret_cast<const T*>(tmp), hi - lo);
            }
        }
        return;
    } else if (mode == NV_REDUCE) {
        if (r == a.root)
            for (int j = 0; j < n; j++) {
                const size_t lo = lo_of(j), hi = hi_of(j);
                if (hi <= lo) continue;
                char* dst = reinterpret_cast<char*>(recv + (size_t)j * stride + lo);
                const char* src = mc_stage + ((size_t)j * g.slot_stride + lo) * ES;
                if (aligned16(dst)) nvls_pass<T, OP>(src, nullptr, dst, vecs(hi - lo), (hi - lo) * ES, avg, n);
                else {
                    // element-wise: one element per ld_reduce would need per-type scalar forms; go through registers
                    const int tid = threadIdx.x, nt = blockDim.x;
                    for (size_t i = tid; i < vecs(hi - lo); i += nt) {
                        uint4 v = mm_ld_reduce16<T, OP>(src + i * 16);
                        if (avg) v = avg16<T>(v, n);
                        const T* e = reinterpret_cast<const T*>(&v);
                        for (size_t k = 0; k < 16 / ES && i * (16 / ES) + k < hi - lo; k++) reinterpret_cast<T*>(dst)[i * (16 / ES) + k] = e[k];
                    }
                }
            }
        return;
    }

    /* copy out: all-reduce, all-gather, broadcast */
    if (mode == NV_BROADCAST && r == a.root) {
        if (recv != send)
            for (int j = 0; j < n; j++) {
                const size_t lo = lo_of(j), hi = hi_of(j);
                if (hi > lo) copy_range<T>(recv + (size_t)j * stride + lo, send + (size_t)j * stride + lo, hi - lo);
            }
        return;
    }
    for (int j = 0; j < n; j++) {
        const size_t lo = lo_of(j), hi = hi_of(j);
        if (hi <= lo) continue;
        if (mode == NV_ALLGATHER && j == r) {
            if (recv + (size_t)r * stride != send) copy_range<T>(recv + (size_t)r * stride + lo, send + lo, hi - lo);
            continue;
        }
        copy_range<T>(recv + (size_t)j * stride + lo, my_stage + (size_t)j * g.slot_stride + lo, hi - lo);
    }
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_nvls(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    nvls_body<T, OP>(a, x);
    finish_call(x);
}

bool nvls_supports(ncclDataType_t dt, ncclRedOp_t op) {
    const bool sum = op == ncclSum || op == ncclAvg, mm = op == ncclMax || op == ncclMin;
    switch (dt) {
    case ncclFloat32: case ncclFloat64: return sum;
    case ncclFloat16: case ncclBfloat16: return sum || mm;
    case ncclInt32: case ncclUint32: case ncclInt64: case ncclUint64: return sum || mm;
    default: return false;
    }
}

size_t nvls_capacity(int mode, int nranks, size_t es, size_t stage_bytes) {
    const size_t ve = 16 / es, stage_elems = stage_bytes / es, n = (size_t)nranks;
    auto floor_ve = [&](size_t x) { return x / ve * ve; };
    if (mode == NV_REDUCESCATTER || mode == NV_ALLGATHER) return floor_ve(stage_elems / n);   // per-rank count
    return n * floor_ve(stage_elems / n);
}

cudaError_t launch_nvls(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg) {
    if (a.mode == NV_ALLGATHER || a.mode == NV_BROADCAST) {
        // data movement only: any element type moves as 32-bit words or bytes
        const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                          : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
        CollArgs b = a;
        b.count = a.count * es;
        b.stride = a.stride * es;
        b.op = (int)ncclSum;
        return launch_coll(k_nvls<uint8_t, OP_SUM>, b, cfg);
    }
    const int op = a.op == (int)ncclAvg ? (int)ncclSum : a.op;
    switch (dt) {
#define NV_CASE(DT, T)                                                                      \
    case DT:                                                                                \
        if (op == (int)ncclSum) return launch_coll(k_nvls<T, OP_SUM>, a, cfg);              \
        if (op == (int)ncclMax) return launch_coll(k_nvls<T, OP_MAX>, a, cfg);              \
        if (op == (int)ncclMin) return launch_coll(k_nvls<T, OP_MIN>, a, cfg);              \
        break;
#define NV_CASE_SUM(DT, T)                                                                  \
    case DT:                                                                                \
        if (op == (int)ncclSum) return launch_coll(k_nvls<T, OP_SUM>, a, cfg);              \
        break;
    NV_CASE_SUM(ncclFloat32, float)
    NV_CASE_SUM(ncclFloat64, double)
    NV_CASE(ncclFloat16, __half)
    NV_CASE(ncclBfloat16, __nv_bfloat16)
    NV_CASE(ncclInt32, int32_t)
    NV_CASE(ncclUint32, uint32_t)
    NV_CASE(ncclInt64, long long)
    NV_CASE(ncclUint64, unsigned long long)
#undef NV_CASE
#undef NV_CASE_SUM
    default: break;
    }
    return cudaErrorInvalidValue;
}

} // namespace dccl
