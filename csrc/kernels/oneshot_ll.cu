/**
 * One-shot all-reduce for small messages with the flag carried inside the data.
 *
 * Each rank pushes its whole input to every peer as 16-byte packets
 * {data0, tag, data1, tag} (8 payload bytes + two copies of this call's
 * sequence number, each 8-byte half stored atomically), then polls the packets
 * that arrive in its own pool, reduces all ranks' values in rank order and
 * writes the result. There is no separate barrier and no second round trip:
 * one kernel launch and one NVLink crossing per call, which is what the
 * latency-bound end of the sweep needs. (The ring of the original costs
 * 2(n-1) network round trips plus n host syncs at any size, reference
 * src/core/all_reduce_ring.cpp:8-79.) All ranks add in the same order, so all
 * ranks get bit-identical results. Packets alternate between two generations
 * of the packet region, so a fast rank can start the next call while a slow
 * one still reads the previous one.
 */
#include "kernels.hpp"
#include "../device/reduce_ops.cuh"

namespace dccl {

size_t oneshot_ll_capacity_bytes() { return kLLMaxPayload; }

__device__ __forceinline__ char* ll_slot(const DevComm& c, int owner, int parity, int src) {
    return c.pool[owner] + kLLOff + ((size_t)parity * kMaxPeers + (size_t)src) * kLLSlotBytes;
}

template <typename T, int OP>
__device__ __forceinline__ void oneshot_ll_body(const CollArgs& a, const Ctx& x) {
    using A = typename Traits<T>::Acc;
    constexpr int N = 8 / (int)sizeof(T);
    const DevComm& c = *x.c;
    const int n = c.nranks, r = c.rank;
    const char* send = reinterpret_cast<const char*>(x.io->send);
    char* recv = reinterpret_cast<char*>(x.io->recv);
    const size_t nbytes = a.count * sizeof(T);
    const size_t npk = (nbytes + 7) / 8;
    const uint32_t tag = x.seq;
    const bool avg = a.op == (int)ncclAvg;
    if (!DCCL_BOUNDS_OK(c, npk * 16 <= kLLSlotBytes, 1903, npk)) return;   // one packet slot per source rank
    const bool fast_in = (reinterpret_cast<uintptr_t>(send) & 7u) == 0, fast_out = (reinterpret_cast<uintptr_t>(recv) & 7u) == 0;

    for (size_t i = (size_t)x.bid * blockDim.x + threadIdx.x; i < npk; i += (size_t)x.nb * blockDim.x) {
        const size_t off = i * 8;
        const int valid = nbytes - off >= 8 ? 8 : (int)(nbytes - off);
        union { uint2 u; T e[N]; unsigned char b[8]; } mine;
        mine.u = make_uint2(0u, 0u);
        if (fast_in && valid == 8) mine.u = *reinterpret_cast<const uint2*>(send + off);
        else for (int k = 0; k < valid; k++) mine.b[k] = (unsigned char)send[off + k];

        const uint4 pkt = make_uint4(mine.u.x, tag, mine.u.y, tag);
        for (int k = 1; k < n; k++) {
            const int p = (r + k) % n;
            st_volatile_v4(ll_slot(c, p, x.parity, r) + i * 16, pkt);
        }

        A acc[N];
        bool first = true, ok = true;
        for (int p = 0; p < n && ok; p++) {
            union { uint2 u; T e[N]; } theirs;
            if (p == r) theirs.u = mine.u;
            else {
                const char* slot = ll_slot(c, r, x.parity, p) + i * 16;
                uint4 v = ld_volatile_v4(slot);
                uint32_t spins = 0;
                unsigned long long t0 = 0;
                while (v.y != tag || v.w != tag) {
                    if ((++spins & 0xffu) == 0) {
                        unsigned long long now = global_timer_ns();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > c.timeout_ns) { report_failure(c, DEV_TIMEOUT, p, 300, x.seq); ok = false; break; }
                        if ((spins & 0xfffu) == 0 && ld_volatile_u32(c.abort_word) != 0) { report_failure(c, DEV_ABORTED, p, 300, x.seq); ok = false; break; }
                    }
                    v = ld_volatile_v4(slot);
                }
                theirs.u = make_uint2(v.x, v.z);
            }
            if (first) {
#pragma unroll
                for (int e = 0; e < N; e++) acc[e] = Traits<T>::up(theirs.e[e]);
                first = false;
            } else {
#pragma unroll
                for (int e = 0; e < N; e++) acc[e] = op_apply<OP, A>(acc[e], Traits<T>::up(theirs.e[e]));
            }
        }
        if (!ok) return;
        union { uint2 u; T e[N]; unsigned char b[8]; } out;
#pragma unroll
        for (int e = 0; e < N; e++) out.e[e] = Traits<T>::down(avg ? avg_finish<A>(acc[e], n) : acc[e]);
        if (fast_out && valid == 8) *reinterpret_cast<uint2*>(recv + off) = out.u;
        else for (int k = 0; k < valid; k++) recv[off + k] = (char)out.b[k];
    }
}

template <typename T, int OP>
__global__ void __launch_bounds__(512) k_oneshot_ll(const __grid_constant__ CollArgs a) {
    const Ctx x = make_ctx(a);
    oneshot_ll_body<T, OP>(a, x);
    finish_call(x);
}

cudaError_t launch_oneshot_ll(const CollArgs& a, ncclDataType_t dt, const LaunchCfg& cfg_in) {
    LaunchCfg cfg = cfg_in;
    const size_t es = dt == ncclInt8 || dt == ncclUint8 ? 1 : dt == ncclFloat16 || dt == ncclBfloat16 ? 2
                      : dt == ncclInt32 || dt == ncclUint32 || dt == ncclFloat32 ? 4 : 8;
    const size_t npk = (a.count * es + 7) / 8;
    // every rank derives the same shape from the same arguments
    int threads = (int)((npk + 31) / 32 * 32);
    if (threads > 512) threads = 512;
    if (threads < 32) threads = 32;
    int ctas = (int)((npk + threads - 1) / threads);
    if (ctas > cfg.ctas) ctas = cfg.ctas;
    if (ctas < 1) ctas = 1;
    cfg.threads = threads;
    cfg.ctas = ctas;
#define CALL(T, OP) return launch_coll(k_oneshot_ll<T, OP>, a, cfg)
    DCCL_DISPATCH_TYPE_OP((int)dt, a.op, CALL)
#undef CALL
    return cudaErrorInvalidValue;
}

} // namespace dccl
