/**
 * Single-GPU emulation of a multi-rank communicator, for tests.
 *
 * The collective kernels take their rank from the CTA index when an array of
 * per-rank views is passed, so ONE cooperative launch of ranks x ctas CTAs
 * plays every rank on one GPU: each virtual rank gets its own pool and its own
 * user buffers in ordinary device memory, "peer" pointers simply point at the
 * other virtual ranks' pools. The code path inside the kernels (flags,
 * barriers, staging halves, packets, reduction) is exactly the multi-GPU one;
 * only the multimem (NVSwitch) variants cannot be played this way. Ranks that
 * wait on each other never run as separate launches here: the cooperative
 * launch guarantees all CTAs are resident.
 */
#include "../kernels/kernels.hpp"
#include "../core/types.hpp"
#include "gpu_comm.hpp"
#include "canary.hpp"
#include <cstdio>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

using namespace dccl;

namespace {

// set by dccl_emu_set_device_seq: the virtual ranks keep their sequence numbers in device counters
int g_device_seq = 0;
// set by dccl_emu_set_peer_buffers: the user buffers count as addressable by every rank (symmetric / registered
// memory), so that the two-shot all-reduce takes its zero-copy form
int g_peer_buffers = 0;
int g_bcast_chunks = 0;
// set by dccl_emu_set_mix: (collective, variant) pairs launched before every call under test
std::vector<std::pair<int, GpuAlgo>> g_mix;
// set by dccl_emu_set_guard: guard words in the unused parts of every virtual rank's pool, checked after each run
int g_guard = 0;
// set by dccl_emu_declare_stage_bytes (range-checking builds only): the staging size the kernels are TOLD, smaller
// than what is allocated, so that their range checks can be seen to refuse a call while every address they could
// compute still lies inside the allocation
#ifdef DCCL_DEBUG_BOUNDS
size_t g_declared_stage = 0;
#endif
#ifdef DCCL_HOST_SIM
// Host simulation only (a single GPU has no NVSwitch to play): which switch kernel serves algorithm "nvls".
// 0 staged (nvls.cu), 1 pipelined all-reduce / reduce-scatter (nvls_pipe.cu), 2 pipelined broadcast / reduce (nvls_rooted.cu)
int g_switch_form = 0;
int g_pipe_nv = 0;
int g_pipe_teams = 2;      // dccl_emu_set_pipe(chunk, 100 * teams + switch CTAs)

#endif
// set by dccl_emu_set_p2p_rendezvous: how large send / recv messages of the emulated ranks travel.
// 0 FIFO only; 1 rendezvous, every receive buffer is mapped by its sender (zero-copy); 2 rendezvous, no buffer is
// mapped (every sender answers "FIFO"); 3 rendezvous, only the buffers of even ranks are mapped (both paths in one launch)
int g_p2p_rdv = 0;

/** Fill the rendezvous fields of the emulated ranks' operations (per pair and direction: large messages are numbered in
 *  the order of the operations) and the table of mappings: with all ranks in one address space a buffer is "mapped" at
 *  its own address. `rdv_base[src][dst]`: large messages of earlier launches. */
void emu_rendezvous(std::vector<P2pOp>& ops, size_t nranks, const std::vector<int>& nops, std::vector<unsigned long long>& rdv_base, P2pArgs* a) {
    a->nmaps = 0;
    if (!g_p2p_rdv) return;
    std::vector<unsigned long long> sent(rdv_base), recvd(rdv_base);     // [src * n + dst]
    for (size_t r = 0; r < nranks; r++)
        for (int k = 0; k < nops[r]; k++) {
            P2pOp& o = ops[r * kMaxP2pOps + (size_t)k];
            if (o.bytes < kP2pRdvMinBytes) continue;
            o.rdv = 1;
            if (o.is_send) o.rdv_index = sent[r * nranks + (size_t)o.peer]++;
            else {
                o.rdv_index = recvd[(size_t)o.peer * nranks + r]++;
                const bool mapped = g_p2p_rdv == 1 || (g_p2p_rdv == 3 && r % 2 == 0);
                o.dst_kind = g_p2p_rdv == 2 ? P2P_DST_NONE : P2P_DST_IPC;
                o.dst_a = (unsigned long long)(uintptr_t)o.buf; o.dst_id = 1; o.dst_off = 0;
                if (mapped && a->nmaps < kMaxP2pMaps) {
                    P2pMap& m = a->maps[a->nmaps++];
                    m.peer = (int)r; m.kind = P2P_DST_IPC; m.a = o.dst_a; m.id = 1; m.size = o.bytes; m.mapped = o.buf;
                }
            }
        }
    rdv_base = sent;
}

// Pools of finished emulation runs, kept for the next run of the same size (the tests make thousands of short
// runs; allocating and clearing 8 x 80 MB for each would dominate them).
std::vector<char*> g_spare_pools;
size_t g_spare_pool_bytes = 0;

char* take_pool(size_t bytes) {
    if (g_spare_pool_bytes != bytes) {
        for (char* p : g_spare_pools) cudaFree(p);
        g_spare_pools.clear();
        g_spare_pool_bytes = bytes;
    }
    if (!g_spare_pools.empty()) { char* p = g_spare_pools.back(); g_spare_pools.pop_back(); return p; }
    char* p = nullptr;
    return cudaMalloc((void**)&p, bytes) == cudaSuccess ? p : nullptr;
}

void give_pool(char* p, size_t bytes) {
    if (bytes == g_spare_pool_bytes && g_spare_pools.size() < (size_t)kMaxPeers) g_spare_pools.push_back(p);
    else cudaFree(p);
}

/** Flags, credit words and packet tags must start from zero; FIFO and staging contents do not matter. */
bool clear_pool_control(char* pool) {
    return cudaMemset(pool, 0, kLLOff + kLLBytes) == cudaSuccess &&
           cudaMemset(pool + kLL2Off, 0, 2 * (size_t)kMaxPeers * 2 * kLL2PhaseBytes) == cudaSuccess;
}

struct EmuWorld {
    int n = 0;
    size_t stage_bytes = 0, pool_bytes = 0;
    std::vector<char*> pools;
    uint32_t* status = nullptr;      // device memory: ST_WORDS + abort word
    DevComm* d_comms = nullptr;
    uint32_t* seq_words = nullptr;   // per virtual rank: {next sequence number, CTAs done}, 64 bytes apart
    std::vector<DevComm> comms;
    char* mc = nullptr;              // host simulation: multicast alias of the pools
    ~EmuWorld() {
#ifdef DCCL_HOST_SIM
        if (mc) ::dccl_sim::mc_destroy(mc);
#endif
        if (seq_words) cudaFree(seq_words);
        cudaDeviceSynchronize();
        for (char* p : pools) if (p) give_pool(p, pool_bytes);
        if (status) cudaFree(status);
        if (d_comms) cudaFree(d_comms);
    }
    bool create(int nranks, size_t stage, unsigned long long timeout_ms) {
        n = nranks;
        stage_bytes = stage;
        pool_bytes = kStageOff + 2 * stage;
        pools.assign(n, nullptr);
        for (int r = 0; r < n; r++) {
            if ((pools[r] = take_pool(pool_bytes)) == nullptr) return false;
            if (!clear_pool_control(pools[r])) return false;
            if (g_guard && !canary_fill(pools[r], canary_copy_cuda)) return false;
        }
        if (cudaMalloc((void**)&status, (ST_WORDS + 8) * sizeof(uint32_t)) != cudaSuccess) return false;
        cudaMemset(status, 0, (ST_WORDS + 8) * sizeof(uint32_t));
        if (g_device_seq) {
            std::vector<uint32_t> init((size_t)n * 16, 0u);
            for (int r = 0; r < n; r++) init[(size_t)r * 16] = 1u;   // the first call has number 1
            if (cudaMalloc((void**)&seq_words, init.size() * sizeof(uint32_t)) != cudaSuccess) return false;
            if (cudaMemcpy(seq_words, init.data(), init.size() * sizeof(uint32_t), cudaMemcpyHostToDevice) != cudaSuccess) return false;
        }
#ifdef DCCL_HOST_SIM
        if ((mc = ::dccl_sim::mc_create(pool_bytes, n, pools.data())) == nullptr) return false;
#endif
        comms.resize(n);
        for (int r = 0; r < n; r++) {
            DevComm& c = comms[r];
            memset(&c, 0, sizeof(c));
            if (seq_words) { c.seq_word = seq_words + (size_t)r * 16; c.done_word = c.seq_word + 1; }
            c.rank = r;
            c.nranks = n;
            for (int p = 0; p < n; p++) c.pool[p] = pools[p];
            c.mc_pool = mc;           // nullptr on a GPU: the multimem variants are not emulated there
            c.status = status;
            c.abort_word = status + ST_WORDS;
            c.timeout_ns = timeout_ms * 1000000ull;
            c.stage_bytes = stage;
#ifdef DCCL_DEBUG_BOUNDS
            if (g_declared_stage && g_declared_stage < stage) c.stage_bytes = g_declared_stage;
#endif
        }
        if (cudaMalloc((void**)&d_comms, n * sizeof(DevComm)) != cudaSuccess) return false;
        return cudaMemcpy(d_comms, comms.data(), n * sizeof(DevComm), cudaMemcpyHostToDevice) == cudaSuccess;
    }
    /** 0, or 200 + number of the damaged gap (1-based) of the first pool whose guard words were overwritten. */
    int check_guards() const {
        if (!g_guard) return 0;
        for (int r = 0; r < n; r++) {
            size_t bad = 0;
            const int rc = canary_check(pools[r], canary_copy_cuda, &bad);
            if (rc != 0) {
                fprintf(stderr, "dccl emulation: guard words of virtual rank %d damaged (gap %d, pool offset %zu)\n", r, rc, bad);
                return rc < 0 ? -5 : 200 + rc;
            }
        }
        return 0;
    }
};

int fail(const char* what) {
    cudaError_t e = cudaGetLastError();
    fprintf(stderr, "dccl emulation: %s (%s)\n", what, cudaGetErrorString(e));
    return -1;
}

} // namespace

extern "C" {

/** 1: the emulated ranks count their calls in device memory (the mode that makes launches replayable
 *  from a CUDA graph); the launch arguments then carry a wrong sequence number on purpose. 0: host counts. */
void dccl_emu_set_device_seq(int on) { g_device_seq = on ? 1 : 0; }

/**
 * Collectives to run before every call of the following dccl_emu_collective runs, in the same virtual world and on
 * the same buffers, e.g. "allreduce:oneshot,broadcast:oneshot": sequences of different kernels share flags, packet
 * generations and staging halves, and a kernel must cope with whatever its predecessors left there. Same element
 * count, type and operator as the call under test (out of place, aligned runs only); their results are not checked.
 * Empty string or NULL: none. Returns the number of entries, -1 on a name that is not known.
 */
int dccl_emu_set_mix(const char* spec) {
    g_mix.clear();
    if (!spec) return 0;
    std::string s(spec);
    size_t pos = 0;
    while (pos < s.size()) {
        size_t comma = s.find(',', pos);
        if (comma == std::string::npos) comma = s.size();
        const std::string item = s.substr(pos, comma - pos);
        pos = comma + 1;
        if (item.empty()) continue;
        const size_t colon = item.find(':');
        if (colon == std::string::npos) { g_mix.clear(); return -1; }
        const int c = parse_collective_name(item.substr(0, colon).c_str());
        const GpuAlgo al = parse_algo_name(item.substr(colon + 1).c_str());
        if (c < 0 || al == ALGO_COUNT) { g_mix.clear(); return -1; }
        g_mix.emplace_back(c, al);
    }
    return (int)g_mix.size();
}

/** 1: every run fills the unused parts of the virtual ranks' pools with guard words and checks them afterwards;
 *  a run that damaged them returns 200 + the number of the gap (canary.hpp). */
void dccl_emu_set_guard(int on) { g_guard = on ? 1 : 0; }

/**
 * Range-checking builds only (make BOUNDS=1; returns -1 otherwise and changes nothing): tell the kernels of the
 * following runs that a staging half has `bytes` bytes although the usual, larger size is allocated (0: back to the
 * truth). A run whose message needs more than the declared size must then come back with 100 + DEV_BOUNDS and
 * untouched outputs: the kernels refuse before their first access.
 */
int dccl_emu_declare_stage_bytes(size_t bytes) {
#ifdef DCCL_DEBUG_BOUNDS
    g_declared_stage = bytes;
    return 0;
#else
    (void)bytes;
    return -1;
#endif
}

#ifdef DCCL_HOST_SIM
/** Host simulation only: the switch kernel behind algorithm "nvls": 0 staged, 1 pipelined all-reduce,
 *  2 pipelined broadcast / reduce. */
void dccl_emu_set_switch_form(int form) { g_switch_form = form; }
/** Host simulation only: target chunk size of the pipelined switch kernels and the size of their switch group
 *  (0: the default share of the grid); 100 * teams + size chooses the number of teams of that group as well (default 2). */
void dccl_emu_set_pipe(size_t chunk_bytes, int nv_ctas) { nvls_pipe_set_chunk_bytes(chunk_bytes); g_pipe_nv = nv_ctas % 100; g_pipe_teams = nv_ctas >= 100 ? nv_ctas / 100 : 2; }
#endif

/** How large send / recv messages of the emulated ranks travel: 0 FIFO only, 1 rendezvous with every receive buffer
 *  mapped by its sender (zero-copy), 2 rendezvous with none mapped (FIFO after the rendezvous), 3 only even ranks' buffers
 *  mapped. */
void dccl_emu_set_p2p_rendezvous(int mode) { g_p2p_rdv = mode; }

/** 1: all-reduce, reduce-scatter, broadcast and reduce with the two-shot variant run their zero-copy forms on the emulated ranks' user buffers. */
void dccl_emu_set_peer_buffers(int on) { g_peer_buffers = on ? 1 : 0; }

/** Chunks per shard of the zero-copy broadcast (0: by message size, as the library does). */
void dccl_emu_set_bcast_chunks(int chunks) { g_bcast_chunks = chunks; }

/**
 * Run `iters` back-to-back calls of one collective among `nranks` virtual ranks on the current
 * device and return every rank's output of the last call.
 *   kind: allreduce | reducescatter | allgather | broadcast | reduce
 *   algo: oneshot | twoshot | twoshot_ll | ring | rabenseifner
 *   count: all-reduce / broadcast / reduce: elements per rank; reduce-scatter: recvcount; all-gather: sendcount
 *   host_in:  nranks consecutive inputs;  host_out: nranks consecutive outputs
 *   misalign: bytes added to every user pointer (exercises the unaligned paths)
 * Returns 0, a negative value on a CUDA / argument error, or 100 + device status code when a kernel
 * reported a failure.
 */
int dccl_emu_collective(const char* kind_s, const char* algo_s, int nranks, int dtype, int op, size_t count, int root, int ctas,
                        int in_place, size_t misalign, int iters, size_t stage_bytes, const void* host_in, void* host_out) {
    const int coll = parse_collective_name(kind_s);
    const GpuAlgo algo = parse_algo_name(algo_s);
    if (coll < 0 || algo == ALGO_COUNT || nranks < 1 || nranks > kMaxPeers || ctas < 1) return -2;
    const ncclDataType_t dt = (ncclDataType_t)dtype;
    const size_t es = size_of_type(dt);
    if (!es) return -2;
    const size_t n = (size_t)nranks;
    size_t in_elems = count, out_elems = count;
    if (coll == COLL_REDUCESCATTER) in_elems = count * n;
    if (coll == COLL_ALLGATHER) out_elems = count * n;
    if (stage_bytes == 0) stage_bytes = 8u << 20;
    stage_bytes = (stage_bytes + 4095) / 4096 * 4096;

    EmuWorld w;
    if (!w.create(nranks, stage_bytes, 2000)) return fail("cannot create the virtual ranks");

    // user buffers
    std::vector<char*> sendb(n, nullptr), recvb(n, nullptr);
    std::vector<RankIO> ios(n);
    size_t buf_elems = in_elems > out_elems ? in_elems : out_elems;
    if (!g_mix.empty()) buf_elems = count * n;      // a reduce-scatter reads, an all-gather writes n slots
    for (size_t r = 0; r < n; r++) {
        if (cudaMalloc((void**)&sendb[r], buf_elems * es + misalign + 64) != cudaSuccess) return fail("cudaMalloc");
        if (cudaMalloc((void**)&recvb[r], buf_elems * es + misalign + 64) != cudaSuccess) return fail("cudaMalloc");
        cudaMemset(recvb[r], 0xEE, buf_elems * es + misalign + 64);
        memset(&ios[r], 0, sizeof(RankIO));
        char* s = sendb[r] + misalign;
        char* d = in_place ? s : recvb[r] + misalign;
        if (in_place && coll == COLL_REDUCESCATTER) d = s + r * count * es;       // output is the rank's slot of the input
        if (in_place && coll == COLL_ALLGATHER) { d = s; s = s + r * count * es; } // input is the rank's slot of the output
        ios[r].send = s;
        ios[r].recv = d;
    }
    for (size_t r = 0; r < n; r++)
        for (size_t p = 0; p < n; p++) {
            ios[r].send_peer[p] = (const char*)ios[p].send;
            ios[r].recv_peer[p] = (char*)ios[p].recv;
        }
    const bool direct = g_peer_buffers && algo == ALGO_TWOSHOT && misalign % 16 == 0 &&
                        (coll == COLL_ALLREDUCE || coll == COLL_REDUCE || coll == COLL_BROADCAST || (coll == COLL_REDUCESCATTER && (count * es) % 16 == 0));
#ifdef DCCL_HOST_SIM
    // with "peer buffers" on, the user buffers also count as multicast-bound (what dcclMemAlloc memory is): the switch
    // kernels then run their zero-copy forms on them
    char *send_mc = nullptr, *recv_mc = nullptr;
    const bool sym_switch = g_peer_buffers && algo == ALGO_NVLS && misalign % 16 == 0 && !in_place;
    if (sym_switch) {
        send_mc = ::dccl_sim::mc_create(buf_elems * es + misalign + 64, nranks, sendb.data());
        recv_mc = ::dccl_sim::mc_create(buf_elems * es + misalign + 64, nranks, recvb.data());
        if (!send_mc || !recv_mc) return fail("multicast mapping of the user buffers");
        for (size_t r = 0; r < n; r++) { ios[r].send_mc = send_mc + misalign; ios[r].recv_mc = recv_mc + misalign; }
    }
#endif
    RankIO* d_ios = nullptr;
    if (cudaMalloc((void**)&d_ios, n * sizeof(RankIO)) != cudaSuccess) return fail("cudaMalloc");
    cudaMemcpy(d_ios, ios.data(), n * sizeof(RankIO), cudaMemcpyHostToDevice);

    LaunchCfg cfg;
    cfg.ctas = ctas;
    cfg.ranks_in_launch = nranks;
    int rc = 0;
    uint32_t next_seq_no = 1;
    for (int it = 0; it < iters && rc == 0; it++) {
        // fresh inputs every call (in-place runs overwrite them)
        for (size_t r = 0; r < n; r++) {
            const char* src = (const char*)host_in + r * in_elems * es;
            if (in_place && coll == COLL_ALLGATHER) cudaMemcpy((char*)ios[r].send, src, in_elems * es, cudaMemcpyHostToDevice);
            else cudaMemcpy((char*)ios[r].send, src, in_elems * es, cudaMemcpyHostToDevice);
        }
        CollArgs a;
        memset(&a, 0, sizeof(a));
        a.emu = w.d_comms;
        a.emu_io = d_ios;
        a.count = count;
        a.stride = count;
        // sequence numbers count launches (set below); with the device-side counter the launch carries a wrong one on purpose
        a.op = op;
        a.root = root;
        // one launch of (collective, variant) on the buffers of this run; the arguments are a copy, the caller's stay as they are
        uint32_t extra_seqs = 0;       // call numbers a launch used beyond its own (the pipelined switch forms)
        auto launch_one = [&](int coll, GpuAlgo algo, CollArgs a, size_t* cap_out) -> cudaError_t {
            cudaError_t e = cudaErrorInvalidValue;
            size_t cap = 0;
            extra_seqs = 0;
#ifdef DCCL_HOST_SIM
            if (algo == ALGO_NVLS) {
                // the switch kernels on ordinary buffers (staged through the pool), played by the simulated multicast mapping
                const bool reducing = coll == COLL_ALLREDUCE || coll == COLL_REDUCESCATTER || coll == COLL_REDUCE;
                const bool switch_op = !reducing || (op != (int)ncclProd && !((dt == ncclFloat32 || dt == ncclFloat64) && (op == (int)ncclMax || op == (int)ncclMin)) &&
                                                     dt != ncclInt8 && dt != ncclUint8);
                if (!switch_op) e = cudaErrorInvalidValue;
                else if (coll == COLL_ALLREDUCE && g_switch_form == 1) {
                    // with host-counted sequence numbers the staging half is a ring and takes any length
                    cap = g_device_seq ? nvls_pipe_capacity(es, stage_bytes, nranks, false) : count;
                    LaunchCfg pc = cfg;
                    pc.ctas = cfg.ctas < 3 ? 3 : cfg.ctas;
                    if (count <= cap) { e = launch_nvls_pipe(a, dt, pc, false, stage_bytes, g_pipe_nv, g_pipe_teams, g_device_seq != 0); extra_seqs = nvls_pipe_extra_seqs(count, es, stage_bytes, nranks, false, g_device_seq != 0); }
                } else if (coll == COLL_REDUCESCATTER && g_switch_form == 1) {
                    cap = g_device_seq ? nvls_pipe_capacity(es, stage_bytes, nranks, true) : count;
                    LaunchCfg pc = cfg;
                    pc.ctas = cfg.ctas < 2 ? 2 : cfg.ctas;
                    if (count <= cap) { e = launch_nvls_pipe(a, dt, pc, true, stage_bytes, g_pipe_nv, g_pipe_teams, g_device_seq != 0); extra_seqs = nvls_pipe_extra_seqs(count, es, stage_bytes, nranks, true, g_device_seq != 0); }
                } else if ((coll == COLL_BROADCAST || coll == COLL_REDUCE) && g_switch_form == 2) {
                    a.mode = coll == COLL_BROADCAST ? ROOTED_BROADCAST : ROOTED_REDUCE;
                    cap = nvls_pipe_capacity(es, stage_bytes, nranks, false);
                    if (count <= cap) e = launch_nvls_rooted(a, dt, cfg);
                } else {
                    a.mode = coll == COLL_ALLREDUCE ? NV_ALLREDUCE : coll == COLL_REDUCESCATTER ? NV_REDUCESCATTER : coll == COLL_ALLGATHER ? NV_ALLGATHER
                             : coll == COLL_BROADCAST ? NV_BROADCAST : NV_REDUCE;
                    a.symmetric = sym_switch && (count * es) % 16 == 0 ? 1 : 0;      // zero-copy: whole 16-byte vectors per slot
                    cap = a.symmetric ? count : nvls_capacity(a.mode, nranks, es, stage_bytes);
                    if (count <= cap) e = launch_nvls(a, dt, cfg);
                }
            } else
#endif
            if (coll == COLL_ALLREDUCE) {
                if (algo == ALGO_ONESHOT) { cap = oneshot_ll_capacity_bytes() / es; if (count <= cap) e = launch_oneshot_ll(a, dt, cfg); }
                else if (algo == ALGO_TWOSHOT_LL) { a.mode = LL2_ALLREDUCE; cap = ll_twoshot_capacity_bytes(nranks) / es; if (count <= cap) e = launch_ll_twoshot(a, dt, cfg); }
                else if (algo == ALGO_RING) { a.mode = RING_ALLREDUCE; cap = ring_capacity(a.mode, nranks, es, stage_bytes); if (count <= cap) e = launch_ring(a, dt, cfg); }
                else if (algo == ALGO_RABENSEIFNER) { cap = hd_capacity(nranks, es, stage_bytes); if (count <= cap) e = launch_hd(a, dt, cfg); }
                else if (direct) { a.symmetric = 1; a.mode = DIRECT_ALLREDUCE; cap = count; e = launch_direct(a, dt, cfg); }
                else { a.mode = TS_ALLREDUCE; cap = twoshot_capacity(a.mode, nranks, es, stage_bytes); if (count <= cap) e = launch_twoshot(a, dt, cfg); }
            } else if (coll == COLL_REDUCE && algo == ALGO_TWOSHOT_LL) {
                a.mode = LL2_REDUCE;
                cap = ll_twoshot_capacity_bytes(nranks) / es;
                if (count <= cap) e = launch_ll_twoshot(a, dt, cfg);
            } else if (coll != COLL_ALLREDUCE && algo == ALGO_ONESHOT && count * es <= oneshot_ll_capacity_bytes()) {
                a.mode = coll == COLL_REDUCESCATTER ? LL_REDUCESCATTER : coll == COLL_ALLGATHER ? LL_ALLGATHER : coll == COLL_BROADCAST ? LL_BROADCAST : LL_REDUCE;
                cap = oneshot_ll_capacity_bytes() / es;
                e = launch_ll_collective(a, dt, cfg);
            } else if (coll == COLL_REDUCESCATTER) {
                if (algo == ALGO_RING) { a.mode = RING_REDUCESCATTER; cap = ring_capacity(a.mode, nranks, es, stage_bytes); if (count <= cap) e = launch_ring(a, dt, cfg); }
                else if (direct) { a.symmetric = 1; a.mode = DIRECT_REDUCESCATTER; cap = count; e = launch_direct(a, dt, cfg); }
                else { a.mode = TS_REDUCESCATTER; cap = twoshot_capacity(a.mode, nranks, es, stage_bytes); if (count <= cap) e = launch_twoshot(a, dt, cfg); }
            } else if (coll == COLL_ALLGATHER) {
                if (algo == ALGO_RING) { a.mode = RING_ALLGATHER; cap = ring_capacity(a.mode, nranks, es, stage_bytes); if (count <= cap) e = launch_ring(a, dt, cfg); }
                else { a.mode = TS_ALLGATHER; cap = twoshot_capacity(a.mode, nranks, es, stage_bytes); if (count <= cap) e = launch_twoshot(a, dt, cfg); }
            } else if (coll == COLL_BROADCAST && direct) {
                a.symmetric = 1; cap = count; e = launch_direct_bcast(a, count * es, nranks, cfg, g_bcast_chunks);
            } else if (coll == COLL_REDUCE && direct) {
                a.symmetric = 1; a.mode = DIRECT_REDUCE; cap = count; e = launch_direct(a, dt, cfg);
            } else if (coll == COLL_BROADCAST) {
                a.mode = algo == ALGO_ONESHOT ? TS_BROADCAST_DIRECT : TS_BROADCAST;
                cap = twoshot_capacity(a.mode, nranks, es, stage_bytes);
                if (count <= cap) e = launch_twoshot(a, dt, cfg);
            } else if (coll == COLL_REDUCE) {
                a.mode = TS_REDUCE;
                cap = twoshot_capacity(a.mode, nranks, es, stage_bytes);
                if (count <= cap) e = launch_twoshot(a, dt, cfg);
            }
            *cap_out = cap;
            return e;
        };
        size_t cap = 0;
        cudaError_t e = cudaSuccess;
        // other collectives first, in the same world and on the same buffers (dccl_emu_set_mix): what they leave behind in
        // flags, packet generations and staging halves is what the call under test starts from
        for (size_t k = 0; k < g_mix.size() && e == cudaSuccess; k++) {
            a.seq = next_seq_no++;
            a.parity = (int)(a.seq & 1u);
            if (g_device_seq) { a.seq = 0x5eed0000u; a.parity = 0; }
            e = launch_one(g_mix[k].first, g_mix[k].second, a, &cap);
            next_seq_no += extra_seqs;
            if (e == cudaSuccess && cudaDeviceSynchronize() != cudaSuccess) e = cudaErrorLaunchFailure;
        }
        a.seq = next_seq_no++;
        a.parity = (int)(a.seq & 1u);
        if (g_device_seq) { a.seq = 0x5eed0000u; a.parity = 0; }
        if (e == cudaSuccess) { e = launch_one(coll, algo, a, &cap); next_seq_no += extra_seqs; }
        if (e != cudaSuccess) { fprintf(stderr, "dccl emulation: launch failed or count %zu above capacity %zu: %s\n", count, cap, cudaGetErrorString(e)); rc = -3; break; }
        if (cudaDeviceSynchronize() != cudaSuccess) { rc = fail("kernel"); break; }
        uint32_t st[ST_WORDS];
        cudaMemcpy(st, w.status, sizeof(st), cudaMemcpyDeviceToHost);
        if (st[ST_CODE] != DEV_OK) {
            fprintf(stderr, "dccl emulation: kernel reported code %u peer %u site %u seq %u\n", st[ST_CODE], st[ST_PEER], st[ST_SITE], st[ST_SEQ]);
            rc = 100 + (int)st[ST_CODE];
        }
    }
    if (rc == 0) rc = w.check_guards();
    if (rc == 0)
        for (size_t r = 0; r < n; r++)
            cudaMemcpy((char*)host_out + r * out_elems * es, ios[r].recv, out_elems * es, cudaMemcpyDeviceToHost);
#ifdef DCCL_HOST_SIM
    if (send_mc) ::dccl_sim::mc_destroy(send_mc);
    if (recv_mc) ::dccl_sim::mc_destroy(recv_mc);
#endif
    for (size_t r = 0; r < n; r++) { cudaFree(sendb[r]); cudaFree(recvb[r]); }
    cudaFree(d_ios);
    if (rc == 0 && cudaGetLastError() != cudaSuccess) rc = -4;
    return rc;
}

/**
 * Ring of send/recv pairs among virtual ranks: rank r sends `window` messages of `bytes` to r+1 and receives
 * `window` messages from r-1, `iters` times, all in one launch per iteration (the grouped form; several
 * operations address the same peer). host_in: nranks x window messages; host_out: what each rank received last.
 */
int dccl_emu_sendrecv_ring(int nranks, size_t bytes, int window, int ctas_per_op, int iters, const void* host_in, void* host_out) {
    if (nranks < 2 || nranks > kMaxPeers || ctas_per_op < 1 || ctas_per_op > kP2pCtas || window < 1 || 2 * window > kMaxP2pOps) return -2;
    EmuWorld w;
    if (!w.create(nranks, 1u << 20, 2000)) return fail("cannot create the virtual ranks");
    const size_t n = (size_t)nranks, W = (size_t)window;
    std::vector<char*> sb(n), rb(n);
    for (size_t r = 0; r < n; r++) {
        if (cudaMalloc((void**)&sb[r], W * bytes + 16) != cudaSuccess || cudaMalloc((void**)&rb[r], W * bytes + 16) != cudaSuccess) return fail("cudaMalloc");
        cudaMemcpy(sb[r], (const char*)host_in + r * W * bytes, W * bytes, cudaMemcpyHostToDevice);
        cudaMemset(rb[r], 0xEE, W * bytes);
    }
    P2pOp* d_ops = nullptr;
    int* d_nops = nullptr;
    cudaMalloc((void**)&d_ops, n * kMaxP2pOps * sizeof(P2pOp));
    cudaMalloc((void**)&d_nops, n * sizeof(int));
    std::vector<int> nops(n, 2 * window);
    cudaMemcpy(d_nops, nops.data(), n * sizeof(int), cudaMemcpyHostToDevice);
    int rc = 0;
    unsigned long long chunk_base = 0;
    std::vector<unsigned long long> rdv_base(n * n, 0ull);
    for (int it = 0; it < iters && rc == 0; it++) {
        std::vector<P2pOp> ops(n * kMaxP2pOps);
        for (size_t r = 0; r < n; r++)
            for (size_t k = 0; k < W; k++) {
                P2pOp& s = ops[r * kMaxP2pOps + 2 * k];
                P2pOp& d = ops[r * kMaxP2pOps + 2 * k + 1];
                s.is_send = 1; s.peer = (int)((r + 1) % n); s.buf = sb[r] + k * bytes; s.bytes = bytes; s.chunk_base = chunk_base + k * p2p_chunks(bytes);
                d.is_send = 0; d.peer = (int)((r + n - 1) % n); d.buf = rb[r] + k * bytes; d.bytes = bytes; d.chunk_base = chunk_base + k * p2p_chunks(bytes);
            }
        chunk_base += W * p2p_chunks(bytes);
        P2pArgs a;
        memset(&a, 0, sizeof(a));
        emu_rendezvous(ops, n, nops, rdv_base, &a);
        cudaMemcpy(d_ops, ops.data(), ops.size() * sizeof(P2pOp), cudaMemcpyHostToDevice);
        a.emu = w.d_comms;
        a.emu_ops = d_ops;
        a.emu_nops = d_nops;
        a.ctas_per_op = ctas_per_op;
        a.ctas_per_rank = 2 * window * ctas_per_op;
        LaunchCfg cfg;
        cfg.ctas = a.ctas_per_rank;
        cfg.ranks_in_launch = nranks;
        if (launch_p2p(a, cfg) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { rc = fail("send/recv kernel"); break; }
        uint32_t st[ST_WORDS];
        cudaMemcpy(st, w.status, sizeof(st), cudaMemcpyDeviceToHost);
        if (st[ST_CODE] != DEV_OK) rc = 100 + (int)st[ST_CODE];
    }
    if (rc == 0) rc = w.check_guards();
    if (rc == 0) for (size_t r = 0; r < n; r++) cudaMemcpy((char*)host_out + r * W * bytes, rb[r], W * bytes, cudaMemcpyDeviceToHost);
    for (size_t r = 0; r < n; r++) { cudaFree(sb[r]); cudaFree(rb[r]); }
    cudaFree(d_ops);
    cudaFree(d_nops);
    return rc;
}

/**
 * All-to-all among virtual ranks as the library composes it from grouped send / recv: every rank records its
 * receives from rank - k and then its sends to rank + k (k = 1 .. n-1) and launches them together, `iters` times.
 * Block p of a rank's input (`bytes` each) goes to rank p; the own block is not moved by the kernel and is copied here.
 * host_in / host_out: nranks x nranks blocks.
 */
int dccl_emu_all_to_all(int nranks, size_t bytes, int ctas_per_op, int iters, const void* host_in, void* host_out) {
    if (nranks < 2 || nranks > kMaxPeers || ctas_per_op < 1 || ctas_per_op > kP2pCtas || 2 * (nranks - 1) > kMaxP2pOps) return -2;
    EmuWorld w;
    if (!w.create(nranks, 1u << 20, 2000)) return fail("cannot create the virtual ranks");
    const size_t n = (size_t)nranks;
    std::vector<char*> sb(n), rb(n);
    for (size_t r = 0; r < n; r++) {
        if (cudaMalloc((void**)&sb[r], n * bytes + 16) != cudaSuccess || cudaMalloc((void**)&rb[r], n * bytes + 16) != cudaSuccess) return fail("cudaMalloc");
        cudaMemcpy(sb[r], (const char*)host_in + r * n * bytes, n * bytes, cudaMemcpyHostToDevice);
        cudaMemset(rb[r], 0xEE, n * bytes);
    }
    P2pOp* d_ops = nullptr;
    int* d_nops = nullptr;
    cudaMalloc((void**)&d_ops, n * kMaxP2pOps * sizeof(P2pOp));
    cudaMalloc((void**)&d_nops, n * sizeof(int));
    const int nops = 2 * (nranks - 1);
    std::vector<int> nops_v(n, nops);
    cudaMemcpy(d_nops, nops_v.data(), n * sizeof(int), cudaMemcpyHostToDevice);
    int rc = 0;
    // chunks moved so far per ordered pair (every pair moves one message per iteration)
    unsigned long long chunk_base = 0;
    std::vector<unsigned long long> rdv_base(n * n, 0ull);
    for (int it = 0; it < iters && rc == 0; it++) {
        std::vector<P2pOp> ops(n * kMaxP2pOps);
        for (size_t r = 0; r < n; r++) {
            int k = 0;
            for (size_t d = 1; d < n; d++) {        // receivers first: they get the lower block numbers
                const size_t p = (r + n - d) % n;
                P2pOp& o = ops[r * kMaxP2pOps + k++];
                o.is_send = 0; o.peer = (int)p; o.buf = rb[r] + p * bytes; o.bytes = bytes; o.chunk_base = chunk_base;
            }
            for (size_t d = 1; d < n; d++) {
                const size_t p = (r + d) % n;
                P2pOp& o = ops[r * kMaxP2pOps + k++];
                o.is_send = 1; o.peer = (int)p; o.buf = sb[r] + p * bytes; o.bytes = bytes; o.chunk_base = chunk_base;
            }
        }
        chunk_base += p2p_chunks(bytes);
        P2pArgs a;
        memset(&a, 0, sizeof(a));
        emu_rendezvous(ops, n, nops_v, rdv_base, &a);
        cudaMemcpy(d_ops, ops.data(), ops.size() * sizeof(P2pOp), cudaMemcpyHostToDevice);
        a.emu = w.d_comms;
        a.emu_ops = d_ops;
        a.emu_nops = d_nops;
        a.ctas_per_op = ctas_per_op;
        a.ctas_per_rank = nops * ctas_per_op;
        LaunchCfg cfg;
        cfg.ctas = a.ctas_per_rank;
        cfg.ranks_in_launch = nranks;
        if (launch_p2p(a, cfg) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { rc = fail("all-to-all kernel"); break; }
        uint32_t st[ST_WORDS];
        cudaMemcpy(st, w.status, sizeof(st), cudaMemcpyDeviceToHost);
        if (st[ST_CODE] != DEV_OK) rc = 100 + (int)st[ST_CODE];
    }
    if (rc == 0) rc = w.check_guards();
    if (rc == 0)
        for (size_t r = 0; r < n; r++) {
            cudaMemcpy(rb[r] + r * bytes, sb[r] + r * bytes, bytes, cudaMemcpyDeviceToDevice);    // the own block
            cudaMemcpy((char*)host_out + r * n * bytes, rb[r], n * bytes, cudaMemcpyDeviceToHost);
        }
    for (size_t r = 0; r < n; r++) { cudaFree(sb[r]); cudaFree(rb[r]); }
    cudaFree(d_ops);
    cudaFree(d_nops);
    return rc;
}

/**
 * Bounded-wait check: one thread waits, with a `timeout_ms` budget, for a flag that nothing sets.
 * Returns the status code the kernel recorded (DEV_TIMEOUT = 1 is the expected answer) and the time
 * the kernel took in milliseconds through *elapsed_ms. The context stays usable afterwards.
 */
int dccl_emu_wait_probe(unsigned timeout_ms, float* elapsed_ms) {
    EmuWorld w;
    if (!w.create(1, 4096, timeout_ms)) return fail("cannot create the virtual rank");
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaEventRecord(t0);
    if (launch_wait_probe(w.comms[0], nullptr) != cudaSuccess) return fail("launch");
    cudaEventRecord(t1);
    if (cudaDeviceSynchronize() != cudaSuccess) return fail("probe kernel");
    float ms = 0;
    cudaEventElapsedTime(&ms, t0, t1);
    if (elapsed_ms) *elapsed_ms = ms;
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    uint32_t st[ST_WORDS];
    cudaMemcpy(st, w.status, sizeof(st), cudaMemcpyDeviceToHost);
    return (int)st[ST_CODE];
}

/** Pairwise reduce and copy kernels, for single-GPU numerics tests: acc = op(acc, in). */
int dccl_local_reduce(void* host_acc, const void* host_in, size_t count, int dtype, int op) {
    const size_t es = size_of_type((ncclDataType_t)dtype);
    char *a = nullptr, *b = nullptr;
    if (cudaMalloc((void**)&a, count * es + 16) != cudaSuccess || cudaMalloc((void**)&b, count * es + 16) != cudaSuccess) return fail("cudaMalloc");
    cudaMemcpy(a, host_acc, count * es, cudaMemcpyHostToDevice);
    cudaMemcpy(b, host_in, count * es, cudaMemcpyHostToDevice);
    cudaError_t e = launch_local_reduce(a, b, count, (ncclDataType_t)dtype, (ncclRedOp_t)op, nullptr);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) cudaMemcpy(host_acc, a, count * es, cudaMemcpyDeviceToHost);
    cudaFree(a);
    cudaFree(b);
    return e == cudaSuccess ? 0 : fail("local reduce");
}

/** The same kernel on buffers that already live on the device, on `stream` (no synchronisation): for timing. */
int dccl_local_reduce_device(void* dev_acc, const void* dev_in, size_t count, int dtype, int op, void* stream) {
    return launch_local_reduce(dev_acc, dev_in, count, (ncclDataType_t)dtype, (ncclRedOp_t)op, (cudaStream_t)stream) == cudaSuccess ? 0 : fail("local reduce");
}

} // extern "C"
