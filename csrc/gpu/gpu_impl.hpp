/** Implementation class behind GpuComm; split over gpu_comm.cu (life cycle, memory) and
 *  gpu_collectives.cu (variant choice, chunking, launches). */
#pragma once
#include "gpu_comm.hpp"
#include "symmem.hpp"
#include "topology.hpp"
#include "../kernels/kernels.hpp"
#include "../tuner/tuner.hpp"
#include <atomic>
#include <map>
#include <vector>

namespace dccl {

struct RegisteredBuffer {
    char* base = nullptr;             // as given by the user
    size_t size = 0;
    char* peer[kMaxPeers] = {nullptr};   // the same buffer of every rank, mapped here
    void* opened[kMaxPeers] = {nullptr}; // what cudaIpcOpenMemHandle returned (to close it)
};

/** Lazy registration (auto_register.cu): an allocation of this rank that the peers have been told about ... */
struct AutoExport {
    unsigned long long id = 0;
    size_t size = 0;
    cudaIpcMemHandle_t handle;
    bool announced = false;           // the peers have seen it in an exchange
    bool posted = false;              // it is on this rank's bulletin (send / recv peers pick it up from there)
    bool refused = false;             // cannot be exported, or a peer could not open it: not offered (again)
};
/** ... and a peer's allocation as mapped here. */
struct AutoImport {
    unsigned long long id = 0;
    void* mapped = nullptr;
    size_t size = 0;                  // of the allocation
    unsigned long long stamp = 0;     // when it was mapped (newer mappings are offered to a send first)
    std::string hkey;                 // its entry in the table of opened handles
};

class GpuCommImpl : public GpuComm {
public:
    GpuCommImpl(Bootstrap* bs, int device);
    ~GpuCommImpl() override;
    bool init(std::string* err);

    ncclResult_t all_reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, GpuAlgo algo, cudaStream_t stream) override;
    ncclResult_t reduce_scatter(const void* send, void* recv, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op, GpuAlgo algo, cudaStream_t stream) override;
    ncclResult_t all_gather(const void* send, void* recv, size_t sendcount, ncclDataType_t dt, GpuAlgo algo, cudaStream_t stream) override;
    ncclResult_t broadcast(const void* send, void* recv, size_t count, ncclDataType_t dt, int root, GpuAlgo algo, cudaStream_t stream) override;
    ncclResult_t reduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root, GpuAlgo algo, cudaStream_t stream) override;
    ncclResult_t send(const void* buf, size_t bytes, int peer, cudaStream_t stream) override;
    ncclResult_t recv(void* buf, size_t bytes, int peer, cudaStream_t stream) override;
    void group_start() override { in_group_ = true; }
    ncclResult_t group_end() override;
    void group_same_shape(int nops) override {
        int per = nops > 0 ? sm_count_ / nops : p2p_ctas_;
        if (per > p2p_ctas_) per = p2p_ctas_;
        if (per < 1) per = 1;
        group_ctas_ = per;
    }
    ncclResult_t local_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream) override {
        DeviceGuard g(dev_);
        launches_++;
        return cuda_result(launch_local_copy(dst, src, bytes, stream), "local copy");
    }

    ncclResult_t mem_alloc(void** ptr, size_t size) override;
    ncclResult_t mem_free(void* ptr) override;
    ncclResult_t register_buffer(void* buf, size_t size) override;
    ncclResult_t deregister_buffer(void* buf) override;

    ncclResult_t async_error(char* msg, size_t msg_len) override;
    ncclResult_t debug_check(char* msg, size_t msg_len) override;
    void abort(int failed_rank) override;
    void quiesce() override { DeviceGuard g(dev_); cudaDeviceSynchronize(); cudaGetLastError(); }
    GpuAlgo last_algo(int coll) const override { return last_[coll]; }
    int device() const override { return dev_; }
    std::string topology() const override { return topology_json(topo_); }
    bool has_multicast() const override { return pool_.mc_base != nullptr; }
    uint64_t launches() const override { return launches_; }
    uint64_t stat(const char* name) const override;
    bool is_symmetric(const void* p, size_t bytes) const override {
        for (const auto& s : user_segs_) if ((const char*)p >= s.base[rank_] && (const char*)p + bytes <= s.base[rank_] + s.size) return true;
        return false;
    }
    bool set_param(const char* name, int value) override;

private:
    struct DeviceGuard {
        int prev = -1;
        explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
        ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
    };
    ncclResult_t precheck();
    ncclResult_t cuda_result(cudaError_t e, const char* what);
    CollArgs base_args(const void* send, void* recv, ncclRedOp_t op, int root);
    /** Fill the symmetric views of a user buffer; false when it is not inside a dcclMemAlloc segment. */
    bool sym_view(const void* p, size_t bytes, const char** peers, const char** mc) const;
    /** Lazy registration: the ranks exchange which allocations `send` and `recv` lie in and open what is new. True
     *  (on every rank alike) when all ranks can address all buffers; fills the peers' views of both. Collective. */
    bool auto_view(const void* send, const void* recv, const char** send_peers, const char** recv_peers);
    void close_import(const AutoImport& im);
    /** Map (or find) allocation `id` at `base` of rank `owner`; nullptr when it cannot be opened. */
    AutoImport* import_allocation(int owner, unsigned long long base, unsigned long long id, size_t size, const cudaIpcMemHandle_t& handle);
    /** A large receive: where `buf` lies, for the sender (symmetric segment, exported allocation, or neither). */
    void describe_receive_buffer(const void* buf, size_t bytes, P2pOp* op);
    /** A large send: pick up what `peer` has exported since the last look. */
    void poll_exports(int peer);
    int ctas_for(int tuned) const;
    /** Move the sequence number to the device counter (calls become replayable from a CUDA graph) or back to
     *  the host. Every rank must switch at the same point of its call order. Waits for the device to go idle.
     *  Graphs captured in device mode must not be replayed after switching back: they would go on from the device
     *  word while eager calls have moved the host's number. */
    bool set_device_seq(bool on);
    /** Refuse what a capturing stream cannot replay correctly. */
    ncclResult_t capture_check(cudaStream_t stream, bool p2p);
    ncclResult_t p2p_launch(std::vector<P2pOp>& ops, cudaStream_t stream, int ctas_per_op = 0);
    /** With DCCL/device_stamps on: log a timestamp when `stream` reaches this point (kernel begin / end on the device time line). */
    void stamp(cudaStream_t stream, uint64_t tag, uint64_t extra);
public:
    void stamp_begin(cudaStream_t s, uint64_t coll) { stamp(s, TT_DEVICE_KERNEL_BEGIN, coll); }
    void stamp_end(cudaStream_t s, uint64_t coll) { stamp(s, TT_DEVICE_KERNEL_END, coll); }
private:

    /** Every rank describes its GPU and its view of the peers' GPUs; all ranks end with the same table. */
    bool discover_topology(std::string* err);
    Topology topo_;
    Bootstrap* bs_;
    int dev_, rank_, n_;
    SymAllocator* sym_ = nullptr;
    SymSegment pool_;
    DevComm dc_;
    uint32_t* status_host_ = nullptr;   // ST_WORDS status words, then the abort word
    uint32_t* status_dev_ = nullptr;
    size_t stage_bytes_ = 0;
    uint32_t seq_ = 0;                  // last sequence number given out by the host
    uint32_t* seq_dev_ = nullptr;       // device counter: {next sequence number, CTAs done}
    bool device_seq_ = false;
    Tuner tuner_;
    GpuAlgo last_[COLL_COUNT];
    uint64_t launches_ = 0;
    int ctas_override_ = 0;
    int p2p_ctas_ = 32;                   // measured: 574 / 649 GB/s per direction at 64 / 256 MB with 32 CTAs per operation, 558 / 629 with 16
    int threads_ = 512;
    int sm_count_ = 148;
    size_t pipe_min_bytes_ = 16u << 20;   // ordinary-buffer switch all-reduce is pipelined from this size on (0 = never)
    int pipe_ctas_ = 112;                 // grid of the pipelined switch all-reduce: pipe_nv_ctas_ switch CTAs, the rest copy in / out
    int pipe_nv_ctas_ = 16;
    int pipe_teams_ = 2;                  // the switch CTAs take the chunks in turn, in this many teams
    int pipe_unroll_ = 4;                 // vectors in flight per thread in the pipeline's switch pass
    int unroll_ = 8;
    bool rooted_pipe_ = false;            // broadcast / reduce of large ordinary buffers: pipelined switch form (nvls_rooted.cu)
    size_t rooted_pipe_min_bytes_ = 16u << 20;
    bool direct_rooted_ = true;           // reduce from the lazy-registration threshold on, broadcast from direct_bcast_min_bytes_
    int direct_rooted_ctas_ = 64;         // on: zero-copy peer forms (direct.cu). Grid of the reduce (8 GPUs, 256 MB: 598 us with 64 CTAs, 640 with 128)
    bool direct_reduce_small_ = false;    // worlds of 2-4 ranks: zero-copy reduce from the lazy-registration threshold on too (default: from 32 MB)
    int direct_bcast_ctas_ = 128;         // and of the broadcast (506 us with 64, 487 with 128)
    size_t direct_bcast_min_bytes_ = 32u << 20;   // below it the two hops of the zero-copy broadcast cost more than the staging copy
    bool sticky_error_ = false;
    bool guard_ = false;                  // guard words in the unused parts of the pool (canary.hpp)
    bool device_stamps_ = false;
    std::vector<SymSegment> user_segs_;
    std::vector<RegisteredBuffer> regs_;
    std::map<std::string, void*> ipc_opened_;   // handle bytes -> mapping, one open per allocation
    std::map<unsigned long long, AutoExport> auto_exports_;                  // by base address of the allocation
    std::map<std::pair<int, unsigned long long>, AutoImport> auto_imports_;  // by (owner, base address at the owner)
    size_t auto_min_bytes_ = 4u << 20;          // lazy registration serves calls from this size on (0: never)
    bool direct_rs_ = true;                     // reduce-scatter on addressable buffers: zero-copy pull, from direct_rs_min_bytes_ on
    size_t direct_rs_min_bytes_ = 32u << 20;    // (two ranks: from the lazy-registration threshold on)
    uint64_t symmetric_calls_ = 0;              // calls that the switch served in place on symmetric (dcclMemAlloc) buffers
    uint64_t zero_copy_calls_ = 0;              // calls served straight out of / into user memory by peer kernels
    unsigned long long sent_chunks_[kMaxPeers], recv_chunks_[kMaxPeers];
    unsigned long long sent_rdv_[kMaxPeers] = {0}, recv_rdv_[kMaxPeers] = {0};   // large (rendezvous) messages per peer and direction
    uint64_t bulletin_seen_[kMaxPeers] = {0};   // notes of each peer's bulletin read so far
    unsigned long long import_stamp_ = 0;
    bool p2p_rdv_ = true;                       // large send / recv meet and go zero-copy where the buffer is mapped
    bool in_group_ = false;
    std::vector<P2pOp> group_ops_;
    cudaStream_t group_stream_ = nullptr;
    int group_ctas_ = 0;               // CTAs per operation of the group being recorded (0: p2p_ctas_)
};

} // namespace dccl
