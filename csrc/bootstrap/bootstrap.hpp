/**
 * Single-box bootstrap: the replacement for the Derecho group join of the
 * original (reference src/core/dccl.cpp:287-332).
 *
 *  - control plane: rank 0 runs a small TCP server thread; every rank (rank 0
 *    included) is a client. The only primitive is an all-gather of equal-size
 *    blobs (barrier = all-gather of nothing), executed in lock step.
 *  - handle plane: one abstract unix datagram socket per rank, used to pass
 *    file descriptors (cuMem shareable handles) with SCM_RIGHTS.
 *  - liveness: a POSIX shared-memory control segment with one heartbeat word
 *    and pid per rank plus a group-wide abort word; a watchdog thread per rank
 *    bumps its own heartbeat every heartbeat_ms (100 ms, like the original's
 *    failure detector, reference cfg/n0/derecho.cfg:20-25) and flips `abort`
 *    when a peer process has exited or has not been heard from for too long.
 *  - data plane for host buffers: a second shared-memory segment with one
 *    byte FIFO per ordered rank pair.
 *
 * Fault injection for tests, all on the host: DCCL_FAULT is a comma separated
 * list of  drop_hello@<rank>  (that rank never says hello: peers time out),
 * delay_ms=<n>@<rank>  (that rank sleeps before every control message) and
 * exit_at_barrier=<k>@<rank>  (that rank _exit()s when it reaches its k-th
 * control operation).
 */
#pragma once
#include <dccl/dccl.hpp>
#include <atomic>
#include <cstdint>
#include <deque>
#include <functional>
#include <string>
#include <thread>
#include <vector>

namespace dccl {

static const int kMaxRanks = 64;       // host backend limit
static const int kMaxGpuRanks = 8;     // one NVSwitch box

struct UniqueIdData {
    uint32_t magic;
    uint32_t port;
    uint64_t token;
    char addr[64];
};
static_assert(sizeof(UniqueIdData) <= sizeof(dcclUniqueId), "unique id too large");

/** Layout of the shared control segment. */
struct CtlRank {
    std::atomic<uint64_t> heartbeat;
    std::atomic<int32_t> pid;
    std::atomic<int32_t> state;   // 0 = not joined, 1 = alive, 2 = left cleanly
    char pad[48];
};
/** Rendezvous of the group that the survivors of a failure form (dcclCommShrink). */
struct CtlShrink {
    std::atomic<uint32_t> generation;  // bumped by the leader after it filled in the fields below
    uint32_t pad;
    uint64_t alive_mask;               // ranks of this group that are members of the next one
    UniqueIdData id;                   // where the next group meets
};
/** One rank's entry of the exchange board: two generations of a small message, each with the number of the
 *  exchange that wrote it (fast_allgather). */
static const size_t kBoardBytes = 240;
struct CtlBoardSlot {
    std::atomic<uint64_t> seq;
    char pad[8];
    char data[kBoardBytes];
};
/** One rank's bulletin: small notes for whoever reads them later (bulletin_post / bulletin_read), kept in a ring. */
static const size_t kBulletinBytes = 96;
static const int kBulletinDepth = 32;
struct CtlBulletin {
    std::atomic<uint64_t> count;       // notes posted so far; note k lives in entry k % kBulletinDepth
    char pad[56];
    char note[kBulletinDepth][kBulletinBytes];
};
struct CtlSegment {
    std::atomic<uint32_t> abort;       // non-zero: somebody failed; value = 1 + failed rank
    std::atomic<uint32_t> abort_code;  // ncclResult_t
    char pad[56];
    CtlRank ranks[kMaxRanks];
    CtlShrink shrink;
    CtlBoardSlot board[kMaxRanks][2];
    CtlBulletin bulletin[kMaxGpuRanks];
};

/** One direction of a rank pair: single-producer single-consumer byte FIFO. */
struct ShmChannel {
    std::atomic<uint64_t> head;   // bytes written by the sender
    char pad0[56];
    std::atomic<uint64_t> tail;   // bytes consumed by the receiver
    char pad1[56];
    // data follows
};

class Bootstrap {
public:
    Bootstrap();
    ~Bootstrap();

    /** Bind + listen on rank 0. port 0 picks a free one. Fills id. */
    static bool create_listener(const std::string& addr, int port, UniqueIdData* id, std::string* err);

    /** Join. Blocks until all `world` ranks said hello or timeout_ms passed. */
    bool init(const UniqueIdData& id, int rank, int world, int timeout_ms, std::string* err);
    void shutdown();

    int rank() const { return rank_; }
    int world() const { return world_; }
    uint64_t token() const { return token_; }

    /** out must hold world*bytes. Returns false on peer failure / timeout. */
    bool allgather(const void* in, size_t bytes, void* out);
    bool barrier();
    bool broadcast(void* buf, size_t bytes, int root);
    /**
     * All-gather of a small message (at most kBoardBytes) through the shared control segment: no system call, a few
     * microseconds when the ranks arrive together. Every rank writes its message with the exchange number into its own
     * board entry and reads the others' once they carry that number. Two generations alternate: a rank can only start
     * exchange k + 2 after every rank has published k + 1, i.e. has read all of k. For per-call agreement on the host
     * (lazy buffer registration); all ranks must call it in the same order. False on abort or after the time limit.
     */
    bool fast_allgather(const void* in, size_t bytes, void* out);
    /**
     * One-sided notes in the shared control segment, for news that peers pick up whenever they next look (which
     * allocations this rank has exported): bulletin_post appends a note of at most kBulletinBytes to this rank's ring
     * and never waits; bulletin_read copies note number `index` of `rank`: 1 = copied, 0 = not posted yet, -1 = it has
     * been overwritten (the ring holds the last kBulletinDepth notes). Ranks 0 .. kMaxGpuRanks-1 only.
     */
    bool bulletin_post(const void* note, size_t bytes);
    int bulletin_read(int rank, uint64_t index, void* out, size_t bytes);

    bool send_fd(int peer, int fd, uint32_t tag);
    bool recv_fd(int peer, uint32_t tag, int* fd, int timeout_ms);
    /** Close every descriptor with this tag that has arrived but was not asked for (an exchange that was called off
     *  after some ranks had already sent). Call it after the ranks have agreed to give up: all sends precede that. */
    void discard_fds(uint32_t tag);

    /* liveness */
    CtlSegment* ctl() { return ctl_; }
    bool aborted() const { return ctl_ && ctl_->abort.load(std::memory_order_acquire) != 0; }
    void set_abort(int failed_rank, ncclResult_t code);
    int failed_rank() const { return ctl_ ? (int)ctl_->abort.load() - 1 : -1; }
    /** Called by the watchdog when it flips abort (lets the GPU side mirror the flag). */
    void on_abort(std::function<void(int)> cb) { abort_cb_ = cb; }
    int heartbeat_ms() const { return heartbeat_ms_; }
    /**
     * The ranks that are still there agree on a smaller group: the lowest surviving rank opens a new
     * rendezvous and publishes it, with the list of members, in the control segment; the others read it.
     * Members are the ranks whose process exists, that joined and did not leave, and that were not the
     * rank reported as failed. Every member must call this; a rank that is not a member gets false.
     */
    bool shrink_rendezvous(int timeout_ms, UniqueIdData* id, int* new_rank, int* new_world, std::string* err);

    /* host data plane */
    ShmChannel* channel(int src, int dst);
    size_t channel_bytes() const { return chan_bytes_; }

    const std::string& last_error() const { return err_; }

private:
    bool client_roundtrip(uint32_t op, const void* in, size_t bytes, void* out, size_t out_bytes);
    void server_loop();
    void watchdog_loop();
    bool map_segments(std::string* err);
    void fault_hook(const char* where);
    void pull_fd();

    int rank_ = -1, world_ = 0;
    uint64_t token_ = 0;
    int sock_ = -1;                 // client connection to the server
    int usock_ = -1;                // unix datagram socket for fds
    int listen_fd_ = -1;            // rank 0 only
    std::thread server_, watchdog_;
    std::atomic<bool> stop_{false};
    std::atomic<int64_t> server_deadline_{0};
    CtlSegment* ctl_ = nullptr;
    char* data_ = nullptr;
    size_t data_bytes_ = 0, chan_bytes_ = 0, chan_stride_ = 0;
    int heartbeat_ms_ = 100, hb_timeout_ms_ = 10000, op_timeout_ms_ = 60000;
    uint64_t ops_ = 0;
    uint64_t board_seq_ = 0;        // exchanges over the board so far
    uint32_t shrink_seen_ = 0;      // generation of the last shrink this rank took part in
    std::string err_;
    std::function<void(int)> abort_cb_;
    struct PendingFd { int src; uint32_t tag; int fd; };
    std::deque<PendingFd> pending_fds_;
    // fault injection
    int fault_delay_ms_ = 0;
    long fault_exit_at_ = -1;
    bool fault_drop_hello_ = false;
};

} // namespace dccl
