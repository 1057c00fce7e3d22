#include "bootstrap.hpp"
#include <sched.h>
#include "../core/config.hpp"
#include "../core/log.hpp"

#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <map>
#include <mutex>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

namespace dccl {

static const uint32_t kMagic = 0xDCC1B200u;
enum : uint32_t { OP_HELLO = 1, OP_ALLGATHER = 2, OP_BYE = 3 };
enum : uint32_t { ST_OK = 0, ST_REMOTE = 1, ST_MISMATCH = 2 };

struct MsgHdr { uint32_t op; uint32_t aux; uint64_t len; };

static std::mutex g_listen_mu;
static std::map<uint64_t, int> g_listeners;  // token -> listening fd

static int64_t now_ms() {
    using namespace std::chrono;
    return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}

static bool write_all(int fd, const void* p, size_t n) {
    const char* c = (const char*)p;
    while (n) {
        ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
        if (w < 0) { if (errno == EINTR) continue; return false; }
        c += w; n -= (size_t)w;
    }
    return true;
}

/** Read exactly n bytes; gives up when `deadline_ms` passes or `*stop` becomes true. */
static bool read_all(int fd, void* p, size_t n, int64_t deadline_ms, const std::function<bool()>& stop) {
    char* c = (char*)p;
    while (n) {
        struct pollfd pf = {fd, POLLIN, 0};
        int pr = ::poll(&pf, 1, 100);
        if (pr < 0) { if (errno == EINTR) continue; return false; }
        if (pr == 0) {
            if (stop && stop()) return false;
            if (deadline_ms > 0 && now_ms() > deadline_ms) return false;
            continue;
        }
        ssize_t r = ::recv(fd, c, n, 0);
        if (r == 0) return false;
        if (r < 0) { if (errno == EINTR || errno == EAGAIN) continue; return false; }
        c += r; n -= (size_t)r;
    }
    return true;
}

static uint64_t random_token() {
    uint64_t t = 0;
    int fd = ::open("/dev/urandom", O_RDONLY);
    if (fd >= 0) { if (::read(fd, &t, sizeof(t)) != (ssize_t)sizeof(t)) t = 0; ::close(fd); }
    if (!t) t = ((uint64_t)now_ms() << 20) ^ (uint64_t)getpid();
    return t | 1ull;
}

Bootstrap::Bootstrap() {}
Bootstrap::~Bootstrap() { shutdown(); }

bool Bootstrap::create_listener(const std::string& addr, int port, UniqueIdData* id, std::string* err) {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) { if (err) *err = "socket() failed"; return false; }
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    struct sockaddr_in sa;
    memset(&sa, 0, sizeof(sa));
    sa.sin_family = AF_INET;
    sa.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, addr.c_str(), &sa.sin_addr) != 1) sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    if (::bind(fd, (struct sockaddr*)&sa, sizeof(sa)) != 0) {
        if (err) *err = "bind(" + addr + ":" + std::to_string(port) + ") failed: " + strerror(errno);
        ::close(fd);
        return false;
    }
    if (::listen(fd, 256) != 0) { if (err) *err = "listen() failed"; ::close(fd); return false; }
    socklen_t sl = sizeof(sa);
    getsockname(fd, (struct sockaddr*)&sa, &sl);
    memset(id, 0, sizeof(*id));
    id->magic = kMagic;
    id->port = ntohs(sa.sin_port);
    id->token = random_token();
    snprintf(id->addr, sizeof(id->addr), "%s", addr.c_str());
    std::lock_guard<std::mutex> g(g_listen_mu);
    g_listeners[id->token] = fd;
    return true;
}

void Bootstrap::fault_hook(const char* where) {
    (void)where;
    if (fault_delay_ms_ > 0) usleep((useconds_t)fault_delay_ms_ * 1000);
    if (fault_exit_at_ >= 0 && (long)ops_ == fault_exit_at_) {
        dccl_warn("fault injection: rank %d exits at control operation %llu", rank_, (unsigned long long)ops_);
        _exit(17);
    }
}

static void parse_faults(int rank, int* delay_ms, long* exit_at, bool* drop_hello) {
    const char* f = getenv("DCCL_FAULT");
    if (!f || !*f) return;
    std::string s(f);
    size_t pos = 0;
    while (pos <= s.size()) {
        size_t c = s.find(',', pos);
        std::string item = s.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
        pos = c == std::string::npos ? s.size() + 1 : c + 1;
        size_t at = item.find('@');
        if (at == std::string::npos) continue;
        if (atoi(item.c_str() + at + 1) != rank) continue;
        std::string what = item.substr(0, at);
        if (what == "drop_hello") *drop_hello = true;
        else if (what.compare(0, 9, "delay_ms=") == 0) *delay_ms = atoi(what.c_str() + 9);
        else if (what.compare(0, 16, "exit_at_barrier=") == 0) *exit_at = atol(what.c_str() + 16);
    }
}

bool Bootstrap::map_segments(std::string* err) {
    char name[96];
    snprintf(name, sizeof(name), "/dccl-%016llx-ctl", (unsigned long long)token_);
    int fd = shm_open(name, rank_ == 0 ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
    if (fd < 0) { if (err) *err = std::string("shm_open ") + name + ": " + strerror(errno); return false; }
    if (rank_ == 0 && ftruncate(fd, sizeof(CtlSegment)) != 0) { if (err) *err = "ftruncate ctl"; ::close(fd); return false; }
    void* p = mmap(nullptr, sizeof(CtlSegment), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) { if (err) *err = "mmap ctl"; return false; }
    ctl_ = (CtlSegment*)p;

    if (world_ > 1) {
        chan_bytes_ = (size_t)Config::global().get_int("DCCL/shm_channel_bytes", 1 << 20);
        if (chan_bytes_ < 4096) chan_bytes_ = 4096;
        chan_bytes_ = (chan_bytes_ + 63) / 64 * 64;
        chan_stride_ = (sizeof(ShmChannel) + chan_bytes_ + 4095) / 4096 * 4096;
        data_bytes_ = chan_stride_ * (size_t)world_ * (size_t)world_;
        snprintf(name, sizeof(name), "/dccl-%016llx-data", (unsigned long long)token_);
        fd = shm_open(name, rank_ == 0 ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
        if (fd < 0) { if (err) *err = std::string("shm_open ") + name + ": " + strerror(errno); return false; }
        if (rank_ == 0 && ftruncate(fd, (off_t)data_bytes_) != 0) { if (err) *err = "ftruncate data"; ::close(fd); return false; }
        p = mmap(nullptr, data_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        ::close(fd);
        if (p == MAP_FAILED) { if (err) *err = "mmap data"; return false; }
        data_ = (char*)p;
    }
    return true;
}

bool Bootstrap::fast_allgather(const void* in, size_t bytes, void* out) {
    if (bytes > kBoardBytes || !ctl_) { err_ = "fast_allgather: message too large"; return false; }
    if (world_ == 1) { memcpy(out, in, bytes); return true; }
    const uint64_t seq = ++board_seq_;
    const int gen = (int)(seq & 1u);
    CtlBoardSlot& mine = ctl_->board[rank_][gen];
    memcpy(mine.data, in, bytes);
    mine.seq.store(seq, std::memory_order_release);
    const int64_t deadline = now_ms() + op_timeout_ms_;
    for (int p = 0; p < world_; p++) {
        CtlBoardSlot& s = ctl_->board[p][gen];
        uint32_t spins = 0;
        while (s.seq.load(std::memory_order_acquire) != seq) {
            if ((++spins & 0x3ffu) == 0) {
                if (aborted()) { err_ = "fast_allgather: group aborted"; return false; }
                if (now_ms() > deadline) { err_ = "fast_allgather: timed out waiting for rank " + std::to_string(p); return false; }
                if (spins > (1u << 16)) sched_yield();
            }
        }
        memcpy((char*)out + (size_t)p * bytes, s.data, bytes);
    }
    return true;
}

bool Bootstrap::bulletin_post(const void* note, size_t bytes) {
    if (!ctl_ || rank_ < 0 || rank_ >= kMaxGpuRanks || bytes > kBulletinBytes) return false;
    CtlBulletin& b = ctl_->bulletin[rank_];
    const uint64_t k = b.count.load(std::memory_order_relaxed);      // this rank is the only writer
    memcpy(b.note[k % kBulletinDepth], note, bytes);
    b.count.store(k + 1, std::memory_order_release);
    return true;
}

int Bootstrap::bulletin_read(int rank, uint64_t index, void* out, size_t bytes) {
    if (!ctl_ || rank < 0 || rank >= kMaxGpuRanks || bytes > kBulletinBytes) return -1;
    CtlBulletin& b = ctl_->bulletin[rank];
    const uint64_t have = b.count.load(std::memory_order_acquire);
    if (index >= have) return 0;
    if (have - index > (uint64_t)kBulletinDepth) return -1;
    memcpy(out, b.note[index % kBulletinDepth], bytes);
    // the writer may have lapped the entry while it was being copied: it starts to overwrite entry `index` when it posts
    // note index + depth, i.e. once the count has reached index + depth
    std::atomic_thread_fence(std::memory_order_acquire);
    return b.count.load(std::memory_order_acquire) - index >= (uint64_t)kBulletinDepth ? -1 : 1;
}

ShmChannel* Bootstrap::channel(int src, int dst) {
    if (!data_) return nullptr;
    return (ShmChannel*)(data_ + chan_stride_ * ((size_t)src * (size_t)world_ + (size_t)dst));
}

bool Bootstrap::init(const UniqueIdData& id, int rank, int world, int timeout_ms, std::string* err) {
    rank_ = rank; world_ = world;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) {
        if (err) *err = "bad rank/world (" + std::to_string(rank) + "/" + std::to_string(world) + ")";
        return false;
    }
    Config& cfg = Config::global();
    heartbeat_ms_ = (int)cfg.get_int("DERECHO/heartbeat_ms", 100);
    heartbeat_ms_ = (int)cfg.get_int("DCCL/heartbeat_ms", heartbeat_ms_);
    if (heartbeat_ms_ < 1) heartbeat_ms_ = 1;
    hb_timeout_ms_ = (int)cfg.get_int("DCCL/heartbeat_timeout_ms", 10000);
    op_timeout_ms_ = (int)cfg.get_int("DCCL/bootstrap_timeout_ms", 60000);
    parse_faults(rank, &fault_delay_ms_, &fault_exit_at_, &fault_drop_hello_);
    int64_t deadline = now_ms() + timeout_ms;

    token_ = id.token;
    if (world == 1) {  // a world of one needs no sockets, no threads and no named segments
        void* p = mmap(nullptr, sizeof(CtlSegment), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
        if (p == MAP_FAILED) { if (err) *err = "mmap ctl"; return false; }
        ctl_ = (CtlSegment*)p;
        ctl_->ranks[0].pid.store((int32_t)getpid());
        ctl_->ranks[0].state.store(1);
        if (id.token) {  // a listener may exist for this id: it is not needed
            std::lock_guard<std::mutex> g(g_listen_mu);
            auto it = g_listeners.find(id.token);
            if (it != g_listeners.end()) { ::close(it->second); g_listeners.erase(it); }
        }
        return true;
    }
    if (rank == 0) {
        {
            std::lock_guard<std::mutex> g(g_listen_mu);
            auto it = g_listeners.find(id.token);
            if (it == g_listeners.end()) { if (err) *err = "rank 0 has no listener for this id"; return false; }
            listen_fd_ = it->second;
            g_listeners.erase(it);
        }
        if (!map_segments(err)) return false;
        server_ = std::thread([this] { server_loop(); });
    }

    if (fault_drop_hello_) {
        dccl_warn("fault injection: rank %d never says hello", rank_);
        while (now_ms() < deadline) usleep(50000);
        if (err) *err = "fault injection: hello dropped";
        return false;
    }

    // connect with retry: rank 0 may not be listening yet (cfg-directory recipe)
    struct sockaddr_in sa;
    memset(&sa, 0, sizeof(sa));
    sa.sin_family = AF_INET;
    sa.sin_port = htons((uint16_t)id.port);
    if (inet_pton(AF_INET, id.addr, &sa.sin_addr) != 1) sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    while (true) {
        sock_ = ::socket(AF_INET, SOCK_STREAM, 0);
        if (sock_ < 0) { if (err) *err = "socket() failed"; return false; }
        if (::connect(sock_, (struct sockaddr*)&sa, sizeof(sa)) == 0) break;
        ::close(sock_); sock_ = -1;
        if (now_ms() > deadline) {
            if (err) *err = std::string("cannot reach rank 0 at ") + id.addr + ":" + std::to_string(id.port);
            return false;
        }
        usleep(20000);
    }
    int one = 1;
    setsockopt(sock_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));

    fault_hook("hello");
    MsgHdr h = {OP_HELLO, (uint32_t)rank, (uint64_t)world};
    uint32_t magic = kMagic;
    if (!write_all(sock_, &magic, 4) || !write_all(sock_, &h, sizeof(h))) { if (err) *err = "hello send failed"; return false; }
    MsgHdr rh;
    uint64_t tok = 0;
    if (!read_all(sock_, &rh, sizeof(rh), deadline, nullptr) || rh.len != 8 || !read_all(sock_, &tok, 8, deadline, nullptr)) {
        if (err) *err = "timed out waiting for all " + std::to_string(world) + " ranks to join";
        return false;
    }
    if (rh.aux != ST_OK) { if (err) *err = "rank 0 refused the join (world size or rank mismatch)"; return false; }
    if (rank != 0) token_ = tok;   // rank 0 made the token; its server thread reads it concurrently
    if (rank != 0 && !map_segments(err)) return false;

    // unix datagram socket for file-descriptor passing
    usock_ = ::socket(AF_UNIX, SOCK_DGRAM, 0);
    if (usock_ >= 0) {
        struct sockaddr_un ua;
        memset(&ua, 0, sizeof(ua));
        ua.sun_family = AF_UNIX;
        int n = snprintf(ua.sun_path + 1, sizeof(ua.sun_path) - 1, "dccl-%016llx-%d", (unsigned long long)token_, rank_);
        if (::bind(usock_, (struct sockaddr*)&ua, (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + n)) != 0) {
            dccl_warn("cannot bind the unix socket for handle passing: %s", strerror(errno));
            ::close(usock_); usock_ = -1;
        }
    }

    ctl_->ranks[rank_].pid.store((int32_t)getpid());
    ctl_->ranks[rank_].heartbeat.store(1);
    ctl_->ranks[rank_].state.store(1, std::memory_order_release);
    if (!barrier()) { if (err) *err = "first barrier failed: " + err_; return false; }
    if (rank_ == 0) {  // everyone has mapped the segments: remove the names
        char name[96];
        snprintf(name, sizeof(name), "/dccl-%016llx-ctl", (unsigned long long)token_); shm_unlink(name);
        snprintf(name, sizeof(name), "/dccl-%016llx-data", (unsigned long long)token_); shm_unlink(name);
    }
    watchdog_ = std::thread([this] { watchdog_loop(); });
    return true;
}

void Bootstrap::set_abort(int failed_rank, ncclResult_t code) {
    if (!ctl_) return;
    uint32_t expect = 0;
    if (ctl_->abort.compare_exchange_strong(expect, (uint32_t)(failed_rank + 1))) ctl_->abort_code.store((uint32_t)code);
}

bool Bootstrap::shrink_rendezvous(int timeout_ms, UniqueIdData* id, int* new_rank, int* new_world, std::string* err) {
    if (!ctl_ || rank_ < 0) { if (err) *err = "not initialised"; return false; }
    const int failed = failed_rank();
    auto member = [&](int r) {
        if (r == failed) return false;
        if (ctl_->ranks[r].state.load(std::memory_order_acquire) != 1) return false;
        const int32_t pid = ctl_->ranks[r].pid.load(std::memory_order_acquire);
        return pid > 0 && (::kill((pid_t)pid, 0) == 0 || errno == EPERM);
    };
    if (!member(rank_)) { if (err) *err = "this rank was reported as failed or has left: it cannot be part of the smaller group"; return false; }
    int leader = -1;
    for (int r = 0; r < world_ && leader < 0; r++) if (member(r)) leader = r;
    CtlShrink& sh = ctl_->shrink;
    if (leader == rank_) {
        uint64_t mask = 0;
        for (int r = 0; r < world_; r++) if (member(r)) mask |= 1ull << r;
        UniqueIdData nid;
        std::string e;
        if (!create_listener("127.0.0.1", 0, &nid, &e)) { if (err) *err = e; return false; }
        sh.alive_mask = mask;
        sh.id = nid;
        shrink_seen_ = sh.generation.load(std::memory_order_relaxed) + 1;
        sh.generation.store(shrink_seen_, std::memory_order_release);
    } else {
        const int64_t deadline = now_ms() + timeout_ms;
        while (sh.generation.load(std::memory_order_acquire) == shrink_seen_) {
            if (now_ms() > deadline) { if (err) *err = "rank " + std::to_string(leader) + " did not open the smaller group in time"; return false; }
            if (!member(leader)) { if (err) *err = "rank " + std::to_string(leader) + " went away while the smaller group was being formed; call again"; return false; }
            usleep(200);
        }
        shrink_seen_ = sh.generation.load(std::memory_order_acquire);
    }
    const uint64_t mask = sh.alive_mask;
    if (!(mask >> rank_ & 1ull)) { if (err) *err = "the leader does not count this rank among the survivors"; return false; }
    *id = sh.id;
    int nr = 0, nw = 0;
    for (int r = 0; r < world_; r++) {
        if (!(mask >> r & 1ull)) continue;
        if (r < rank_) nr++;
        nw++;
    }
    *new_rank = nr;
    *new_world = nw;
    return true;
}

void Bootstrap::watchdog_loop() {
    std::vector<uint64_t> last(world_, 0);
    std::vector<int64_t> seen(world_, now_ms());
    bool reported = false;
    while (!stop_.load()) {
        ctl_->ranks[rank_].heartbeat.fetch_add(1, std::memory_order_relaxed);
        int64_t t = now_ms();
        for (int p = 0; p < world_ && !reported; p++) {
            if (p == rank_) continue;
            int st = ctl_->ranks[p].state.load(std::memory_order_acquire);
            if (st != 1) continue;
            int pid = ctl_->ranks[p].pid.load();
            if (pid > 0 && ::kill(pid, 0) != 0 && errno == ESRCH) {
                if (ctl_->ranks[p].state.load() == 1) {
                    dccl_error("rank %d (pid %d) has exited without leaving the group", p, pid);
                    set_abort(p, ncclRemoteError);
                }
                continue;
            }
            uint64_t hb = ctl_->ranks[p].heartbeat.load(std::memory_order_relaxed);
            if (hb != last[p]) { last[p] = hb; seen[p] = t; }
            else if (t - seen[p] > hb_timeout_ms_) {
                dccl_error("rank %d has not been heard from for %d ms", p, hb_timeout_ms_);
                set_abort(p, ncclRemoteError);
            }
        }
        if (!reported && aborted()) {
            reported = true;
            if (abort_cb_) abort_cb_(failed_rank());
        }
        usleep((useconds_t)heartbeat_ms_ * 1000);
    }
}

/* ---------------------------------------------------------------------- */

void Bootstrap::server_loop() {
    struct Client { int fd = -1; bool left = false; bool has = false; MsgHdr h{}; std::vector<char> payload; };
    std::vector<Client> cl(world_);
    int joined = 0;
    bool failed = false;
    int64_t join_deadline = now_ms() + (int64_t)Config::global().get_int("DCCL/init_timeout_ms", 120000);

    // phase 1: accept until everyone said hello
    while (joined < world_ && !stop_.load()) {
        struct pollfd pf = {listen_fd_, POLLIN, 0};
        int pr = ::poll(&pf, 1, 100);
        if (pr <= 0) { if (now_ms() > join_deadline) break; continue; }
        int fd = ::accept(listen_fd_, nullptr, nullptr);
        if (fd < 0) continue;
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        uint32_t magic = 0;
        MsgHdr h;
        int64_t dl = now_ms() + 5000;
        if (!read_all(fd, &magic, 4, dl, nullptr) || magic != kMagic || !read_all(fd, &h, sizeof(h), dl, nullptr) || h.op != OP_HELLO) {
            ::close(fd);
            continue;
        }
        int r = (int)h.aux;
        if (r < 0 || r >= world_ || (int)h.len != world_ || cl[r].fd >= 0) {
            MsgHdr rh = {OP_HELLO, ST_MISMATCH, 8};
            uint64_t z = 0;
            write_all(fd, &rh, sizeof(rh)); write_all(fd, &z, 8);
            ::close(fd);
            dccl_error("bootstrap: refused a hello (rank %d, world %llu; expected world %d)", r, (unsigned long long)h.len, world_);
            continue;
        }
        cl[r].fd = fd;
        joined++;
    }
    ::close(listen_fd_); listen_fd_ = -1;
    if (joined < world_) {
        dccl_error("bootstrap: only %d of %d ranks joined", joined, world_);
        for (auto& c : cl) if (c.fd >= 0) { ::close(c.fd); c.fd = -1; }   // joiners see EOF and fail
        return;
    }
    for (auto& c : cl) {
        MsgHdr rh = {OP_HELLO, ST_OK, 8};
        write_all(c.fd, &rh, sizeof(rh));
        write_all(c.fd, &token_, 8);
    }

    // phase 2: lock-step rounds
    auto reply_error = [&](Client& c) {
        MsgHdr rh = {OP_ALLGATHER, ST_REMOTE, 0};
        write_all(c.fd, &rh, sizeof(rh));
        c.has = false;
    };
    std::vector<struct pollfd> pfs;
    std::vector<int> idx;
    while (true) {
        // after this rank's own shutdown the server lingers a little for late leavers
        int64_t dl = server_deadline_.load();
        if (dl && now_ms() > dl) break;
        pfs.clear(); idx.clear();
        int alive = 0;
        for (int r = 0; r < world_; r++) {
            if (cl[r].fd < 0) continue;
            alive++;
            if (!cl[r].has) { pfs.push_back({cl[r].fd, POLLIN, 0}); idx.push_back(r); }
        }
        if (alive == 0) break;
        if (!pfs.empty()) {
            int pr = ::poll(pfs.data(), pfs.size(), 100);
            if (pr < 0 && errno != EINTR) break;
            for (size_t i = 0; i < pfs.size() && pr > 0; i++) {
                if (!(pfs[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
                Client& c = cl[idx[i]];
                MsgHdr h;
                bool ok = read_all(c.fd, &h, sizeof(h), now_ms() + 5000, nullptr);
                if (ok && h.op == OP_BYE) { c.left = true; ::close(c.fd); c.fd = -1; continue; }
                if (ok && h.len <= (1ull << 30)) {
                    c.payload.resize(h.len);
                    ok = h.len == 0 || read_all(c.fd, c.payload.data(), h.len, now_ms() + 30000, nullptr);
                } else ok = false;
                if (!ok) {  // connection lost without a goodbye: that rank failed
                    ::close(c.fd); c.fd = -1;
                    if (!c.left) {
                        if (!failed) dccl_error("bootstrap: lost rank %d", idx[i]);
                        failed = true;
                        set_abort(idx[i], ncclRemoteError);
                    }
                    continue;
                }
                c.h = h; c.has = true;
            }
        }
        if (failed) { for (auto& c : cl) if (c.fd >= 0 && c.has) reply_error(c); continue; }
        // a rank that left cleanly can no longer take part: remaining requests fail
        bool all = true, any_left = false;
        for (auto& c : cl) { if (c.fd < 0) { any_left = true; } else if (!c.has) all = false; }
        if (any_left) { for (auto& c : cl) if (c.fd >= 0 && c.has) reply_error(c); continue; }
        if (!all) continue;
        uint64_t len = cl[0].h.len;
        bool same = true;
        for (auto& c : cl) if (c.h.op != cl[0].h.op || c.h.len != len) same = false;
        if (!same) {
            dccl_error("bootstrap: ranks disagree on a control operation (different call order?)");
            for (auto& c : cl) { MsgHdr rh = {OP_ALLGATHER, ST_MISMATCH, 0}; write_all(c.fd, &rh, sizeof(rh)); c.has = false; }
            continue;
        }
        std::vector<char> all_data(len * (size_t)world_);
        for (int r = 0; r < world_; r++) if (len) memcpy(all_data.data() + len * r, cl[r].payload.data(), len);
        for (auto& c : cl) {
            MsgHdr rh = {OP_ALLGATHER, ST_OK, (uint64_t)all_data.size()};
            write_all(c.fd, &rh, sizeof(rh));
            if (!all_data.empty()) write_all(c.fd, all_data.data(), all_data.size());
            c.has = false;
        }
    }
    for (auto& c : cl) if (c.fd >= 0) ::close(c.fd);
}

bool Bootstrap::client_roundtrip(uint32_t op, const void* in, size_t bytes, void* out, size_t out_bytes) {
    ops_++;
    fault_hook("op");
    if (sock_ < 0) { err_ = "not connected"; return false; }
    if (aborted()) { err_ = "group aborted (rank " + std::to_string(failed_rank()) + " failed)"; return false; }
    MsgHdr h = {op, 0, (uint64_t)bytes};
    if (!write_all(sock_, &h, sizeof(h)) || (bytes && !write_all(sock_, in, bytes))) { err_ = "control send failed"; return false; }
    MsgHdr rh;
    int64_t deadline = now_ms() + op_timeout_ms_;
    auto stop = [this] { return aborted() || stop_.load(); };
    if (!read_all(sock_, &rh, sizeof(rh), deadline, stop)) {
        err_ = aborted() ? "group aborted (rank " + std::to_string(failed_rank()) + " failed)" : "control operation timed out";
        return false;
    }
    if (rh.aux != ST_OK) { err_ = rh.aux == ST_REMOTE ? "a peer failed or left" : "ranks disagree on the operation"; return false; }
    if (rh.len != out_bytes) { err_ = "control reply has unexpected size"; return false; }
    if (out_bytes && !read_all(sock_, out, out_bytes, deadline, stop)) { err_ = "control reply truncated"; return false; }
    return true;
}

bool Bootstrap::allgather(const void* in, size_t bytes, void* out) {
    if (world_ == 1) { if (bytes) memcpy(out, in, bytes); return true; }
    return client_roundtrip(OP_ALLGATHER, in, bytes, out, bytes * (size_t)world_);
}

bool Bootstrap::barrier() {
    if (world_ == 1) return true;
    return client_roundtrip(OP_ALLGATHER, nullptr, 0, nullptr, 0);
}

bool Bootstrap::broadcast(void* buf, size_t bytes, int root) {
    if (world_ == 1) return true;
    std::vector<char> all(bytes * (size_t)world_);
    if (!allgather(buf, bytes, all.data())) return false;
    memcpy(buf, all.data() + bytes * (size_t)root, bytes);
    return true;
}

/* ---------------- file-descriptor passing ---------------- */

bool Bootstrap::send_fd(int peer, int fd, uint32_t tag) {
    if (usock_ < 0) return false;
    struct sockaddr_un ua;
    memset(&ua, 0, sizeof(ua));
    ua.sun_family = AF_UNIX;
    int n = snprintf(ua.sun_path + 1, sizeof(ua.sun_path) - 1, "dccl-%016llx-%d", (unsigned long long)token_, peer);
    uint32_t body[2] = {(uint32_t)rank_, tag};
    struct iovec iov = {body, sizeof(body)};
    char cbuf[CMSG_SPACE(sizeof(int))];
    memset(cbuf, 0, sizeof(cbuf));
    struct msghdr msg;
    memset(&msg, 0, sizeof(msg));
    msg.msg_name = &ua;
    msg.msg_namelen = (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + n);
    msg.msg_iov = &iov; msg.msg_iovlen = 1;
    msg.msg_control = cbuf; msg.msg_controllen = sizeof(cbuf);
    struct cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET; cm->cmsg_type = SCM_RIGHTS; cm->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(cm), &fd, sizeof(int));
    for (int tries = 0; tries < 200; tries++) {
        if (::sendmsg(usock_, &msg, 0) >= 0) return true;
        if (errno != EAGAIN && errno != ENOBUFS && errno != EINTR && errno != ECONNREFUSED) break;
        usleep(5000);
    }
    err_ = std::string("sendmsg(SCM_RIGHTS) failed: ") + strerror(errno);
    return false;
}

bool Bootstrap::recv_fd(int peer, uint32_t tag, int* fd, int timeout_ms) {
    int64_t deadline = now_ms() + timeout_ms;
    while (true) {
        for (auto it = pending_fds_.begin(); it != pending_fds_.end(); ++it)
            if (it->src == peer && it->tag == tag) { *fd = it->fd; pending_fds_.erase(it); return true; }
        if (usock_ < 0) return false;
        struct pollfd pf = {usock_, POLLIN, 0};
        int pr = ::poll(&pf, 1, 100);
        if (pr <= 0) {
            if (aborted() || now_ms() > deadline) { err_ = "timed out waiting for a handle from rank " + std::to_string(peer); return false; }
            continue;
        }
        pull_fd();
    }
}

/** Take one datagram off the descriptor socket and park its descriptor in pending_fds_. */
void Bootstrap::pull_fd() {
    uint32_t body[2] = {0, 0};
    struct iovec iov = {body, sizeof(body)};
    char cbuf[CMSG_SPACE(sizeof(int))];
    struct msghdr msg;
    memset(&msg, 0, sizeof(msg));
    msg.msg_iov = &iov; msg.msg_iovlen = 1;
    msg.msg_control = cbuf; msg.msg_controllen = sizeof(cbuf);
    ssize_t r = ::recvmsg(usock_, &msg, MSG_DONTWAIT);
    if (r < (ssize_t)sizeof(body)) return;
    struct cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    if (!cm || cm->cmsg_type != SCM_RIGHTS) return;
    int got;
    memcpy(&got, CMSG_DATA(cm), sizeof(int));
    pending_fds_.push_back({(int)body[0], body[1], got});
}

void Bootstrap::discard_fds(uint32_t tag) {
    while (usock_ >= 0) {   // whatever has arrived by now, without waiting
        struct pollfd pf = {usock_, POLLIN, 0};
        if (::poll(&pf, 1, 0) <= 0) break;
        const size_t before = pending_fds_.size();
        pull_fd();
        if (pending_fds_.size() == before) break;
    }
    for (auto it = pending_fds_.begin(); it != pending_fds_.end();) {
        if (it->tag == tag) { ::close(it->fd); it = pending_fds_.erase(it); }
        else ++it;
    }
}

void Bootstrap::shutdown() {
    if (rank_ < 0) return;
    stop_.store(true);
    if (watchdog_.joinable()) watchdog_.join();
    if (ctl_) ctl_->ranks[rank_].state.store(2, std::memory_order_release);
    if (sock_ >= 0) {
        MsgHdr h = {OP_BYE, 0, 0};
        write_all(sock_, &h, sizeof(h));
        ::close(sock_); sock_ = -1;
    }
    if (server_.joinable()) {
        // the server ends when every client has left or vanished; the deadline covers a stuck one
        server_deadline_.store(now_ms() + 3000);
        server_.join();
    }
    if (usock_ >= 0) { ::close(usock_); usock_ = -1; }
    for (auto& p : pending_fds_) ::close(p.fd);
    pending_fds_.clear();
    if (data_) { munmap(data_, data_bytes_); data_ = nullptr; }
    if (ctl_) { munmap(ctl_, sizeof(CtlSegment)); ctl_ = nullptr; }
    rank_ = -1;
}

} // namespace dccl
