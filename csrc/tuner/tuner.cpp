#include "tuner.hpp"
#include "../core/config.hpp"
#include "../core/log.hpp"
#include <algorithm>
#include <cstdlib>
#include <fstream>
#include <sstream>

namespace dccl {

static const size_t kInf = ~(size_t)0;

/* Built-in table. Message bytes are the per-rank buffer for all-reduce /
 * broadcast / reduce and the full gathered vector for reduce-scatter /
 * all-gather. */
static const TuneRule kBuiltin[] = {
    // Measured on 8 x B200 (bf16 sum; sweep of every variant x CTA count, best per size bucket).
    // all-reduce, ordinary buffers: packets while latency bound (8-15 us to 64 KB), the two-shot packet form to 2 MB
    // (16.5-23 us where the staged switch form and NCCL take 28-32), then the switch through staging, pipelined from
    // 16 MB on (staging half as a ring of 16 MB chunk slots, grid of 112 CTAs: 812-822 GB/s at 1 GB against 728 for NCCL)
    {COLL_ALLREDUCE, 0, 64u << 10, ALGO_ONESHOT, 8},
    {COLL_ALLREDUCE, 0, 2u << 20, ALGO_TWOSHOT_LL, 32},
    {COLL_ALLREDUCE, 0, 8u << 20, ALGO_NVLS, 64},
    {COLL_ALLREDUCE, 0, kInf, ALGO_NVLS, 128},
    // two ranks (measured on 2 x B200): the switch fetches the local copy over NVLink as well, so the peer-to-peer
    // variants win for large messages, zero-copy on buffers the peers can address (symmetric, registered, or mapped
    // lazily inside the call): 670 GB/s at 1 GB against 410 through the switch and 567 for NCCL. Between 64 KB and
    // 1 MB the two-shot packet form (no barrier) takes 8.5 us where the barrier forms take 19-21 and NCCL 10.7-13.
    {COLL_ALLREDUCE, 2, 64u << 10, ALGO_ONESHOT, 8},
    {COLL_ALLREDUCE, 2, 1u << 20, ALGO_TWOSHOT_LL, 32},
    {COLL_ALLREDUCE, 2, kInf, ALGO_TWOSHOT, 128},
    {TUNE_ALLREDUCE_SYM, 2, 64u << 10, ALGO_ONESHOT, 8},
    {TUNE_ALLREDUCE_SYM, 2, 1u << 20, ALGO_TWOSHOT_LL, 32},
    {TUNE_ALLREDUCE_SYM, 2, kInf, ALGO_TWOSHOT, 128},
    {TUNE_REDUCESCATTER_SYM, 2, 256u << 10, ALGO_ONESHOT, 8},
    {TUNE_REDUCESCATTER_SYM, 2, kInf, ALGO_TWOSHOT, 128},
    // four ranks (measured on 4 x B200, bf16): packets to 64 KB, the two-shot packet form to 2 MB (10.5-19 us against 16-22
    // for the staged switch form and for NCCL), then the zero-copy peer form on ordinary buffers (lazy registration):
    // 606 / 651 / 667 GB/s at 64 MB / 256 MB / 1 GB against 535 / 568 / 611 for NCCL; buffers that cannot be exported fall
    // back to the pipelined switch form (dispatcher). Symmetric buffers: the switch in place, 690 GB/s at 1 GB with 8-32 CTAs.
    {COLL_ALLREDUCE, 4, 64u << 10, ALGO_ONESHOT, 8},
    {COLL_ALLREDUCE, 4, 2u << 20, ALGO_TWOSHOT_LL, 32},
    {COLL_ALLREDUCE, 4, kInf, ALGO_TWOSHOT, 128},
    {TUNE_ALLREDUCE_SYM, 4, 64u << 10, ALGO_ONESHOT, 8},
    {TUNE_ALLREDUCE_SYM, 4, 2u << 20, ALGO_TWOSHOT_LL, 32},
    {TUNE_ALLREDUCE_SYM, 4, kInf, ALGO_NVLS, 16},
    // all-reduce, symmetric buffers: zero-copy switch variant; 8-32 CTAs saturate it, more only add contention
    {TUNE_ALLREDUCE_SYM, 0, 64u << 10, ALGO_ONESHOT, 8},
    {TUNE_ALLREDUCE_SYM, 0, kInf, ALGO_NVLS, 16},
    // reduce-scatter from a symmetric send buffer: in-switch reduction straight out of the user's memory wins from 64 MB on
    {TUNE_REDUCESCATTER_SYM, 0, 256u << 10, ALGO_ONESHOT, 8},
    {TUNE_REDUCESCATTER_SYM, 0, 1u << 20, ALGO_TWOSHOT, 32},
    {TUNE_REDUCESCATTER_SYM, 0, 48u << 20, ALGO_TWOSHOT, 128},
    {TUNE_REDUCESCATTER_SYM, 0, kInf, ALGO_NVLS, 64},
    {COLL_REDUCESCATTER, 0, 256u << 10, ALGO_ONESHOT, 8},
    {COLL_REDUCESCATTER, 0, 1u << 20, ALGO_TWOSHOT, 32},
    {COLL_REDUCESCATTER, 0, kInf, ALGO_TWOSHOT, 128},
    {COLL_ALLGATHER, 2, 64u << 10, ALGO_ONESHOT, 8},
    {COLL_ALLGATHER, 2, 8u << 20, ALGO_NVLS, 128},
    {COLL_ALLGATHER, 2, kInf, ALGO_TWOSHOT, 128},
    {COLL_ALLGATHER, 0, 256u << 10, ALGO_ONESHOT, 8},
    {COLL_ALLGATHER, 0, 1u << 20, ALGO_NVLS, 32},
    {COLL_ALLGATHER, 0, 16u << 20, ALGO_NVLS, 128},       // 16 MB: 40 us through the switch, 47 by peer loads
    {COLL_ALLGATHER, 0, kInf, ALGO_TWOSHOT, 128},
    // broadcast / reduce: packets, then the switch through staging; on buffers the peers can address (or can map on first
    // use) the dispatcher takes the zero-copy peer forms instead: reduce from 4 MB on (worlds of up to four ranks: 32 MB), broadcast from 32 MB (two ranks: 16 MB)
    {COLL_BROADCAST, 0, 256u << 10, ALGO_ONESHOT, 16},
    {COLL_BROADCAST, 0, kInf, ALGO_NVLS, 64},
    {COLL_REDUCE, 0, 64u << 10, ALGO_ONESHOT, 8},
    {COLL_REDUCE, 0, 2u << 20, ALGO_TWOSHOT_LL, 32},       // folded shards to the root as packets: no barrier (the staged form has two)
    {COLL_REDUCE, 0, kInf, ALGO_NVLS, 128},
};

Tuner::Tuner() {
    for (const auto& r : kBuiltin) add(r);
    std::string path = Config::global().get_str("DCCL/tune_file", "");
    if (!path.empty()) {
        std::string err;
        if (!load_file(path, &err)) dccl_warn("tuning file %s: %s", path.c_str(), err.c_str());
    }
}

void Tuner::add(const TuneRule& r) {
    for (auto& x : rules_)
        if (x.coll == r.coll && x.nranks == r.nranks && x.max_bytes == r.max_bytes && x.esize == r.esize) { x = r; return; }
    rules_.push_back(r);
    std::stable_sort(rules_.begin(), rules_.end(), [](const TuneRule& a, const TuneRule& b) {
        if (a.coll != b.coll) return a.coll < b.coll;
        if (a.nranks != b.nranks) return a.nranks > b.nranks;   // exact world sizes before the wildcard
        if (a.esize != b.esize) return a.esize > b.esize;       // exact element widths before the wildcard
        return a.max_bytes < b.max_bytes;
    });
}

std::string Tuner::dump() const {
    static const char* const kNames[] = {"allreduce", "reducescatter", "allgather", "broadcast", "reduce"};
    std::ostringstream out;
    for (const TuneRule& r : rules_) {
        const char* coll = r.coll == TUNE_ALLREDUCE_SYM ? "allreduce_sym" : r.coll == TUNE_REDUCESCATTER_SYM ? "reducescatter_sym"
                           : r.coll >= 0 && r.coll < (int)(sizeof(kNames) / sizeof(kNames[0])) ? kNames[r.coll] : nullptr;
        if (!coll) continue;
        out << coll << ' ';
        if (r.nranks) out << r.nranks; else out << '*';
        out << ' ';
        if (r.max_bytes == kInf) out << "inf";
        else if (r.max_bytes % (1u << 20) == 0) out << (r.max_bytes >> 20) << 'm';
        else if (r.max_bytes % (1u << 10) == 0) out << (r.max_bytes >> 10) << 'k';
        else out << r.max_bytes;
        out << ' ' << algo_name(r.algo) << ' ' << r.ctas;
        if (r.esize) out << ' ' << r.esize;
        out << '\n';
    }
    return out.str();
}

static bool parse_bytes(const std::string& s, size_t* out) {
    if (s == "inf" || s == "*") { *out = kInf; return true; }
    char* end = nullptr;
    unsigned long long v = strtoull(s.c_str(), &end, 0);
    if (end == s.c_str()) return false;
    if (*end == 'k' || *end == 'K') v <<= 10;
    else if (*end == 'm' || *end == 'M') v <<= 20;
    else if (*end == 'g' || *end == 'G') v <<= 30;
    else if (*end) return false;
    *out = (size_t)v;
    return true;
}

int Tuner::load_text(const std::string& text, std::string* err) {
    std::istringstream in(text);
    std::string line;
    int ok = 0, lineno = 0;
    bool cleared[TUNE_KEYS] = {false};
    while (std::getline(in, line)) {
        lineno++;
        size_t h = line.find('#');
        if (h != std::string::npos) line = line.substr(0, h);
        std::istringstream ls(line);
        std::string coll, nr, mb, algo;
        int ctas = 0;
        if (!(ls >> coll)) continue;
        if (!(ls >> nr >> mb >> algo >> ctas)) { if (err) *err += "line " + std::to_string(lineno) + ": expected 5 fields; "; continue; }
        TuneRule r;
        std::string width;
        r.esize = (ls >> width) && width != "*" ? atoi(width.c_str()) : 0;
        r.coll = coll == "allreduce_sym" ? TUNE_ALLREDUCE_SYM : coll == "reducescatter_sym" ? TUNE_REDUCESCATTER_SYM : parse_collective_name(coll.c_str());
        r.nranks = nr == "*" ? 0 : atoi(nr.c_str());
        r.algo = parse_algo_name(algo.c_str());
        r.ctas = ctas;
        if (r.coll < 0 || r.algo == ALGO_COUNT || !parse_bytes(mb, &r.max_bytes) || ctas < 1 || ctas > 256 ||
            (r.esize != 0 && r.esize != 1 && r.esize != 2 && r.esize != 4 && r.esize != 8)) {
            if (err) *err += "line " + std::to_string(lineno) + ": bad value; ";
            continue;
        }
        // a file that mentions a collective replaces the built-in rows of that collective
        if (!cleared[r.coll]) {
            cleared[r.coll] = true;
            rules_.erase(std::remove_if(rules_.begin(), rules_.end(), [&](const TuneRule& x) { return x.coll == r.coll; }), rules_.end());
        }
        add(r);
        ok++;
    }
    return ok;
}

bool Tuner::load_file(const std::string& path, std::string* err) {
    std::ifstream f(path);
    if (!f) { if (err) *err = "cannot open"; return false; }
    std::stringstream ss;
    ss << f.rdbuf();
    std::string e;
    int n = load_text(ss.str(), &e);
    if (err) *err = e;
    return n > 0;
}

TuneChoice Tuner::choose(int coll, int nranks, size_t bytes, bool nvls_ok, int esize) const {
    TuneChoice fallback = {ALGO_TWOSHOT, 32};
    // (exact world size, exact width), (exact world size, any width), (any world size, exact width), (any, any)
    for (int pass = 0; pass < 4; pass++) {
        if ((pass == 0 || pass == 2) && esize == 0) continue;
        for (const auto& r : rules_) {
            if (r.coll != coll) continue;
            if (pass < 2 ? r.nranks != nranks : r.nranks != 0) continue;
            if ((pass == 0 || pass == 2) ? r.esize != esize : r.esize != 0) continue;
            if (bytes > r.max_bytes) continue;
            if (r.algo == ALGO_NVLS && !nvls_ok) { fallback.ctas = r.ctas; continue; }
            return TuneChoice{r.algo, r.ctas};
        }
    }
    return fallback;
}

} // namespace dccl
