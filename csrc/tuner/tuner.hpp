/**
 * Variant selection: which kernel variant and how many CTAs serve a call.
 *
 * The original picks between ring and Rabenseifner from one configuration key
 * (reference src/core/dccl.cpp:412-413,454). Here the choice is made per
 * (collective, world size, element width, message bytes) from a table of
 * measured bus bandwidths: the built-in table was filled from sweeps on 2, 4
 * and 8 B200s, and a file named by DCCL_TUNE_FILE (or DCCL/tune_file) replaces
 * rows of it. File format, one rule per line, '#' comments:
 *
 *     <collective> <nranks|*> <max_bytes> <algorithm> <ctas> [<element bytes|*>]
 *
 * The optional last field binds a rule to one element width (1, 2, 4 or 8
 * bytes); rules without it serve every width. A rule for the exact world size
 * beats a wildcard one, and among those a rule for the exact width beats one
 * for every width.
 *
 * <collective> is allreduce, reducescatter, allgather, broadcast, reduce, or
 * allreduce_sym (all-reduce whose buffers live in symmetric memory, where the
 * switch variant copies nothing and wants fewer CTAs), or reducescatter_sym
 * (reduce-scatter whose send buffer is symmetric memory).
 *
 * Rules of one (collective, nranks) are tried in ascending max_bytes; the
 * first whose max_bytes >= message bytes wins (max_bytes accepts k/m/g
 * suffixes and "inf").
 */
#pragma once
#include "../gpu/gpu_comm.hpp"
#include <cstddef>
#include <string>
#include <vector>

namespace dccl {

/** Extra table key: all-reduce on symmetric (dcclMemAlloc) buffers. */
constexpr int TUNE_ALLREDUCE_SYM = COLL_COUNT;
/** Extra table key: reduce-scatter whose send buffer is symmetric memory (the switch can read it in place). */
constexpr int TUNE_REDUCESCATTER_SYM = COLL_COUNT + 1;
constexpr int TUNE_KEYS = COLL_COUNT + 2;

struct TuneRule {
    int coll;
    int nranks;          // 0 = any
    size_t max_bytes;    // inclusive upper bound
    GpuAlgo algo;
    int ctas;
    int esize = 0;       // element bytes this rule is for; 0 = any
};

struct TuneChoice {
    GpuAlgo algo;
    int ctas;
};

class Tuner {
public:
    Tuner();
    /** Replace / add rules from text in the file format. Returns rules accepted; bad lines go to *err. */
    int load_text(const std::string& text, std::string* err);
    bool load_file(const std::string& path, std::string* err);
    /** nvls_ok: the variant can serve this (dtype, op, buffers) on this communicator. */
    TuneChoice choose(int coll, int nranks, size_t bytes, bool nvls_ok, int esize = 0) const;
    const std::vector<TuneRule>& rules() const { return rules_; }
    /** The table in the file format (one rule per line), so that it can be written out, edited and loaded again. */
    std::string dump() const;

private:
    void add(const TuneRule& r);
    std::vector<TuneRule> rules_;
};

} // namespace dccl
