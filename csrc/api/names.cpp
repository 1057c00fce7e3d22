/** Names of algorithms and collectives as configuration files and tools spell them. */
#include "../gpu/gpu_comm.hpp"
#include <strings.h>

namespace dccl {

static const char* kAlgoNames[ALGO_COUNT] = {"auto", "ring", "rabenseifner", "oneshot", "twoshot", "nvls", "local", "twoshot_ll"};

const char* algo_name(GpuAlgo a) { return (int)a >= 0 && a < ALGO_COUNT ? kAlgoNames[a] : "?"; }

GpuAlgo parse_algo_name(const char* s) {
    if (!s) return ALGO_COUNT;
    for (int i = 0; i < ALGO_COUNT; i++) if (!strcasecmp(s, kAlgoNames[i])) return (GpuAlgo)i;
    if (!strcasecmp(s, "rhd") || !strcasecmp(s, "halving_doubling")) return ALGO_RABENSEIFNER;
    return ALGO_COUNT;
}

int parse_collective_name(const char* s) {
    if (!s) return -1;
    if (!strcasecmp(s, "allreduce") || !strcasecmp(s, "all_reduce")) return COLL_ALLREDUCE;
    if (!strcasecmp(s, "reducescatter") || !strcasecmp(s, "reduce_scatter")) return COLL_REDUCESCATTER;
    if (!strcasecmp(s, "allgather") || !strcasecmp(s, "all_gather")) return COLL_ALLGATHER;
    if (!strcasecmp(s, "broadcast") || !strcasecmp(s, "bcast")) return COLL_BROADCAST;
    if (!strcasecmp(s, "reduce")) return COLL_REDUCE;
    if (!strcasecmp(s, "sendrecv") || !strcasecmp(s, "send") || !strcasecmp(s, "recv")) return COLL_SENDRECV;
    return -1;
}

} // namespace dccl
