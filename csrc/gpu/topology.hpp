/**
 * What the box looks like to a communicator: the GPU of every rank, which pairs can address each other's memory,
 * how many NVLink links each GPU has up and whether they end in a switch, and whether multicast (NVLS) is there.
 *
 * The original learns about its peers from the Derecho view (reference src/core/dccl.cpp:38-51,
 * internal_common.hpp:284-305) and about the fabric from libfabric; here the facts come from the CUDA runtime and,
 * read-only, from NVML (loaded at run time; without it the link fields stay unknown).
 */
#pragma once
#include <string>

namespace dccl {

constexpr int kTopoMaxRanks = 8;   // one NVSwitch domain (same number as kTopoMaxRanks of the device code)

struct GpuInfo {
    int device = -1;               // CUDA ordinal in the owning process
    char name[64] = {0};
    char pci[20] = {0};            // domain:bus:device.function
    int sm_count = 0;
    unsigned long long mem_bytes = 0;
    int cc_major = 0, cc_minor = 0;
    int multicast = 0;             // CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED
    int nvlinks_active = -1;       // -1: unknown (no NVML)
    int nvlink_version = -1;       // NVML's number for the first active link (NVML_NVLINK_VERSION_*)
    int nvlinks_to_switch = -1;    // active links whose remote end is a switch
};

struct Topology {
    int nranks = 0;
    GpuInfo gpu[kTopoMaxRanks];
    // access[a][b]: 1 = the process of rank a can address rank b's GPU memory (peer access), 0 = not, 2 = same GPU,
    // 255 = rank b's GPU is not visible to rank a's process, so only the memory mapping itself can tell
    unsigned char access[kTopoMaxRanks][kTopoMaxRanks];
    unsigned char atomics[kTopoMaxRanks][kTopoMaxRanks];   // native atomics over the link
};

/** CUDA runtime facts of one device of this process, plus its NVLink links when NVML can be loaded. */
bool discover_gpu(int device, GpuInfo* out, std::string* err);
/** Row of the access / atomics matrix of this process's `device` against the GPUs named by PCI bus id. */
void discover_peer_row(int device, const GpuInfo* gpus, int n, unsigned char* access, unsigned char* atomics);
/** One line for the log, e.g. "8 x NVIDIA B200 (148 SMs, 178 GB), 18 NVLink links each (18 to a switch), all pairs peer-accessible, multicast yes". */
std::string topology_summary(const Topology& t);
std::string topology_json(const Topology& t);

/** NVML only (no CUDA): links per GPU as JSON; library path from `lib` or DCCL_NVML_LIB or libnvidia-ml.so.1. False when NVML cannot be loaded. */
bool nvml_link_report(const char* lib, std::string* json, std::string* err);

} // namespace dccl
