#include "topology.hpp"
#include "../device/prims.cuh"
#include "../core/log.hpp"
#include "driver_api.hpp"
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <nvml.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>

namespace dccl {

static_assert(kTopoMaxRanks == kMaxPeers, "the topology table and the device code disagree on the number of ranks");

namespace {

/** The read-only NVML entry points used here, resolved with dlopen so that the library does not depend on NVML. */
struct Nvml {
    void* h = nullptr;
    nvmlReturn_t (*Init)(void) = nullptr;
    nvmlReturn_t (*Shutdown)(void) = nullptr;
    nvmlReturn_t (*GetCount)(unsigned int*) = nullptr;
    nvmlReturn_t (*ByIndex)(unsigned int, nvmlDevice_t*) = nullptr;
    nvmlReturn_t (*ByPci)(const char*, nvmlDevice_t*) = nullptr;
    nvmlReturn_t (*Name)(nvmlDevice_t, char*, unsigned int) = nullptr;
    nvmlReturn_t (*LinkState)(nvmlDevice_t, unsigned int, nvmlEnableState_t*) = nullptr;
    nvmlReturn_t (*LinkVersion)(nvmlDevice_t, unsigned int, unsigned int*) = nullptr;
    nvmlReturn_t (*LinkRemoteType)(nvmlDevice_t, unsigned int, nvmlIntNvLinkDeviceType_t*) = nullptr;
    bool ok = false;
};

bool load_nvml(const char* lib, Nvml* n, std::string* err) {
    const char* path = lib && *lib ? lib : getenv("DCCL_NVML_LIB");
    if (!path || !*path) path = "libnvidia-ml.so.1";
    n->h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!n->h) { if (err) *err = std::string("cannot load ") + path; return false; }
    auto sym = [&](const char* a, const char* b) { void* p = dlsym(n->h, a); return p ? p : (b ? dlsym(n->h, b) : nullptr); };
    n->Init = (nvmlReturn_t (*)(void))sym("nvmlInit_v2", "nvmlInit");
    n->Shutdown = (nvmlReturn_t (*)(void))sym("nvmlShutdown", nullptr);
    n->GetCount = (nvmlReturn_t (*)(unsigned int*))sym("nvmlDeviceGetCount_v2", "nvmlDeviceGetCount");
    n->ByIndex = (nvmlReturn_t (*)(unsigned int, nvmlDevice_t*))sym("nvmlDeviceGetHandleByIndex_v2", "nvmlDeviceGetHandleByIndex");
    n->ByPci = (nvmlReturn_t (*)(const char*, nvmlDevice_t*))sym("nvmlDeviceGetHandleByPciBusId_v2", "nvmlDeviceGetHandleByPciBusId");
    n->Name = (nvmlReturn_t (*)(nvmlDevice_t, char*, unsigned int))sym("nvmlDeviceGetName", nullptr);
    n->LinkState = (nvmlReturn_t (*)(nvmlDevice_t, unsigned int, nvmlEnableState_t*))sym("nvmlDeviceGetNvLinkState", nullptr);
    n->LinkVersion = (nvmlReturn_t (*)(nvmlDevice_t, unsigned int, unsigned int*))sym("nvmlDeviceGetNvLinkVersion", nullptr);
    n->LinkRemoteType = (nvmlReturn_t (*)(nvmlDevice_t, unsigned int, nvmlIntNvLinkDeviceType_t*))sym("nvmlDeviceGetNvLinkRemoteDeviceType", nullptr);
    if (!n->Init || !n->Shutdown || !n->GetCount || !n->ByIndex || !n->LinkState) { if (err) *err = "NVML lacks the entry points"; dlclose(n->h); n->h = nullptr; return false; }
    if (n->Init() != NVML_SUCCESS) { if (err) *err = "nvmlInit failed"; dlclose(n->h); n->h = nullptr; return false; }
    n->ok = true;
    return true;
}

/** Ends the NVML session. The library itself stays loaded for the life of the process: other parts of the
 *  process (a framework's memory statistics, say) may hold it too, and unloading a driver library buys nothing. */
void unload_nvml(Nvml* n) {
    if (n->ok) n->Shutdown();
    n->h = nullptr;
    n->ok = false;
}

/** Active links, version of the first active one, links that end in a switch. */
void count_links(const Nvml& n, nvmlDevice_t dev, int* active, int* version, int* to_switch) {
    *active = 0; *version = -1; *to_switch = n.LinkRemoteType ? 0 : -1;
    for (unsigned int l = 0; l < NVML_NVLINK_MAX_LINKS; l++) {
        nvmlEnableState_t st = NVML_FEATURE_DISABLED;
        if (n.LinkState(dev, l, &st) != NVML_SUCCESS || st != NVML_FEATURE_ENABLED) continue;
        (*active)++;
        unsigned int v = 0;
        if (*version < 0 && n.LinkVersion && n.LinkVersion(dev, l, &v) == NVML_SUCCESS) *version = (int)v;
        nvmlIntNvLinkDeviceType_t rt;
        if (n.LinkRemoteType && n.LinkRemoteType(dev, l, &rt) == NVML_SUCCESS && rt == NVML_NVLINK_DEVICE_TYPE_SWITCH) (*to_switch)++;
    }
}

} // namespace

bool nvml_link_report(const char* lib, std::string* json, std::string* err) {
    Nvml n;
    if (!load_nvml(lib, &n, err)) return false;
    unsigned int count = 0;
    std::ostringstream o;
    o << "{\"gpus\": [";
    if (n.GetCount(&count) == NVML_SUCCESS)
        for (unsigned int i = 0; i < count; i++) {
            nvmlDevice_t dev;
            if (n.ByIndex(i, &dev) != NVML_SUCCESS) continue;
            char name[96] = "?";
            if (n.Name) n.Name(dev, name, sizeof(name));
            int active, version, to_switch;
            count_links(n, dev, &active, &version, &to_switch);
            o << (i ? ", " : "") << "{\"index\": " << i << ", \"name\": \"" << name << "\", \"nvlinks_active\": " << active
              << ", \"nvlink_version\": " << version << ", \"nvlinks_to_switch\": " << to_switch << "}";
        }
    o << "]}";
    unload_nvml(&n);
    if (json) *json = o.str();
    return true;
}

bool discover_gpu(int device, GpuInfo* out, std::string* err) {
    *out = GpuInfo();
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) { cudaGetLastError(); if (err) *err = "cudaGetDeviceProperties failed"; return false; }
    out->device = device;
    snprintf(out->name, sizeof(out->name), "%.63s", p.name);
    cudaDeviceGetPCIBusId(out->pci, (int)sizeof(out->pci), device);
    out->sm_count = p.multiProcessorCount;
    out->mem_bytes = (unsigned long long)p.totalGlobalMem;
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    std::string derr;
    const DriverApi* d = driver_api(&derr);
    CUdevice cu;
    int mc = 0;
    if (d && d->multicast_ok && d->DeviceGet(&cu, device) == CUDA_SUCCESS &&
        d->DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cu) == CUDA_SUCCESS) out->multicast = mc;
    Nvml n;
    std::string e;
    if (load_nvml(nullptr, &n, &e)) {
        nvmlDevice_t dev;
        if (n.ByPci && n.ByPci(out->pci, &dev) == NVML_SUCCESS) count_links(n, dev, &out->nvlinks_active, &out->nvlink_version, &out->nvlinks_to_switch);
        unload_nvml(&n);
    } else dccl_debug("NVLink links not counted: %s", e.c_str());
    return true;
}

void discover_peer_row(int device, const GpuInfo* gpus, int n, unsigned char* access, unsigned char* atomics) {
    for (int b = 0; b < n; b++) {
        access[b] = 255;
        atomics[b] = 0;
        int other = -1;
        if (cudaDeviceGetByPCIBusId(&other, gpus[b].pci) != cudaSuccess) { cudaGetLastError(); continue; }
        if (other == device) { access[b] = 2; atomics[b] = 1; continue; }
        int can = 0, at = 0;
        if (cudaDeviceCanAccessPeer(&can, device, other) != cudaSuccess) { cudaGetLastError(); continue; }
        access[b] = can ? 1 : 0;
        if (can && cudaDeviceGetP2PAttribute(&at, cudaDevP2PAttrNativeAtomicSupported, device, other) == cudaSuccess) atomics[b] = at ? 1 : 0;
        else cudaGetLastError();
    }
}

std::string topology_summary(const Topology& t) {
    if (t.nranks < 1) return "no GPUs";
    bool same = true, all_access = true, all_mc = true;
    int min_links = 1 << 30, min_switch = 1 << 30;
    for (int a = 0; a < t.nranks; a++) {
        if (strcmp(t.gpu[a].name, t.gpu[0].name)) same = false;
        if (!t.gpu[a].multicast) all_mc = false;
        if (t.gpu[a].nvlinks_active < min_links) min_links = t.gpu[a].nvlinks_active;
        if (t.gpu[a].nvlinks_to_switch < min_switch) min_switch = t.gpu[a].nvlinks_to_switch;
        for (int b = 0; b < t.nranks; b++) if (a != b && t.access[a][b] == 0) all_access = false;
    }
    char buf[320];
    char links[96] = "NVLink links unknown";
    if (min_links >= 0) snprintf(links, sizeof(links), "%d NVLink links up per GPU at least (%d to a switch)", min_links, min_switch < 0 ? 0 : min_switch);
    snprintf(buf, sizeof(buf), "%d x %s (%d SMs, %llu GB), %s, %s, multicast %s", t.nranks, same ? t.gpu[0].name : "mixed GPUs",
             t.gpu[0].sm_count, t.gpu[0].mem_bytes >> 30, links, all_access ? "all pairs peer-accessible" : "SOME PAIRS CANNOT ADDRESS EACH OTHER",
             all_mc ? "yes" : "no");
    return buf;
}

std::string topology_json(const Topology& t) {
    std::ostringstream o;
    o << "{\"nranks\": " << t.nranks << ", \"gpus\": [";
    for (int a = 0; a < t.nranks; a++) {
        const GpuInfo& g = t.gpu[a];
        o << (a ? ", " : "") << "{\"rank\": " << a << ", \"device\": " << g.device << ", \"name\": \"" << g.name << "\", \"pci\": \"" << g.pci
          << "\", \"sm_count\": " << g.sm_count << ", \"mem_bytes\": " << g.mem_bytes << ", \"cc\": \"" << g.cc_major << "." << g.cc_minor
          << "\", \"multicast\": " << g.multicast << ", \"nvlinks_active\": " << g.nvlinks_active << ", \"nvlink_version\": " << g.nvlink_version
          << ", \"nvlinks_to_switch\": " << g.nvlinks_to_switch << "}";
    }
    o << "], \"peer_access\": [";
    for (int a = 0; a < t.nranks; a++) {
        o << (a ? ", [" : "[");
        for (int b = 0; b < t.nranks; b++) o << (b ? ", " : "") << (int)t.access[a][b];
        o << "]";
    }
    o << "], \"peer_atomics\": [";
    for (int a = 0; a < t.nranks; a++) {
        o << (a ? ", [" : "[");
        for (int b = 0; b < t.nranks; b++) o << (b ? ", " : "") << (int)t.atomics[a][b];
        o << "]";
    }
    o << "]}";
    return o.str();
}

} // namespace dccl

extern "C" {

/**
 * The GPUs this process can see, described like the ranks of a communicator (rank = CUDA ordinal), for the
 * dccl_topo tool. Returns the number of GPUs (0 and an empty table when there is no usable driver).
 */
int dccl_local_topology_json(char* out, size_t len) {
    using namespace dccl;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); n = 0; }
    if (n > kTopoMaxRanks) n = kTopoMaxRanks;
    Topology t;
    t.nranks = n;
    memset(t.access, 0, sizeof(t.access));
    memset(t.atomics, 0, sizeof(t.atomics));
    std::string err;
    for (int d = 0; d < n; d++) discover_gpu(d, &t.gpu[d], &err);
    for (int d = 0; d < n; d++) discover_peer_row(d, t.gpu, n, t.access[d], t.atomics[d]);
    if (out && len) {
        const std::string j = topology_json(t);
        const std::string s = n ? topology_summary(t) : std::string("no CUDA devices");
        snprintf(out, len, "{\"summary\": \"%s\", \"topology\": %s}", s.c_str(), j.c_str());
    }
    return n;
}

} // extern "C"
