/**
 * dccl_topo: what the library sees of this machine before any communicator exists. Prints, as JSON, the visible
 * GPUs (name, PCI address, SMs, memory, multicast support, NVLink links up and how many of them end in a switch),
 * the peer-access and peer-atomics matrices, and a one-line summary. `dccl_topo --nvml [library]` prints the
 * NVLink links per GPU from NVML alone. The original has no such tool: its fabric is described by the libfabric
 * provider in derecho.cfg (reference src/application/cfg/n0/derecho.cfg:115-146).
 */
#include <cstdio>
#include <cstring>
#include <vector>

extern "C" int dccl_local_topology_json(char* out, size_t len);
extern "C" int dccl_nvml_link_report(const char* lib, char* out, size_t len);

int main(int argc, char** argv) {
    std::vector<char> buf(65536);
    if (argc > 1 && !strcmp(argv[1], "--nvml")) {
        const int rc = dccl_nvml_link_report(argc > 2 ? argv[2] : nullptr, buf.data(), buf.size());
        printf("%s\n", buf.data());
        return rc == 0 ? 0 : 1;
    }
    if (argc > 1) {
        fprintf(stderr, "usage: dccl_topo [--nvml [libnvidia-ml.so.1]]\n");
        return 2;
    }
    dccl_local_topology_json(buf.data(), buf.size());
    printf("%s\n", buf.data());
    return 0;
}
