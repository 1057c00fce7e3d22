/**
 * Host-only build (make CUDA=0): the library keeps its full API, every pointer
 * is host memory and device calls are refused. Mirrors the original's ability
 * to build without CUDA (reference CMakeLists.txt:70-89).
 */
#include "gpu_comm.hpp"

namespace dccl {

bool is_device_pointer(const void*, int* device) { if (device) *device = -1; return false; }
int cuda_device_count() { return 0; }
GpuComm* GpuComm::create(Bootstrap*, int, std::string* err) {
    if (err) *err = "this build of the library has no CUDA support";
    return nullptr;
}

} // namespace dccl
