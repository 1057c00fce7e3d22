/**
 * The same start-up, query and all-reduce written with NCCL's spellings (ncclGetUniqueId, ncclCommInitRank,
 * ncclCommCount, ncclCommUserRank, ncclCommGetAsyncError, ncclGroupStart / End, ncclCommRegister / Deregister,
 * ncclAlltoAll / ncclGather / ncclScatter, ncclCommDestroy): code that
 * was written against NCCL compiles against this header with `using namespace dccl;`.
 */
#include <dccl/dccl.hpp>
#include <cstdio>
using namespace dccl;
int main() {
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return 1;
    ncclComm_t c;
    if (ncclCommInitRank(&c, 1, id, 0) != ncclSuccess) return 2;
    int n = 0, r = -1;
    ncclCommCount(c, &n); ncclCommUserRank(c, &r);
    ncclResult_t e;
    ncclCommGetAsyncError(c, &e);
    float x = 2.f, y = 0.f;
    ncclGroupStart(); ncclGroupEnd();
    ncclAllReduce(&x, &y, 1, ncclFloat32, ncclSum, c, nullptr);
    alignas(64) static float a[16], b[16];
    void* handle = nullptr;
    if (ncclCommRegister(c, a, sizeof(a), &handle) != ncclSuccess || handle != a) return 4;
    a[0] = 5.f;
    if (ncclAlltoAll(a, b, 16, ncclFloat32, c, nullptr) != ncclSuccess || b[0] != 5.f) return 5;
    a[1] = 6.f;
    if (ncclGather(a, b, 16, ncclFloat32, 0, c, nullptr) != ncclSuccess || b[1] != 6.f) return 6;
    a[2] = 7.f;
    if (ncclScatter(a, b, 16, ncclFloat32, 0, c, nullptr) != ncclSuccess || b[2] != 7.f) return 7;
    if (ncclCommDeregister(c, handle) != ncclSuccess) return 8;
    printf("%d %d %s %.1f\n", n, r, ncclGetErrorString(e), y);
    return ncclCommDestroy(c) == ncclSuccess ? 0 : 3;
}
