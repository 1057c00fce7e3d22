/**
 * The same start-up, query and all-reduce written with NCCL's spellings (ncclGetUniqueId, ncclCommInitRank,
 * ncclCommCount, ncclCommUserRank, ncclCommGetAsyncError, ncclGroupStart / End, ncclCommDestroy): code that
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
    printf("%d %d %s %.1f\n", n, r, ncclGetErrorString(e), y);
    return ncclCommDestroy(c) == ncclSuccess ? 0 : 3;
}
