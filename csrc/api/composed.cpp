/**
 * All-to-all, gather and scatter, composed of the grouped point-to-point calls.
 *
 * The original has no such entry points (its API ends with ncclSend / ncclRecv,
 * reference include/dccl/dccl.hpp:143-420, and a pair of those blocks the
 * host). Here every rank records its sends and receives between
 * dcclGroupStart and dcclGroupEnd, which issues them together: one kernel on
 * the stream for device buffers (one group of CTAs per peer), one progress
 * loop over the shared-memory FIFOs for host buffers. The rank's own block is
 * a local copy.
 */
#include "comm.hpp"
#include "../core/log.hpp"
#include "../core/types.hpp"
#include <cstring>
#include <vector>

namespace dccl {

namespace {

/** dst = src for the rank's own block; overlapping or identical ranges are left to memmove / skipped. */
ncclResult_t self_copy(dcclComm* c, void* dst, const void* src, size_t bytes, cudaStream_t stream) {
    if (!bytes || dst == src) return ncclSuccess;
    int dev = -1;
    if (!is_device_pointer(dst, &dev)) { memmove(dst, src, bytes); return ncclSuccess; }
    ncclResult_t r = ensure_gpu(c, dev);
    if (r != ncclSuccess) return r;
    return c->gpu->local_copy(dst, src, bytes, stream);
}

/** Both buffers (where given) on the host, or both on the device: the own block is copied between them. */
bool same_side(const void* a, const void* b) {
    if (!a || !b) return true;
    int da = -1, db = -1;
    return is_device_pointer(a, &da) == is_device_pointer(b, &db);
}

struct GroupScope {
    GroupScope() { dcclGroupStart(); }
    ncclResult_t end() { done = true; return dcclGroupEnd(); }
    ~GroupScope() { if (!done) dcclGroupEnd(); }
    bool done = false;
};

} // namespace

/** `uniform`: every rank is known to record the same operations (equal, non-empty blocks everywhere). */
static ncclResult_t all_to_all_impl(const void* sendbuff, const size_t* sendcounts, const size_t* sdispls, void* recvbuff,
                                    const size_t* recvcounts, const size_t* rdispls, ncclDataType_t dt, ncclComm_t comm, cudaStream_t stream,
                                    bool uniform) {
    if (!comm) return ncclInvalidArgument;
    const int rank = comm->bs.rank(), n = comm->bs.world();
    const size_t es = size_of_type(dt);
    if (!es || !sendcounts || !sdispls || !recvcounts || !rdispls) return ncclInvalidArgument;
    size_t total_s = 0, total_r = 0;
    for (int p = 0; p < n; p++) { total_s += sendcounts[p]; total_r += recvcounts[p]; }
    if ((total_s && !sendbuff) || (total_r && !recvbuff)) return ncclInvalidArgument;
    if (!same_side(sendbuff, recvbuff)) { dccl_error("dcclAllToAll: sendbuff and recvbuff must both be host or both be device memory"); return ncclInvalidArgument; }
    if (sendcounts[rank] != recvcounts[rank]) { dccl_error("dcclAllToAllv: rank %d sends %zu elements to itself but expects %zu", rank, sendcounts[rank], recvcounts[rank]); return ncclInvalidArgument; }
    const char* s = (const char*)sendbuff;
    char* r = (char*)recvbuff;
    ncclResult_t res = ncclSuccess;
    {
        GroupScope g;
        // receives are recorded first: on the device their CTAs get the lower block numbers and are resident
        // before any sender can wait for them
        for (int k = 1; k < n && res == ncclSuccess; k++) {
            const int p = (rank - k + n) % n;
            if (recvcounts[p]) res = ncclRecv(r + rdispls[p] * es, recvcounts[p], dt, p, comm, stream);
        }
        for (int k = 1; k < n && res == ncclSuccess; k++) {
            const int p = (rank + k) % n;
            if (sendcounts[p]) res = ncclSend(s + sdispls[p] * es, sendcounts[p], dt, p, comm, stream);
        }
        // every rank records the same 2 (n - 1) operations: the launch may shrink its CTA groups so that all of them
        // are resident together (with per-peer counts a rank cannot know what the others record, so it does not)
        if (comm->gpu && uniform && n > 1) comm->gpu->group_same_shape(2 * (n - 1));
        ncclResult_t e = g.end();
        if (res == ncclSuccess) res = e;
    }
    if (res == ncclSuccess) res = self_copy(comm, r + rdispls[rank] * es, s + sdispls[rank] * es, sendcounts[rank] * es, stream);
    return res;
}

ncclResult_t dcclAllToAllv(const void* sendbuff, const size_t* sendcounts, const size_t* sdispls, void* recvbuff,
                           const size_t* recvcounts, const size_t* rdispls, ncclDataType_t dt, ncclComm_t comm, cudaStream_t stream) {
    return all_to_all_impl(sendbuff, sendcounts, sdispls, recvbuff, recvcounts, rdispls, dt, comm, stream, false);
}

ncclResult_t dcclAllToAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t dt, ncclComm_t comm, cudaStream_t stream) {
    if (!comm) return ncclInvalidArgument;
    const int n = comm->bs.world();
    std::vector<size_t> counts((size_t)n, count), displs((size_t)n);
    for (int p = 0; p < n; p++) displs[(size_t)p] = (size_t)p * count;
    return all_to_all_impl(sendbuff, counts.data(), displs.data(), recvbuff, counts.data(), displs.data(), dt, comm, stream, count > 0);
}

ncclResult_t dcclGather(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t stream) {
    if (!comm) return ncclInvalidArgument;
    const int rank = comm->bs.rank(), n = comm->bs.world();
    const size_t es = size_of_type(dt);
    if (!es || root < 0 || root >= n || (count && !sendbuff) || (count && rank == root && !recvbuff)) return ncclInvalidArgument;
    if (!count) return ncclSuccess;
    if (rank == root && !same_side(sendbuff, recvbuff)) { dccl_error("dcclGather: sendbuff and recvbuff must both be host or both be device memory"); return ncclInvalidArgument; }
    if (rank != root) return ncclSend(sendbuff, count, dt, root, comm, stream);
    char* r = (char*)recvbuff;
    ncclResult_t res = ncclSuccess;
    {
        GroupScope g;
        for (int p = 0; p < n && res == ncclSuccess; p++)
            if (p != root) res = ncclRecv(r + (size_t)p * count * es, count, dt, p, comm, stream);
        ncclResult_t e = g.end();
        if (res == ncclSuccess) res = e;
    }
    if (res == ncclSuccess) res = self_copy(comm, r + (size_t)root * count * es, sendbuff, count * es, stream);
    return res;
}

ncclResult_t dcclScatter(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t stream) {
    if (!comm) return ncclInvalidArgument;
    const int rank = comm->bs.rank(), n = comm->bs.world();
    const size_t es = size_of_type(dt);
    if (!es || root < 0 || root >= n || (count && !recvbuff) || (count && rank == root && !sendbuff)) return ncclInvalidArgument;
    if (!count) return ncclSuccess;
    if (rank == root && !same_side(sendbuff, recvbuff)) { dccl_error("dcclScatter: sendbuff and recvbuff must both be host or both be device memory"); return ncclInvalidArgument; }
    if (rank != root) return ncclRecv(recvbuff, count, dt, root, comm, stream);
    const char* s = (const char*)sendbuff;
    ncclResult_t res = ncclSuccess;
    {
        GroupScope g;
        for (int p = 0; p < n && res == ncclSuccess; p++)
            if (p != root) res = ncclSend(s + (size_t)p * count * es, count, dt, p, comm, stream);
        ncclResult_t e = g.end();
        if (res == ncclSuccess) res = e;
    }
    if (res == ncclSuccess) res = self_copy(comm, recvbuff, s + (size_t)root * count * es, count * es, stream);
    return res;
}

} // namespace dccl
