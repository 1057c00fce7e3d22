/**
 * All-reduce among buffers that live on ONE device, through an entry point that
 * allocates nothing.
 *
 * This entry point has no counterpart in the original DCCL; it exists for
 * callers of this library that are not allowed to allocate device memory at
 * the moment they need a reduction:
 *
 *   - code that runs while the device memory is fully handed out to a
 *     framework's caching allocator or to a serving engine's KV-cache pool, so
 *     that a cudaMalloc may fail or stall (it synchronises the whole device);
 *   - code on a latency-critical path (one process driving several model
 *     replicas or pipeline partitions on one GPU, "threads as ranks") where
 *     the implicit device-wide synchronisation of cudaMalloc / cudaFree is not
 *     acceptable;
 *   - health checks that must work in a process whose memory budget is spent.
 *
 * The communicator-based API creates a pool per communicator (cuMemCreate /
 * cudaMalloc at init) and the test harness dccl_emu_collective allocates the
 * pools of its virtual ranks on every call. This entry point instead keeps the
 * scratch the two-shot all-reduce kernel needs (flag words and the staging
 * slots the ranks push their shards into) in a device array that is part of
 * the library image.
 *
 * What it computes: for r in [0, nranks): outputs[r][i] = op(inputs[0][i], ...,
 * inputs[nranks-1][i]), i in [0, count). Same kernel phases, flag protocol and
 * accumulation order as the two-shot variant of ncclAllReduce (push shards to
 * their owners, reduce, pull the result shards), with "ranks" being groups of
 * CTAs of one cooperative launch.
 *
 * Limits and rules:
 *   - nranks 1..DCCL_NOALLOC_MAX_RANKS, count * element size <=
 *     DCCL_NOALLOC_MAX_BYTES per rank; larger requests are refused with
 *     DCCL_NOALLOC_TOO_LARGE and a message on stderr, nothing is launched.
 *   - The scratch array is DCCL_NOALLOC_SCRATCH_BYTES (about 3.2 MB). Every
 *     device context that loads the library holds it until the process exits.
 *   - All calls on a device share that one array. The call clears the flag and
 *     status words it depends on (a memset on `stream`, ordered before the
 *     kernel); the staging part keeps the previous call's bytes, which are
 *     always overwritten before they are read. Two calls that overlap on the
 *     GPU (different streams, no ordering between them) race on the array:
 *     order them, e.g. by using one stream.
 *   - The first call on each device looks up the device address of the array
 *     (cudaGetSymbolAddress, with that device current) and caches it. That
 *     first call should be made before any stream capture begins.
 *   - inputs / outputs are host arrays of nranks device pointers (read during
 *     the call, not kept). Element pointers must be aligned to the element
 *     size; 16-byte aligned pointers take the vector path. outputs[r] may
 *     equal inputs[r].
 *   - device_status, when not null, is a device int the kernel sets to 0 on
 *     success or to 1 if a wait between the CTA groups gave up (bounded wait,
 *     2 s); read it after synchronising the stream.
 *   - The launch is cooperative (nranks x 4 CTAs), so it needs a device that
 *     supports cooperative launches and that many CTAs resident at once.
 *   - No cudaMalloc, cudaFree, cudaMallocAsync, cudaHostAlloc or allocating
 *     library routine is called, on any path.
 */
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DCCL_NOALLOC_MAX_RANKS 8
#define DCCL_NOALLOC_MAX_BYTES (256u * 1024u)
/* per rank: 16 KB of flag words + (ranks + 1) staging slots of MAX_BYTES / ranks (worst case, two ranks:
 * 1.5 x MAX_BYTES) + rounding slack; plus one status page for the whole array */
#define DCCL_NOALLOC_RANK_BYTES (16u * 1024u + DCCL_NOALLOC_MAX_BYTES + DCCL_NOALLOC_MAX_BYTES / 2u + 4096u)
#define DCCL_NOALLOC_SCRATCH_BYTES (DCCL_NOALLOC_MAX_RANKS * DCCL_NOALLOC_RANK_BYTES + 4096u)

#define DCCL_NOALLOC_OK 0
#define DCCL_NOALLOC_BAD_ARGUMENT (-1)
#define DCCL_NOALLOC_TOO_LARGE (-2)
#define DCCL_NOALLOC_CUDA_ERROR (-3)

/**
 * dtype: ncclDataType_t value (0 int8 ... 9 bfloat16); op: ncclRedOp_t value (0 sum, 1 prod, 2 max,
 * 3 min, 4 avg); stream: a cudaStream_t (0 for the default stream). Returns DCCL_NOALLOC_OK when the
 * work was enqueued, or one of the negative codes above after printing the reason to stderr.
 */
int dccl_allreduce_one_device_noalloc(int nranks, int dtype, int op, size_t count, const void* const* inputs,
                                      void* const* outputs, int* device_status, void* stream);

#ifdef __cplusplus
}
#endif
