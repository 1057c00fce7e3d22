/**
 * Guard words in the unused parts of a symmetric pool (debug aid, `DCCL/debug_bounds = 1`).
 *
 * The pool is a fixed layout of regions (flag rows, credit words, two packet regions, send/recv FIFOs, staging
 * halves; csrc/device/prims.cuh). The bytes between two regions belong to nobody. With guarding on, the first and
 * last 4 KB of every such gap hold a fixed pattern, written once after the pool is cleared; a kernel that runs over
 * the end of its region (or under the start of the next) damages the pattern, and the check names the gap and the
 * first damaged byte. The check reads 32 KB from the device: it runs at finalize and on request (dcclDebugCheck),
 * never on the path of a collective. The original has no counterpart (it runs no device code that shares a buffer
 * between ranks, reference src/core/reduce.cu:9-38).
 *
 * The copy between host and pool goes through a function pointer so that the same code can be exercised on a host
 * buffer without a GPU.
 */
#pragma once
#include <cstddef>
#include <cstdint>

namespace dccl {

struct PoolGap { size_t lo, hi; const char* after; };

/** The gaps of the pool layout, in address order. */
int pool_gaps(const PoolGap** gaps);

constexpr size_t kGuardBytes = 4096;
constexpr uint32_t kGuardWord = 0xDCC1CA9Au;

/** dst / src: one of them is inside the pool. Returns false on failure. */
using PoolCopyFn = bool (*)(void* dst, const void* src, size_t bytes);

/** Write the guard pattern into every gap of `pool`. */
bool canary_fill(char* pool, PoolCopyFn to_pool);

/** 0 when every guard word is intact; otherwise 1 + index of the first damaged gap, with the pool offset of the
 *  first damaged byte in *bad_offset; -1 when the pool could not be read. */
int canary_check(const char* pool, PoolCopyFn from_pool, size_t* bad_offset);

/** Host <-> device copies for a real pool. */
bool canary_copy_cuda(void* dst, const void* src, size_t bytes);

} // namespace dccl
