/**
 * Guard words between the regions of a symmetric pool; see canary.hpp.
 */
#include "canary.hpp"
#include "../device/prims.cuh"
#include <cstdlib>
#include <cstring>
#include <vector>

namespace dccl {

namespace {

constexpr size_t kFlagEnd = kFlagOff + (size_t)kMaxCtas * kMaxPeers * sizeof(uint32_t);
constexpr size_t kP2pFlagEnd = kP2pFlagOff + 2 * (size_t)kMaxPeers * kP2pDepth * kP2pCtas * sizeof(unsigned long long);
// rendezvous words of large send / recv: a 64-byte post per (rank, slot), then path, done and arrival words
constexpr size_t kP2pRdvEnd = kP2pRdvOff + (size_t)kMaxPeers * kP2pRdvSlots * (64 + 3 * sizeof(unsigned long long));
constexpr size_t kLLEnd = kLLOff + kLLBytes;
constexpr size_t kP2pEnd = kP2pOff + (size_t)kMaxPeers * kP2pBytesPerSrc;
constexpr size_t kLL2End = kLL2Off + 2 * (size_t)kMaxPeers * 2 * kLL2PhaseBytes;

const PoolGap g_gaps[] = {
    {kFlagEnd, kP2pFlagOff, "the flag rows"},
    {kP2pRdvEnd, kLLOff, "the send/recv credit and rendezvous words"},
    {kLLEnd, kP2pOff, "the packet region"},
    {kLL2End, kStageOff, "the second packet region"},
};
constexpr int kGaps = (int)(sizeof(g_gaps) / sizeof(g_gaps[0]));

static_assert(kFlagEnd + 2 * kGuardBytes <= kP2pFlagOff, "no room for guard words after the flag rows");
static_assert(kP2pFlagEnd <= kP2pRdvOff, "the credit words overlap the rendezvous words");
static_assert(kP2pRdvEnd + 2 * kGuardBytes <= kLLOff, "no room for guard words after the rendezvous words");
static_assert(kLLEnd + 2 * kGuardBytes <= kP2pOff, "no room for guard words after the packet region");
static_assert(kP2pEnd == kLL2Off, "the FIFOs are expected to end where the second packet region starts");
static_assert(kLL2End + 2 * kGuardBytes <= kStageOff, "no room for guard words after the second packet region");

} // namespace

int pool_gaps(const PoolGap** gaps) {
    if (gaps) *gaps = g_gaps;
    return kGaps;
}

bool canary_fill(char* pool, PoolCopyFn to_pool) {
    std::vector<uint32_t> pattern(kGuardBytes / sizeof(uint32_t), kGuardWord);
    for (int i = 0; i < kGaps; i++) {
        if (!to_pool(pool + g_gaps[i].lo, pattern.data(), kGuardBytes)) return false;
        if (!to_pool(pool + g_gaps[i].hi - kGuardBytes, pattern.data(), kGuardBytes)) return false;
    }
    return true;
}

int canary_check(const char* pool, PoolCopyFn from_pool, size_t* bad_offset) {
    std::vector<uint32_t> got(kGuardBytes / sizeof(uint32_t));
    for (int i = 0; i < kGaps; i++)
        for (int side = 0; side < 2; side++) {
            const size_t off = side == 0 ? g_gaps[i].lo : g_gaps[i].hi - kGuardBytes;
            if (!from_pool(got.data(), pool + off, kGuardBytes)) return -1;
            const unsigned char* b = reinterpret_cast<const unsigned char*>(got.data());
            for (size_t k = 0; k < kGuardBytes; k++) {
                const unsigned char want = (unsigned char)(kGuardWord >> (8 * (k & 3)));
                if (b[k] != want) {
                    if (bad_offset) *bad_offset = off + k;
                    return 1 + i;
                }
            }
        }
    return 0;
}

bool canary_copy_cuda(void* dst, const void* src, size_t bytes) {
    return cudaMemcpy(dst, src, bytes, cudaMemcpyDefault) == cudaSuccess;
}

} // namespace dccl

namespace {
bool copy_host(void* dst, const void* src, size_t bytes) { memcpy(dst, src, bytes); return true; }
}

extern "C" {

/** 1 when the device code of this library was compiled with its range checks (make BOUNDS=1). */
int dccl_debug_bounds_build() {
#ifdef DCCL_DEBUG_BOUNDS
    return 1;
#else
    return 0;
#endif
}

/**
 * Self-test of the guard words on a host buffer laid out like a pool (no GPU needed): fill, check (intact), then
 * damage one byte just after each region in turn and one just before the staging area, and check that the
 * report names the right gap and byte. Returns 0, or the number of the step that failed.
 */
int dccl_selftest_canary() {
    using namespace dccl;
    char* pool = static_cast<char*>(calloc(1, kStageOff));   // untouched pages cost nothing
    if (!pool) return 1;
    int rc = 0;
    size_t bad = 0;
    const PoolGap* gaps = nullptr;
    const int n = pool_gaps(&gaps);
    if (!canary_fill(pool, copy_host)) rc = 2;
    else if (canary_check(pool, copy_host, &bad) != 0) rc = 3;
    for (int i = 0; i < n && rc == 0; i++) {
        const char saved = pool[gaps[i].lo];
        pool[gaps[i].lo] = (char)(saved ^ 0x40);                 // the byte right after a region
        if (canary_check(pool, copy_host, &bad) != 1 + i || bad != gaps[i].lo) rc = 10 + i;
        pool[gaps[i].lo] = saved;
        if (rc == 0 && canary_check(pool, copy_host, &bad) != 0) rc = 20 + i;
    }
    if (rc == 0) {
        pool[kStageOff - 1] ^= 0x01;                            // the byte right before the staging area
        if (canary_check(pool, copy_host, &bad) != n || bad != kStageOff - 1) rc = 30;
    }
    // writes inside the regions never disturb the guards
    if (rc == 0) {
        pool[kStageOff - 1] ^= 0x01;
        memset(pool + kLLOff, 0x5a, kLLBytes);
        memset(pool + kP2pOff, 0x5a, (size_t)kMaxPeers * kP2pBytesPerSrc);
        memset(pool + kLL2Off, 0x5a, 2 * (size_t)kMaxPeers * 2 * kLL2PhaseBytes);
        memset(pool, 0x5a, (size_t)kMaxCtas * kMaxPeers * sizeof(uint32_t));
        if (canary_check(pool, copy_host, &bad) != 0) rc = 40;
    }
    free(pool);
    return rc;
}

} // extern "C"
