/**
 * Timestamp log: same record layout and text format as the original
 * (reference src/core/dccl.cpp:913-991), but the buffer is allocated on first
 * use and doubles on demand up to 2^24 entries instead of claiming 512 MB when
 * the library is loaded.
 */
#include <dccl/dccl.hpp>
#include "log.hpp"
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>

namespace dccl {

static const size_t kMaxEntries = 1ull << 24;
static const size_t kFirstEntries = 1ull << 12;

Timestamp Timestamp::_t;

Timestamp::Timestamp(size_t num_entries) : _log(nullptr), capacity(0), position(0), lck(0) {
    if (num_entries) {
        _log = (uint64_t*)malloc(num_entries * 4 * sizeof(uint64_t));
        if (_log) capacity = num_entries;
    }
}

Timestamp::~Timestamp() { free(_log); _log = nullptr; capacity = position = 0; }

uint64_t Timestamp::now_ns() {
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

static inline void spin_lock(volatile int* l) { while (__sync_lock_test_and_set(l, 1)) { while (*l) __builtin_ia32_pause(); } }
static inline void spin_unlock(volatile int* l) { __sync_lock_release(l); }

void Timestamp::instance_log(uint64_t tag, uint64_t rank, uint64_t extra, uint64_t ts_ns) {
    spin_lock(&lck);
    if (position == capacity) {
        size_t ncap = capacity ? capacity * 2 : kFirstEntries;
        if (ncap > kMaxEntries) ncap = kMaxEntries;
        if (ncap > capacity) {
            uint64_t* n = (uint64_t*)realloc(_log, ncap * 4 * sizeof(uint64_t));
            if (n) { _log = n; capacity = ncap; }
        }
    }
    if (position < capacity) {
        uint64_t* e = _log + 4 * position++;
        e[0] = tag; e[1] = rank; e[2] = extra; e[3] = ts_ns;
        spin_unlock(&lck);
    } else {
        spin_unlock(&lck);
        dccl_error("timestamp log is full (%zu entries); entry with tag %llu dropped", capacity, (unsigned long long)tag);
    }
}

void Timestamp::instance_flush(const std::string& filename, bool clear) {
    spin_lock(&lck);
    FILE* f = fopen(filename.c_str(), "w");
    if (f) {
        fprintf(f, "# number of entries:%zu\n", position);
        fprintf(f, "# tag rank extra tsns\n");
        for (size_t i = 0; i < position; i++) {
            const uint64_t* e = _log + 4 * i;
            fprintf(f, "%llu %llu %llu %llu\n", (unsigned long long)e[0], (unsigned long long)e[1],
                    (unsigned long long)e[2], (unsigned long long)e[3]);
        }
        fclose(f);
    }
    if (clear) position = 0;
    spin_unlock(&lck);
    if (!f) dccl_error("cannot open timestamp file %s", filename.c_str());
}

void Timestamp::instance_clear() {
    spin_lock(&lck);
    position = 0;
    spin_unlock(&lck);
}

size_t Timestamp::instance_size() { return position; }

} // namespace dccl
