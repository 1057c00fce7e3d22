#include "log.hpp"
#include "config.hpp"
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <strings.h>
#include <unistd.h>

namespace dccl {

static std::atomic<int> g_level{-1};
static std::atomic<int> g_rank{-1};

LogLevel parse_log_level(const char* s, LogLevel dflt) {
    static const char* names[] = {"trace", "debug", "info", "warn", "error", "critical", "off"};
    if (!s) return dflt;
    for (int i = 0; i <= LOG_OFF; i++) if (!strcasecmp(s, names[i])) return (LogLevel)i;
    if (!strcasecmp(s, "warning")) return LOG_WARN;
    if (!strcasecmp(s, "err")) return LOG_ERROR;
    return dflt;
}

LogLevel log_level() {
    int l = g_level.load(std::memory_order_relaxed);
    if (l >= 0) return (LogLevel)l;
    // first use: environment beats the configuration file
    LogLevel lv = LOG_WARN;
    const char* e = getenv("DCCL_LOG_LEVEL");
    if (e) lv = parse_log_level(e, LOG_WARN);
    else {
        std::string v;
        if (Config::global().get("LOGGER/default_log_level", &v)) lv = parse_log_level(v.c_str(), LOG_WARN);
    }
    int expect = -1;
    g_level.compare_exchange_strong(expect, (int)lv);
    return (LogLevel)g_level.load();
}

void set_log_level(LogLevel l) { g_level.store((int)l); }
void log_set_rank(int rank) { g_rank.store(rank); }

void log_write(LogLevel l, const char* fmt, ...) {
    static const char* tags[] = {"trace", "debug", "info", "warning", "error", "critical", "off"};
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    struct tm tmv;
    localtime_r(&ts.tv_sec, &tmv);
    char line[1200];
    int n = snprintf(line, sizeof(line), "[%02d:%02d:%02d.%06ld] [DCCL] [r%d p%d] [%s] %s\n",
                     tmv.tm_hour, tmv.tm_min, tmv.tm_sec, ts.tv_nsec / 1000, g_rank.load(), (int)getpid(),
                     tags[(int)l], buf);
    if (n > 0) fwrite(line, 1, (size_t)(n < (int)sizeof(line) ? n : (int)sizeof(line) - 1), stderr);
}

} // namespace dccl
