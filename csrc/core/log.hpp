/**
 * Small leveled logger. Level names are the ones the original takes from its
 * configuration file (trace|debug|info|warn|error|critical|off; reference
 * src/core/internal_common.cpp:94-118, internal_common.hpp:36-46).
 * Level comes from DCCL_LOG_LEVEL, else the [LOGGER] default_log_level key of
 * the configuration file, else "warn".
 */
#pragma once
#include <cstdarg>

namespace dccl {

enum LogLevel { LOG_TRACE = 0, LOG_DEBUG, LOG_INFO, LOG_WARN, LOG_ERROR, LOG_CRITICAL, LOG_OFF };

LogLevel log_level();
void set_log_level(LogLevel l);
LogLevel parse_log_level(const char* s, LogLevel dflt);
void log_set_rank(int rank);
void log_write(LogLevel l, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define dccl_log(l, ...)  do { if ((l) >= ::dccl::log_level()) ::dccl::log_write((l), __VA_ARGS__); } while (0)
#define dccl_trace(...) dccl_log(::dccl::LOG_TRACE, __VA_ARGS__)
#define dccl_debug(...) dccl_log(::dccl::LOG_DEBUG, __VA_ARGS__)
#define dccl_info(...)  dccl_log(::dccl::LOG_INFO, __VA_ARGS__)
#define dccl_warn(...)  dccl_log(::dccl::LOG_WARN, __VA_ARGS__)
#define dccl_error(...) dccl_log(::dccl::LOG_ERROR, __VA_ARGS__)
#define dccl_crit(...)  dccl_log(::dccl::LOG_CRITICAL, __VA_ARGS__)

} // namespace dccl
