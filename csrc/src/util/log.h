// Levelled, subsystem-masked logging driven by NVSHMEM_DEBUG,
// NVSHMEM_DEBUG_SUBSYS and NVSHMEM_DEBUG_FILE, with the line format
// "host:pid:tid [dev] NVSHMEM LEVEL text"
// (reference: src/include/internal/host/debug.h, src/host/util/debug.cpp).
#pragma once
#include <cstdarg>
#include <cstdint>
#include <string>

namespace bshmem {

enum LogLevel { LOG_NONE = 0, LOG_VERSION = 1, LOG_WARN = 2, LOG_INFO = 3, LOG_ABORT = 4, LOG_TRACE = 5 };

enum LogSubsys : uint32_t {
  SUB_INIT = 1u << 0,
  SUB_COLL = 1u << 1,
  SUB_P2P = 1u << 2,
  SUB_PROXY = 1u << 3,
  SUB_TRANSPORT = 1u << 4,
  SUB_MEM = 1u << 5,
  SUB_BOOTSTRAP = 1u << 6,
  SUB_TOPO = 1u << 7,
  SUB_UTIL = 1u << 8,
  SUB_TEAM = 1u << 9,
  SUB_ALL = 0xffffffffu,
};

void log_init();                    // (re)reads the environment
void log_set_device(int dev);       // shown in the [dev] field
void log_set_pe(int pe);
// With NVSHMEM_DEBUG at INFO or above: prints the CPUs this process may run on, and installs a SIGSEGV handler
// that writes a backtrace to stderr before the default action takes over (reference: src/host/util/util.cpp:25-38,166).
void log_process_diagnostics();
int log_level();
uint32_t log_mask();
bool log_enabled(LogLevel lvl, uint32_t subsys);
void log_write(LogLevel lvl, uint32_t subsys, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 5, 6)));
// Parses "INIT,COLL" or "^MEM" into a mask (exposed for tests).
uint32_t log_parse_subsys(const std::string& text);
std::string log_expand_filename(const std::string& pattern);  // %h, %p

}  // namespace bshmem

#define BSHMEM_LOG(lvl, sub, ...)                                              \
  do {                                                                         \
    if (::bshmem::log_enabled(lvl, sub)) ::bshmem::log_write(lvl, sub, __FILE__, __LINE__, __VA_ARGS__); \
  } while (0)
#define INFO(sub, ...) BSHMEM_LOG(::bshmem::LOG_INFO, sub, __VA_ARGS__)
#define WARN(...) BSHMEM_LOG(::bshmem::LOG_WARN, ::bshmem::SUB_ALL, __VA_ARGS__)
#define TRACE(sub, ...) BSHMEM_LOG(::bshmem::LOG_TRACE, sub, __VA_ARGS__)
// Errors are always printed; callers return a status instead of exiting.
#define ERROR_PRINT(...) ::bshmem::log_write(::bshmem::LOG_NONE, ::bshmem::SUB_ALL, __FILE__, __LINE__, __VA_ARGS__)
