#include "log.h"

#include <execinfo.h>
#include <sched.h>
#include <signal.h>
#include <unistd.h>

#include <string>

#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <sstream>

#include "env.h"

namespace bshmem {

static int g_level = LOG_NONE;
static uint32_t g_mask = SUB_ALL;
static FILE* g_out = nullptr;
static int g_dev = -1;
static int g_pe = -1;
static char g_host[256] = "";
static std::mutex g_mu;

static std::string upper(std::string s) {
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return toupper(c); });
  return s;
}

uint32_t log_parse_subsys(const std::string& text_in) {
  std::string text = upper(text_in);
  if (text.empty()) return SUB_ALL;
  bool invert = text[0] == '^';
  if (invert) text = text.substr(1);
  static const struct { const char* name; uint32_t bit; } names[] = {
      {"INIT", SUB_INIT}, {"COLL", SUB_COLL}, {"P2P", SUB_P2P}, {"PROXY", SUB_PROXY},
      {"TRANSPORT", SUB_TRANSPORT}, {"MEM", SUB_MEM}, {"BOOTSTRAP", SUB_BOOTSTRAP},
      {"TOPO", SUB_TOPO}, {"UTIL", SUB_UTIL}, {"TEAM", SUB_TEAM}, {"ALL", SUB_ALL}};
  uint32_t mask = 0;
  std::stringstream ss(text);
  std::string tok;
  while (std::getline(ss, tok, ',')) {
    for (auto& n : names)
      if (tok == n.name) mask |= n.bit;
  }
  return invert ? ~mask : mask;
}

std::string log_expand_filename(const std::string& pattern) {
  std::string out;
  char host[256] = "unknown";
  gethostname(host, sizeof(host) - 1);
  for (size_t i = 0; i < pattern.size(); ++i) {
    if (pattern[i] == '%' && i + 1 < pattern.size()) {
      char c = pattern[++i];
      if (c == 'h') out += host;
      else if (c == 'p') out += std::to_string((long)getpid());
      else { out.push_back('%'); out.push_back(c); }
    } else {
      out.push_back(pattern[i]);
    }
  }
  return out;
}

void log_init() {
  std::lock_guard<std::mutex> lk(g_mu);
  const Options& o = options();
  std::string lvl = upper(o.DEBUG);
  if (lvl == "VERSION") g_level = LOG_VERSION;
  else if (lvl == "WARN") g_level = LOG_WARN;
  else if (lvl == "INFO") g_level = LOG_INFO;
  else if (lvl == "ABORT") g_level = LOG_ABORT;
  else if (lvl == "TRACE") g_level = LOG_TRACE;
  else g_level = LOG_NONE;
  g_mask = log_parse_subsys(o.DEBUG_SUBSYS);
  if (g_out && g_out != stdout && g_out != stderr) fclose(g_out);
  g_out = nullptr;
  if (!o.DEBUG_FILE.empty()) {
    g_out = fopen(log_expand_filename(o.DEBUG_FILE).c_str(), "w");
    if (g_out) setvbuf(g_out, nullptr, _IOLBF, 0);
  }
  gethostname(g_host, sizeof(g_host) - 1);
}

void log_set_device(int dev) { g_dev = dev; }
void log_set_pe(int pe) { g_pe = pe; }
int log_level() { return g_level; }
uint32_t log_mask() { return g_mask; }

bool log_enabled(LogLevel lvl, uint32_t subsys) {
  if (lvl == LOG_NONE) return true;
  return g_level >= (int)lvl && (g_mask & subsys) != 0;
}

void log_write(LogLevel lvl, uint32_t, const char* file, int line, const char* fmt, ...) {
  char body[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(body, sizeof(body), fmt, ap);
  va_end(ap);
  const char* tag = lvl == LOG_NONE ? "ERROR" : lvl == LOG_WARN ? "WARN" : lvl == LOG_TRACE ? "TRACE" : "INFO";
  const char* base = strrchr(file, '/');
  base = base ? base + 1 : file;
  if (!g_host[0]) gethostname(g_host, sizeof(g_host) - 1);
  FILE* out = g_out ? g_out : (lvl == LOG_NONE || lvl == LOG_WARN ? stderr : stdout);
  std::lock_guard<std::mutex> lk(g_mu);
  if (lvl == LOG_NONE || lvl == LOG_WARN || lvl == LOG_TRACE)
    fprintf(out, "%s:%d:%ld [%d] NVSHMEM %s %s:%d %s\n", g_host, (int)getpid(), (long)syscall(SYS_gettid), g_dev, tag, base, line, body);
  else
    fprintf(out, "%s:%d:%ld [%d] NVSHMEM %s %s\n", g_host, (int)getpid(), (long)syscall(SYS_gettid), g_dev, tag, body);
  fflush(out);
}

static void segv_backtrace(int sig) {
  void* frames[64];
  const int n = backtrace(frames, 64);
  const char msg[] = "bshmem: caught SIGSEGV, backtrace follows\n";
  ssize_t ignored = write(STDERR_FILENO, msg, sizeof(msg) - 1);
  (void)ignored;
  backtrace_symbols_fd(frames, n, STDERR_FILENO);
  signal(sig, SIG_DFL);  // the default action (core dump / termination) happens on return
  raise(sig);
}

void log_process_diagnostics() {
  if (log_level() < LOG_INFO) return;
  cpu_set_t set;
  CPU_ZERO(&set);
  if (sched_getaffinity(0, sizeof(set), &set) == 0) {
    std::string list;
    int run_start = -1;
    for (int c = 0; c <= CPU_SETSIZE; ++c) {
      const bool on = c < CPU_SETSIZE && CPU_ISSET(c, &set);
      if (on && run_start < 0) run_start = c;
      if (!on && run_start >= 0) {
        if (!list.empty()) list += ",";
        list += std::to_string(run_start);
        if (c - 1 > run_start) list += "-" + std::to_string(c - 1);
        run_start = -1;
      }
    }
    INFO(SUB_INIT, "process %d may run on CPUs %s", (int)getpid(), list.c_str());
  }
  static bool installed = false;
  if (!installed) {
    installed = true;
    struct sigaction old {};
    if (sigaction(SIGSEGV, nullptr, &old) == 0 && old.sa_handler == SIG_DFL) signal(SIGSEGV, segv_backtrace);  // never replaces a handler the program set
  }
}

}  // namespace bshmem
