#include "env.h"

#include <cctype>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>

namespace bshmem {

bool parse_size(const char* text, size_t* out) {
  if (!text || !*text) return false;
  char* end = nullptr;
  double v = strtod(text, &end);
  if (end == text || v < 0 || std::signbit(v) || std::isnan(v)) return false;  // "-0" is a negative number too
  while (*end == ' ') ++end;
  double mult = 1;
  switch (*end) {
    case 0: break;
    case 'k': case 'K': mult = 1024.0; break;
    case 'm': case 'M': mult = 1024.0 * 1024; break;
    case 'g': case 'G': mult = 1024.0 * 1024 * 1024; break;
    case 't': case 'T': mult = 1024.0 * 1024 * 1024 * 1024; break;
    default: return false;
  }
  // Characters after the multiplier are ignored ("20kk" == "20k", "20KiB" == "20k"), as the reference's parser does.
  const double bytes = std::ceil(v * mult);
  if (!std::isfinite(bytes) || bytes >= 18446744073709551616.0) return false;  // does not fit 64 bits
  *out = (size_t)bytes;
  return true;
}

bool parse_bool(const char* text, bool* out) {
  if (!text) return false;
  std::string s;
  for (const char* p = text; *p; ++p) s.push_back((char)tolower(*p));
  // An empty value counts as "set": `NVSHMEM_INFO= prog` switches the flag on.
  if (s.empty() || s == "1" || s == "y" || s == "yes" || s == "on" || s == "true" || s == "t") {
    *out = true;
    return true;
  }
  if (s == "0" || s == "n" || s == "no" || s == "off" || s == "false" || s == "f") {
    *out = false;
    return true;
  }
  return false;
}

namespace {
bool assign(bool* dst, const char* v) { return parse_bool(v, dst); }
bool assign(long* dst, const char* v) {
  char* end = nullptr;
  long r = strtol(v, &end, 0);
  if (end == v || *end) return false;
  *dst = r;
  return true;
}
bool assign(size_t* dst, const char* v) { return parse_size(v, dst); }
bool assign(std::string* dst, const char* v) {
  *dst = v;
  return true;
}
std::string show(bool v) { return v ? "true" : "false"; }
std::string show(long v) { return std::to_string(v); }
std::string show(size_t v) { return std::to_string(v); }
std::string show(const std::string& v) { return "\"" + v + "\""; }
std::string show(const char* v) { return std::string("\"") + v + "\""; }
}  // namespace

int options_init(Options* o, std::vector<std::string>* errors) {
  int bad = 0;
#define X(name, ctype, kind, dflt, cat, help)                             \
  {                                                                       \
    o->name = (ctype)dflt;                                                \
    o->name##_set = false;                                                \
    const char* v = getenv("NVSHMEM_" #name);                             \
    if (v) {                                                              \
      if (assign(&o->name, v)) {                                          \
        o->name##_set = true;                                             \
      } else {                                                            \
        ++bad;                                                            \
        if (errors) errors->push_back(std::string("NVSHMEM_" #name "=") + v); \
      }                                                                   \
    }                                                                     \
  }
  BSHMEM_OPTIONS(X)
#undef X
  return bad;
}

std::vector<OptionInfo> options_describe(const Options& o) {
  std::vector<OptionInfo> out;
#define X(name, ctype, kind, dflt, cat, help) \
  out.push_back(OptionInfo{"NVSHMEM_" #name, OptKind::kind, OptCat::cat, help, show((ctype)dflt), show(o.name), o.name##_set});
  BSHMEM_OPTIONS(X)
#undef X
  return out;
}

static Options g_opts;
static std::once_flag g_once;
static std::mutex g_mu;

const Options& options() {
  std::call_once(g_once, [] { options_init(&g_opts); });
  return g_opts;
}

void options_reload() {
  options();
  std::lock_guard<std::mutex> lk(g_mu);
  options_init(&g_opts);
}

}  // namespace bshmem
