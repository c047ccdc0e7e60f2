// base.cc -- logger, parameter loader and small utilities (see base.h).
#include "base.h"

#include <errno.h>
#include <pthread.h>
#include <stdarg.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include <map>
#include <mutex>

namespace fcx {

// ---------------------------------------------------------------------------
// parameters
// ---------------------------------------------------------------------------
static std::once_flag confOnce;
static std::map<std::string, std::string> *confValues;

static void parseConfFile(const char *path) {
  FILE *f = fopen(path, "r");
  if (!f) return;
  char line[1024];
  while (fgets(line, sizeof line, f)) {
    char *hash = strchr(line, '#');
    if (hash) *hash = 0;
    char *eq = strchr(line, '=');
    if (!eq) continue;
    *eq = 0;
    std::string k(line), v(eq + 1);
    auto trim = [](std::string &s) {
      size_t b = s.find_first_not_of(" \t\r\n");
      size_t e = s.find_last_not_of(" \t\r\n");
      s = (b == std::string::npos) ? "" : s.substr(b, e - b + 1);
    };
    trim(k);
    trim(v);
    if (!k.empty() && !confValues->count(k)) (*confValues)[k] = v;
  }
  fclose(f);
}

static void loadConf() {
  confValues = new std::map<std::string, std::string>();
  // An explicit file wins, then the per-user file, then the system-wide one.
  if (const char *p = getenv("FLAGCX_CONF_FILE")) parseConfFile(p);
  if (const char *home = getenv("HOME")) {
    std::string p = std::string(home) + "/.flagcx.conf";
    parseConfFile(p.c_str());
  }
  parseConfFile("/etc/flagcx.conf");
}

const char *getEnv(const char *name) {
  const char *v = getenv(name);
  if (v) return v;
  std::call_once(confOnce, loadConf);
  auto it = confValues->find(name);
  return it == confValues->end() ? nullptr : it->second.c_str();
}

static bool parseInt(const char *s, int64_t *out) {
  if (!s || !*s) return false;
  errno = 0;
  char *end = nullptr;
  long long v = strtoll(s, &end, 0);
  if (errno || end == s) return false;
  // size suffixes: K, M, G (powers of two)
  if (*end == 'K' || *end == 'k') v <<= 10;
  else if (*end == 'M' || *end == 'm') v <<= 20;
  else if (*end == 'G' || *end == 'g') v <<= 30;
  *out = v;
  return true;
}

int64_t loadParam(const char *name, int64_t dflt) {
  int64_t v;
  const char *s = getEnv(name);
  if (s) {
    if (parseInt(s, &v)) {
      FCX_INFO(SUB_ENV, "%s set to %lld", name, (long long)v);
      return v;
    }
    FCX_WARN("ignoring %s=%s: not an integer", name, s);
  }
  return dflt;
}

int64_t readParam(const char *envSuffix, int64_t dflt) {
  std::string n = std::string("FLAGCX_") + envSuffix;
  int64_t v;
  const char *s = getEnv(n.c_str());
  return (s && parseInt(s, &v)) ? v : dflt;
}

// ---------------------------------------------------------------------------
// logging
// ---------------------------------------------------------------------------
static int gLevel = -1;
static uint32_t gSubsys = SUB_INIT | SUB_ENV | SUB_BOOTSTRAP;
static FILE *gOut = nullptr;
static std::mutex gLogMu;
static thread_local char tlsLastError[512];
static char gHost[256];

static uint32_t subsysFromName(const std::string &n) {
  static const struct { const char *n; uint32_t v; } tbl[] = {
      {"INIT", SUB_INIT},   {"COLL", SUB_COLL},     {"P2P", SUB_P2P},
      {"SHM", SUB_SHM},     {"NET", SUB_NET},       {"GRAPH", SUB_GRAPH},
      {"TUNING", SUB_TUNING}, {"ENV", SUB_ENV},     {"ALLOC", SUB_ALLOC},
      {"CALL", SUB_CALL},   {"PROXY", SUB_PROXY},   {"NVLS", SUB_NVLS},
      {"BOOTSTRAP", SUB_BOOTSTRAP}, {"REG", SUB_REG}, {"ALL", SUB_ALL}};
  for (auto &e : tbl)
    if (strcasecmp(n.c_str(), e.n) == 0) return e.v;
  return 0;
}

void logInit() {
  std::lock_guard<std::mutex> g(gLogMu);
  if (gLevel >= 0) return;
  int lvl = LOG_NONE;
  if (const char *s = getenv("FLAGCX_DEBUG")) {
    if (!strcasecmp(s, "VERSION")) lvl = LOG_VERSION;
    else if (!strcasecmp(s, "WARN")) lvl = LOG_WARN;
    else if (!strcasecmp(s, "INFO")) lvl = LOG_INFO;
    else if (!strcasecmp(s, "ABORT")) lvl = LOG_ABORT;
    else if (!strcasecmp(s, "TRACE")) lvl = LOG_TRACE;
  }
  if (const char *s = getenv("FLAGCX_DEBUG_SUBSYS")) {
    std::string str(s);
    bool invert = !str.empty() && str[0] == '^';
    if (invert) str = str.substr(1);
    uint32_t mask = 0;
    size_t pos = 0;
    while (pos <= str.size()) {
      size_t c = str.find(',', pos);
      if (c == std::string::npos) c = str.size();
      mask |= subsysFromName(str.substr(pos, c - pos));
      pos = c + 1;
    }
    gSubsys = invert ? ~mask : mask;
  }
  gethostname(gHost, sizeof gHost - 1);
  gOut = stderr;
  if (const char *s = getenv("FLAGCX_DEBUG_FILE")) {
    std::string path;
    for (const char *p = s; *p; ++p) {
      if (*p == '%' && p[1] == 'h') { path += gHost; ++p; }
      else if (*p == '%' && p[1] == 'p') { path += std::to_string(getpid()); ++p; }
      else path += *p;
    }
    FILE *f = fopen(path.c_str(), "w");
    if (f) { setvbuf(f, nullptr, _IOLBF, 0); gOut = f; }
  }
  gLevel = lvl;
}

int logLevel() {
  if (gLevel < 0) logInit();
  return gLevel;
}

const char *lastErrorText() { return tlsLastError; }

void logWrite(LogLevel lvl, uint32_t subsys, const char *file, int line,
              const char *fmt, ...) {
  char body[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(body, sizeof body, fmt, ap);
  va_end(ap);
  if (lvl == LOG_WARN) snprintf(tlsLastError, sizeof tlsLastError, "%.*s", (int)sizeof tlsLastError - 1, body);
  int cur = logLevel();
  if (cur < (int)lvl) return;
  if (lvl != LOG_WARN && !(subsys & gSubsys)) return;
  const char *base = strrchr(file, '/');
  base = base ? base + 1 : file;
  const char *tag = lvl == LOG_WARN ? "WARN" : lvl == LOG_INFO ? "INFO" : "TRACE";
  std::lock_guard<std::mutex> g(gLogMu);
  fprintf(gOut, "%s:%d:%lx FLAGCX %s %s:%d %s\n", gHost, (int)getpid(),
          (unsigned long)pthread_self() & 0xffffff, tag, base, line, body);
  fflush(gOut);
}

// ---------------------------------------------------------------------------
// utilities
// ---------------------------------------------------------------------------
uint64_t hashBytes(const void *data, size_t n) {
  const unsigned char *p = (const unsigned char *)data;
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
  return h;
}

std::string hostName() {
  char buf[256] = {0};
  gethostname(buf, sizeof buf - 1);
  return buf;
}

uint64_t hostHash() {
  // FLAGCX_HOSTID lets one machine pose as several (same trick as the FlagCX
  // CI uses to exercise its non-P2P path on one box).
  if (const char *id = getEnv("FLAGCX_HOSTID")) return hashBytes(id, strlen(id));
  std::string s = hostName();
  FILE *f = fopen("/proc/sys/kernel/random/boot_id", "r");
  if (f) {
    char b[128] = {0};
    if (fgets(b, sizeof b, f)) s += b;
    fclose(f);
  }
  return hashBytes(s.data(), s.size());
}

uint64_t pidHash() {
  char b[64];
  int n = snprintf(b, sizeof b, "%d", (int)getpid());
  char ns[128] = {0};
  ssize_t l = readlink("/proc/self/ns/pid", ns, sizeof ns - 1);
  std::string s(b, n);
  if (l > 0) s.append(ns, l);
  return hashBytes(s.data(), s.size());
}

uint64_t nowNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
}

const char *dtypeName(flagcxDataType_t t) {
  static const char *n[] = {"int8",  "uint8", "int32",  "uint32", "int64",
                            "uint64", "half", "float", "double", "bfloat16"};
  return (int)t >= 0 && t < flagcxNumTypes ? n[t] : "?";
}
const char *redOpName(flagcxRedOp_t o) {
  static const char *n[] = {"sum", "prod", "max", "min", "avg"};
  return (int)o >= 0 && o < flagcxNumRedOps ? n[o] : "?";
}
const char *commOpName(flagcxCommOp_t o) {
  static const char *n[] = {"send", "recv", "broadcast", "gather", "scatter",
                            "reduce", "allreduce", "allgather", "reducescatter",
                            "alltoall", "alltoallv", "noop"};
  return (int)o >= 0 && o < flagcxNumCommOps ? n[o] : "?";
}

} // namespace fcx

extern "C" size_t getFlagcxDataTypeSize(flagcxDataType_t dtype) {
  switch (dtype) {
    case flagcxInt8: case flagcxUint8: return 1;
    case flagcxFloat16: case flagcxBfloat16: return 2;
    case flagcxInt32: case flagcxUint32: case flagcxFloat32: return 4;
    case flagcxInt64: case flagcxUint64: case flagcxFloat64: return 8;
    default: return 0;
  }
}
