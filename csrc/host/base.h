// base.h -- logging, environment parameters, error-propagation macros and
// small utilities shared by every host source file.
//
// Same operator contract as the FlagCX service layer (flagcx/service/debug.cc,
// flagcx/service/param.cc in the FlagCX project): FLAGCX_DEBUG picks the level,
// FLAGCX_DEBUG_SUBSYS the subsystems ("^" inverts), FLAGCX_DEBUG_FILE redirects
// (%h host, %p pid); integer knobs are read once through FLAGCX_PARAM and may
// also come from ~/.flagcx.conf or /etc/flagcx.conf.
#pragma once
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>

#include "flagcx.h"

namespace fcx {

// ---- logging ---------------------------------------------------------------
enum LogLevel { LOG_NONE = 0, LOG_VERSION, LOG_WARN, LOG_INFO, LOG_ABORT, LOG_TRACE };
enum LogSubsys : uint32_t {
  SUB_INIT = 1u << 0,
  SUB_COLL = 1u << 1,
  SUB_P2P = 1u << 2,
  SUB_SHM = 1u << 3,
  SUB_NET = 1u << 4,
  SUB_GRAPH = 1u << 5,
  SUB_TUNING = 1u << 6,
  SUB_ENV = 1u << 7,
  SUB_ALLOC = 1u << 8,
  SUB_CALL = 1u << 9,
  SUB_PROXY = 1u << 10,
  SUB_NVLS = 1u << 11,
  SUB_BOOTSTRAP = 1u << 12,
  SUB_REG = 1u << 13,
  SUB_ALL = 0xffffffffu
};

void logInit();
int logLevel();
void logWrite(LogLevel lvl, uint32_t subsys, const char *file, int line,
              const char *fmt, ...) __attribute__((format(printf, 5, 6)));
// The most recent WARN text of this thread (flagcxGetLastError).
const char *lastErrorText();

#define FCX_WARN(...)                                                          \
  ::fcx::logWrite(::fcx::LOG_WARN, ::fcx::SUB_ALL, __FILE__, __LINE__,         \
                  __VA_ARGS__)
#define FCX_INFO(SUB, ...)                                                     \
  do {                                                                         \
    if (::fcx::logLevel() >= ::fcx::LOG_INFO)                                  \
      ::fcx::logWrite(::fcx::LOG_INFO, (SUB), __FILE__, __LINE__,              \
                      __VA_ARGS__);                                            \
  } while (0)
#define FCX_TRACE(SUB, ...)                                                    \
  do {                                                                         \
    if (::fcx::logLevel() >= ::fcx::LOG_TRACE)                                 \
      ::fcx::logWrite(::fcx::LOG_TRACE, (SUB), __FILE__, __LINE__,             \
                      __VA_ARGS__);                                            \
  } while (0)

// ---- parameters --------------------------------------------------------------
// Value of FLAGCX_<name> from the environment, else from a config file, else
// nullptr.  Thread safe; the config files are parsed once.
const char *getEnv(const char *name);
int64_t loadParam(const char *name, int64_t dflt);

#define FCX_PARAM(fn, env, dflt)                                               \
  static inline int64_t param##fn() {                                          \
    static int64_t v = ::fcx::loadParam("FLAGCX_" env, (dflt));                \
    return v;                                                                  \
  }

// Uncached read, for knobs that tests flip between communicators.
int64_t readParam(const char *envSuffix, int64_t dflt);

// ---- error propagation ----------------------------------------------------------
#define FCXCHECK(call)                                                         \
  do {                                                                         \
    flagcxResult_t r__ = (call);                                               \
    if (r__ != flagcxSuccess && r__ != flagcxInProgress) {                     \
      FCX_INFO(::fcx::SUB_ALL, "%s:%d -> %d", __FILE__, __LINE__, (int)r__);   \
      return r__;                                                              \
    }                                                                          \
  } while (0)

#define FCXCHECKGOTO(call, res, label)                                         \
  do {                                                                         \
    (res) = (call);                                                            \
    if ((res) != flagcxSuccess && (res) != flagcxInProgress) {                 \
      FCX_INFO(::fcx::SUB_ALL, "%s:%d -> %d", __FILE__, __LINE__, (int)(res)); \
      goto label;                                                              \
    }                                                                          \
  } while (0)

#define FCX_SYSCHECK(expr, what)                                               \
  do {                                                                         \
    if ((expr) == -1) {                                                        \
      FCX_WARN("%s failed: %s", what, strerror(errno));                        \
      return flagcxSystemError;                                                \
    }                                                                          \
  } while (0)

#define FCX_ARGCHECK(cond, ...)                                                \
  do {                                                                         \
    if (!(cond)) {                                                             \
      FCX_WARN(__VA_ARGS__);                                                   \
      return flagcxInvalidArgument;                                            \
    }                                                                          \
  } while (0)

// ---- utilities ---------------------------------------------------------------------
uint64_t hashBytes(const void *data, size_t n); // FNV-1a 64
// Identifies the machine: FLAGCX_HOSTID if set, else hostname + boot id.
uint64_t hostHash();
uint64_t pidHash();
uint64_t nowNs(); // CLOCK_MONOTONIC
std::string hostName();

static inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline size_t divUp(size_t v, size_t a) { return (v + a - 1) / a; }

const char *dtypeName(flagcxDataType_t t);
const char *redOpName(flagcxRedOp_t o);
const char *commOpName(flagcxCommOp_t o);

} // namespace fcx
