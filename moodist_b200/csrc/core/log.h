// Logging and environment flags.
//
// MOODIST_LOG_LEVEL = NONE|ERROR|INFO|VERBOSE|DEBUG or an integer 0..4; errors go to stderr, the rest
// to stdout, each line prefixed "dd-mm-YYYY HH:MM:SS.uuuuuu moodist: " — the same knobs and line
// format as the reference (core/logging.h:30-116).
#pragma once

#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <ctime>
#include <stdexcept>
#include <string>

namespace moodist {

enum LogLevel : int { LOG_NONE = 0, LOG_ERROR = 1, LOG_INFO = 2, LOG_VERBOSE = 3, LOG_DEBUG = 4 };

inline int parse_log_level(const char* s, int dflt) {
  if (!s || !*s) return dflt;
  if (!strcasecmp(s, "NONE")) return LOG_NONE;
  if (!strcasecmp(s, "ERROR")) return LOG_ERROR;
  if (!strcasecmp(s, "INFO")) return LOG_INFO;
  if (!strcasecmp(s, "VERBOSE")) return LOG_VERBOSE;
  if (!strcasecmp(s, "DEBUG")) return LOG_DEBUG;
  char* e = nullptr;
  long v = strtol(s, &e, 10);
  if (e && *e == 0) return (int)v;
  return dflt;
}

inline int& log_level() {
  static int lvl = parse_log_level(getenv("MOODIST_LOG_LEVEL"), LOG_ERROR);
  return lvl;
}

inline void log_line(int level, const char* fmt, va_list ap) {
  if (level > log_level()) return;
  char msg[4096];
  vsnprintf(msg, sizeof(msg), fmt, ap);
  auto now = std::chrono::system_clock::now();
  time_t t = std::chrono::system_clock::to_time_t(now);
  long us = (long)(std::chrono::duration_cast<std::chrono::microseconds>(now.time_since_epoch()).count() % 1000000);
  struct tm tmv;
  localtime_r(&t, &tmv);
  char ts[64];
  strftime(ts, sizeof(ts), "%d-%m-%Y %H:%M:%S", &tmv);
  FILE* f = level == LOG_ERROR ? stderr : stdout;
  size_t n = strlen(msg);
  fprintf(f, "%s.%06ld moodist: %s%s", ts, us, msg, (n && msg[n - 1] == '\n') ? "" : "\n");
  fflush(f);
}

#define MOODIST_DEFINE_LOG(name, level)                                \
  inline void name(const char* fmt, ...) __attribute__((format(printf, 1, 2))); \
  inline void name(const char* fmt, ...) {                              \
    if (level > log_level()) return;                                    \
    va_list ap;                                                         \
    va_start(ap, fmt);                                                  \
    log_line(level, fmt, ap);                                           \
    va_end(ap);                                                         \
  }
MOODIST_DEFINE_LOG(log_error, LOG_ERROR)
MOODIST_DEFINE_LOG(log_info, LOG_INFO)
MOODIST_DEFINE_LOG(log_verbose, LOG_VERBOSE)
MOODIST_DEFINE_LOG(log_debug, LOG_DEBUG)

inline std::string strf(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
inline std::string strf(const char* fmt, ...) {
  va_list ap, ap2;
  va_start(ap, fmt);
  va_copy(ap2, ap);
  int n = vsnprintf(nullptr, 0, fmt, ap);
  va_end(ap);
  std::string s(n > 0 ? n : 0, '\0');
  if (n > 0) vsnprintf(s.data(), n + 1, fmt, ap2);
  va_end(ap2);
  return s;
}

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
[[noreturn]] inline void fail(const std::string& msg) { throw Error(msg); }

inline long env_long(const char* name, long dflt) {
  const char* s = getenv(name);
  if (!s || !*s) return dflt;
  char* e = nullptr;
  long v = strtol(s, &e, 10);
  return (e && e != s) ? v : dflt;
}
inline bool env_flag(const char* name) { return env_long(name, 0) != 0; }

inline double now_seconds() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Called by long waits of caller threads between slices, with none of the library's locks held. The Python
// bindings install a function that lets pending signal handlers run (and throws when one of them raised, e.g.
// KeyboardInterrupt), so that Ctrl-C ends a collective that will never complete. Set once, before any wait.
inline std::function<void()>& interrupt_hook() {
  static std::function<void()> hook;
  return hook;
}
inline void check_interrupt() {
  auto& hook = interrupt_hook();
  if (hook) hook();
}

// How long (microseconds) a thread looks at a completion flag, and the engine thread keeps polling after its last
// activity, before it blocks. MOODIST_SPIN_US overrides; 0 blocks at once.
inline double spin_microseconds() {
  static const double v = (double)env_long("MOODIST_SPIN_US", 100);
  return v;
}

// Polls `flag` for at most `us` microseconds; true when it was seen set.
inline bool spin_until(const std::atomic<bool>& flag, double us) {
  if (flag.load(std::memory_order_acquire)) return true;
  if (us <= 0) return false;
  const double until = now_seconds() + us * 1e-6;
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (flag.load(std::memory_order_acquire)) return true;
#if defined(__x86_64__) || defined(__i386__)
      __builtin_ia32_pause();
#elif defined(__aarch64__)
      asm volatile("yield");
#endif
    }
    if (now_seconds() >= until) return false;
  }
}

}  // namespace moodist
