// Levelled logging and contract checks for the native code.
//
//   BZ_TRACE / BZ_DEBUG / BZ_INFO / BZ_WARN / BZ_ERROR / BZ_FATAL (printf-style)  ->  "[  12.345678] LEVEL file:line msg"
//   LOG_LEVEL=trace|debug|info|warn|error|fatal in the environment picks the threshold (default info);
//   BLITZ_LOG_FILE redirects the stream (default stderr), which is how one log per rank is produced.
//   Precondition / Postcondition / Invariant / Assertion(expr) throw blitz::ContractViolation with file:line and the
//   expression text; they compile to nothing under -DBLITZ_NO_CONTRACTS.
// Counterpart of the reference's logger and assertion macros (src/include/logger.h, src/include/assertion.h).
#pragma once
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

namespace blitz::log {

enum Level : int { kTrace = 0, kDebug, kInfo, kWarn, kError, kFatal };

inline Level parse_level(const char* s) {
  if (!s) return kInfo;
  static const char* names[] = {"trace", "debug", "info", "warn", "error", "fatal"};
  for (int i = 0; i < 6; ++i)
    if (strcasecmp(s, names[i]) == 0) return static_cast<Level>(i);
  return kInfo;
}

struct State {
  Level threshold = parse_level(std::getenv("LOG_LEVEL"));
  FILE* out = nullptr;
  std::mutex mu;
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  State() {
    const char* f = std::getenv("BLITZ_LOG_FILE");
    out = (f && *f) ? std::fopen(f, "a") : nullptr;
    if (!out) out = stderr;
  }
};

inline State& state() {
  static State s;
  return s;
}

inline void set_threshold(Level l) { state().threshold = l; }
inline bool enabled(Level l) { return l >= state().threshold; }

inline std::string format_line(Level l, const char* file, int line, const char* fmt, va_list ap) {
  static const char* tag[] = {"TRACE", "DEBUG", "INFO ", "WARN ", "ERROR", "FATAL"};
  char msg[2048];
  std::vsnprintf(msg, sizeof msg, fmt, ap);
  const char* base = std::strrchr(file, '/');
  const double t = std::chrono::duration<double>(std::chrono::steady_clock::now() - state().t0).count();
  char head[256];
  std::snprintf(head, sizeof head, "[%11.6f] %s %s:%d ", t, tag[l], base ? base + 1 : file, line);
  return std::string(head) + msg;
}

inline void emit(Level l, const char* file, int line, const char* fmt, ...) {
  if (!enabled(l)) return;
  va_list ap;
  va_start(ap, fmt);
  const std::string s = format_line(l, file, line, fmt, ap);
  va_end(ap);
  State& st = state();
  std::lock_guard<std::mutex> g(st.mu);
  std::fprintf(st.out, "%s\n", s.c_str());
  if (l >= kWarn) std::fflush(st.out);
}

}  // namespace blitz::log

#define BZ_LOG_AT(level, ...) ::blitz::log::emit(level, __FILE__, __LINE__, __VA_ARGS__)
#define BZ_TRACE(...) BZ_LOG_AT(::blitz::log::kTrace, __VA_ARGS__)
#define BZ_DEBUG(...) BZ_LOG_AT(::blitz::log::kDebug, __VA_ARGS__)
#define BZ_INFO(...) BZ_LOG_AT(::blitz::log::kInfo, __VA_ARGS__)
#define BZ_WARN(...) BZ_LOG_AT(::blitz::log::kWarn, __VA_ARGS__)
#define BZ_ERROR(...) BZ_LOG_AT(::blitz::log::kError, __VA_ARGS__)
#define BZ_FATAL(...) BZ_LOG_AT(::blitz::log::kFatal, __VA_ARGS__)

namespace blitz {
struct ContractViolation : std::logic_error {
  using std::logic_error::logic_error;
};
[[noreturn]] inline void contract_failed(const char* kind, const char* expr, const char* file, int line) {
  const char* base = std::strrchr(file, '/');
  const std::string msg = std::string(kind) + " failed: " + expr + " (" + (base ? base + 1 : file) + ":" + std::to_string(line) + ")";
  BZ_ERROR("%s", msg.c_str());
  throw ContractViolation(msg);
}
}  // namespace blitz

#ifdef BLITZ_NO_CONTRACTS
#define BZ_CONTRACT(kind, expr) ((void)0)
#else
#define BZ_CONTRACT(kind, expr) ((expr) ? (void)0 : ::blitz::contract_failed(kind, #expr, __FILE__, __LINE__))
#endif
#define Precondition(expr) BZ_CONTRACT("precondition", expr)
#define Postcondition(expr) BZ_CONTRACT("postcondition", expr)
#define Invariant(expr) BZ_CONTRACT("invariant", expr)
#define Assertion(expr) BZ_CONTRACT("assertion", expr)
