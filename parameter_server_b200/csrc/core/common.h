// Basic types, logging and check macros of the host runtime.
// Counterpart of util/common.h:50-96, util/macros.h:5-13 in the reference.
#pragma once
#include <atomic>
#include <cassert>
#include <chrono>
#include <cinttypes>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <iostream>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <utility>
#include <vector>

namespace PS {

typedef uint64_t Key;
typedef std::string NodeID;
static const Key kMaxKey = UINT64_MAX;  // exclusive end of the key space

typedef std::lock_guard<std::mutex> Lock;
typedef std::unique_lock<std::mutex> ULock;

#define PS_DISALLOW_COPY(T) \
  T(const T&) = delete;     \
  void operator=(const T&) = delete

// A failed CHECK throws; callers (tests, Python) see an exception instead of an abort.
class CheckError : public std::runtime_error {
 public:
  explicit CheckError(const std::string& m) : std::runtime_error(m) {}
};

class CheckStream {
 public:
  CheckStream(const char* file, int line, const char* cond) {
    ss_ << file << ":" << line << " check failed: " << cond << " ";
  }
  template <typename T>
  CheckStream& operator<<(const T& v) { ss_ << v; return *this; }
  [[noreturn]] ~CheckStream() noexcept(false) { throw CheckError(ss_.str()); }
 private:
  std::ostringstream ss_;
};

#define PS_CHECK(c) if (!(c)) ::PS::CheckStream(__FILE__, __LINE__, #c)
#define PS_CHECK_EQ(a, b) PS_CHECK((a) == (b)) << "(" << (a) << " vs " << (b) << ") "
#define PS_CHECK_NE(a, b) PS_CHECK((a) != (b))
#define PS_CHECK_LT(a, b) PS_CHECK((a) < (b)) << "(" << (a) << " vs " << (b) << ") "
#define PS_CHECK_LE(a, b) PS_CHECK((a) <= (b)) << "(" << (a) << " vs " << (b) << ") "
#define PS_CHECK_GT(a, b) PS_CHECK((a) > (b)) << "(" << (a) << " vs " << (b) << ") "
#define PS_CHECK_GE(a, b) PS_CHECK((a) >= (b)) << "(" << (a) << " vs " << (b) << ") "

// Leveled logging to stderr; PSB_VLOG=<n> enables verbose levels.
inline int VerboseLevel() {
  static int v = [] { const char* e = getenv("PSB_VLOG"); return e ? atoi(e) : 0; }();
  return v;
}
class LogLine {
 public:
  LogLine(const char* tag, bool on) : on_(on) { if (on_) ss_ << "[" << tag << "] "; }
  template <typename T>
  LogLine& operator<<(const T& v) { if (on_) ss_ << v; return *this; }
  ~LogLine() {
    if (on_) { ss_ << "\n"; std::string s = ss_.str(); fwrite(s.data(), 1, s.size(), stderr); }
  }
 private:
  bool on_;
  std::ostringstream ss_;
};
#define PS_LOG(tag) ::PS::LogLine(#tag, true)
#define PS_VLOG(n) ::PS::LogLine("V" #n, ::PS::VerboseLevel() >= (n))
#define PS_NOTICE(...) do { fprintf(stdout, __VA_ARGS__); fprintf(stdout, "\n"); fflush(stdout); } while (0)

inline double NowSeconds() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace PS
