// Shared small utilities for the falcata_b200 core: logging, checks, string and
// number formatting helpers, host RNGs and the counter-based Philox generator
// that both the host oracle and the device kernels use.
//
// Parity notes (reference file paths are relative to the Falcata project):
//   logging levels / Fatal-throws semantics  : include/Falcata/utils/log.h:L79-183
//   number formatting for the text model     : include/Falcata/utils/common.h:L1253-1285
//   Philox4x32-10 keying for quantization    : src/treelearner/cuda/cuda_gradient_discretizer.cu:L228-247
#pragma once
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>
#include <algorithm>
#include <chrono>
#include <map>
#include <mutex>

#if defined(__CUDACC__)
#define FB_HD __host__ __device__
#else
#define FB_HD
#endif

namespace fb {

typedef int32_t data_size_t;
typedef float score_t;
typedef float label_t;

constexpr double kEpsilon = 1e-15;
constexpr double kZeroThreshold = 1e-35;
constexpr double kMinScore = -std::numeric_limits<double>::infinity();
constexpr double kSparseThreshold = 0.7;

enum class LogLevel : int { Fatal = -1, Warning = 0, Info = 1, Debug = 2 };

// Process-wide logger. Fatal raises std::runtime_error so that the C API can turn
// it into an error code + message instead of killing the interpreter.
class Log {
 public:
  typedef void (*Callback)(const char*);
  static int& level() { static int lv = 1; return lv; }
  static Callback& callback() { static Callback cb = nullptr; return cb; }
  static void ResetLevel(int lv) { level() = lv; }
  static void Write(LogLevel lv, const char* tag, const char* fmt, va_list ap) {
    if (static_cast<int>(lv) > level()) return;
    char buf[2048];
    vsnprintf(buf, sizeof(buf), fmt, ap);
    char line[2200];
    snprintf(line, sizeof(line), "[falcata_b200] [%s] %s\n", tag, buf);
    if (callback() != nullptr) callback()(line);
    else { fputs(line, stderr); fflush(stderr); }
  }
  static void Debug(const char* fmt, ...) { va_list ap; va_start(ap, fmt); Write(LogLevel::Debug, "Debug", fmt, ap); va_end(ap); }
  static void Info(const char* fmt, ...) { va_list ap; va_start(ap, fmt); Write(LogLevel::Info, "Info", fmt, ap); va_end(ap); }
  static void Warning(const char* fmt, ...) { va_list ap; va_start(ap, fmt); Write(LogLevel::Warning, "Warning", fmt, ap); va_end(ap); }
  [[noreturn]] static void Fatal(const char* fmt, ...) {
    char buf[2048];
    va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof(buf), fmt, ap); va_end(ap);
    throw std::runtime_error(std::string(buf));
  }
};

// Worker threads for a loop over `rows` cheap items: the whole team from 8192 rows on, else the calling thread alone.
// Every parallel region of the library runs either on the full team or on one thread: the OpenMP runtime ends the
// surplus workers whenever a region asks for a smaller team than the last one and starts new ones for the next larger
// region, which costs a hundred times the region itself when team sizes alternate (measured: 240 us against 2.5 us).
int RowThreads(long long rows);
// the team size of every parallel region that is not serial: the OpenMP thread limit
int TeamThreads();

// Debugging switches read once from the environment.
//   FALCATA_DEBUG=diag,dump,sync,canary,maxsplits=N   canary: guard words behind every region of the symmetric heap,
//     checked after every tree; diag: resolved plan, kernel geometry and a line per tree; dump: every
//     split of every tree (host and device learner alike); sync: every kernel launch is followed by a device
//     synchronisation so that an error surfaces at its launch site; maxsplits=N: trees stop after N splits (bisecting)
//   FALCATA_DEBUG_SPLITS=1   the host learner prints each split as it applies it
//   FALCATA_VERIFY=1         fast paths check themselves against the plain implementation: device binning against the
//     host bin mappers on a sample of rows, the tiled predict kernel against the general one
// Parity: src/treelearner/cuda/plan.h:L286-322 (FALCATA_DEBUG keys), tests/gates/README.md:L41-42 (FALCATA_VERIFY).
struct DebugFlags {
  bool diag = false, dump = false, sync = false, canary = false, splits = false, verify = false;
  int maxsplits = 0;
  static const DebugFlags& Get();
};

#define FB_CHECK(cond) do { if (!(cond)) ::fb::Log::Fatal("Check failed: " #cond " at %s:%d", __FILE__, __LINE__); } while (0)

// ---------------------------------------------------------------- timers ----
// Named host wall-clock accumulators (enabled with FALCATA_TIMETAG=1); the
// device side has its own CUDA-event stage timers in the CUDA learner.
class StageTimer {
 public:
  static StageTimer& Get() { static StageTimer t; return t; }
  bool enabled = false;
  void Add(const std::string& name, double sec) { std::lock_guard<std::mutex> g(mu_); acc_[name] += sec; cnt_[name] += 1; }
  std::string Report() const {
    std::ostringstream os;
    for (auto& kv : acc_) os << kv.first << " costs:\t" << kv.second << " s (" << cnt_.at(kv.first) << " calls)\n";
    return os.str();
  }
  void Clear() { acc_.clear(); cnt_.clear(); }
 private:
  std::mutex mu_;
  std::map<std::string, double> acc_;
  std::map<std::string, int64_t> cnt_;
};

struct ScopedTimer {
  std::string name; std::chrono::steady_clock::time_point t0; bool on;
  explicit ScopedTimer(const char* n) : name(n), on(StageTimer::Get().enabled) { if (on) t0 = std::chrono::steady_clock::now(); }
  ~ScopedTimer() { if (on) StageTimer::Get().Add(name, std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count()); }
};

// --------------------------------------------------------------- strings ----
inline std::string Trim(const std::string& s) {
  size_t b = 0, e = s.size();
  while (b < e && (s[b] == ' ' || s[b] == '\t' || s[b] == '\r' || s[b] == '\n')) ++b;
  while (e > b && (s[e - 1] == ' ' || s[e - 1] == '\t' || s[e - 1] == '\r' || s[e - 1] == '\n')) --e;
  return s.substr(b, e - b);
}

inline std::vector<std::string> Split(const std::string& s, char delim) {
  std::vector<std::string> out; std::string cur;
  for (char c : s) { if (c == delim) { out.push_back(cur); cur.clear(); } else cur.push_back(c); }
  out.push_back(cur);
  return out;
}

inline std::vector<std::string> SplitAny(const std::string& s, const char* delims) {
  std::vector<std::string> out; std::string cur;
  for (char c : s) { if (strchr(delims, c) != nullptr) { if (!cur.empty()) out.push_back(cur); cur.clear(); } else cur.push_back(c); }
  if (!cur.empty()) out.push_back(cur);
  return out;
}

inline bool StartsWith(const std::string& s, const std::string& p) { return s.size() >= p.size() && s.compare(0, p.size(), p) == 0; }

inline std::string ToLower(std::string s) { for (auto& c : s) c = static_cast<char>(tolower(c)); return s; }

// Locale-independent number printing. Doubles that must round-trip (thresholds,
// leaf values) use 17 significant digits; display-only arrays use %g.
inline std::string DoubleToStr17(double v) { char b[64]; snprintf(b, sizeof(b), "%.17g", v); return b; }
inline std::string DoubleToStrG(double v) { char b[64]; snprintf(b, sizeof(b), "%g", v); return b; }

template <typename T> inline std::string NumToStr(T v) { return std::to_string(v); }

template <typename T>
inline std::string JoinInts(const T* a, size_t n, const char* sep = " ") {
  std::string s; s.reserve(n * 4);
  for (size_t i = 0; i < n; ++i) { if (i) s += sep; s += std::to_string(a[i]); }
  return s;
}
inline std::string JoinDoubles17(const double* a, size_t n, const char* sep = " ") {
  std::string s; s.reserve(n * 20);
  for (size_t i = 0; i < n; ++i) { if (i) s += sep; s += DoubleToStr17(a[i]); }
  return s;
}
template <typename T>
inline std::string JoinDoublesG(const T* a, size_t n, const char* sep = " ") {
  std::string s; s.reserve(n * 10);
  for (size_t i = 0; i < n; ++i) { if (i) s += sep; s += DoubleToStrG(static_cast<double>(a[i])); }
  return s;
}

inline double ParseDouble(const std::string& s) {
  std::string t = ToLower(Trim(s));
  if (t == "nan") return std::numeric_limits<double>::quiet_NaN();
  if (t == "inf" || t == "infinity" || t == "+inf") return std::numeric_limits<double>::infinity();
  if (t == "-inf" || t == "-infinity") return -std::numeric_limits<double>::infinity();
  return strtod(t.c_str(), nullptr);
}

template <typename T>
inline std::vector<T> ParseNumArray(const std::string& s, char delim = ' ') {
  std::vector<T> out;
  const char* p = s.c_str();
  while (*p) {
    while (*p == delim || *p == ' ') ++p;
    if (!*p) break;
    const char* q = p;
    while (*q && *q != delim && *q != ' ') ++q;
    std::string tok(p, q - p);
    if (std::is_floating_point<T>::value) out.push_back(static_cast<T>(ParseDouble(tok)));
    else out.push_back(static_cast<T>(strtoll(tok.c_str(), nullptr, 10)));
    p = q;
  }
  return out;
}

// ------------------------------------------------------------- host RNGs ----
// Small linear congruential generator for sampling decisions made on the host
// (bin-construction sample, EFB ordering, extra-trees thresholds).
class Random {
 public:
  Random() : x_(123456789u) {}
  explicit Random(int seed) : x_(static_cast<uint32_t>(seed)) {}
  inline int NextShort(int lo, int hi) { return (RandInt16()) % (hi - lo) + lo; }
  inline int NextInt(int lo, int hi) { return static_cast<int>(RandInt32() % static_cast<uint32_t>(hi - lo)) + lo; }
  inline float NextFloat() { return static_cast<float>(RandInt16()) / 32768.0f; }
  // K sorted distinct indices out of N.
  std::vector<int> Sample(int N, int K) {
    std::vector<int> ret; ret.reserve(K);
    if (K >= N) { for (int i = 0; i < N; ++i) ret.push_back(i); return ret; }
    if (K <= 0) return ret;
    if (K > 1 && K > N / std::log2(static_cast<double>(K))) {
      for (int i = 0; i < N; ++i) {
        double prob = (K - static_cast<int>(ret.size())) / static_cast<double>(N - i);
        if (NextFloat() < prob) ret.push_back(i);
      }
    } else {
      std::vector<int> tmp;
      // Floyd's sampling keeps it O(K log K).
      std::map<int, bool> used;
      for (int r = N - K; r < N; ++r) {
        int v = NextInt(0, r + 1);
        if (used.count(v)) v = r;
        used[v] = true;
      }
      for (auto& kv : used) ret.push_back(kv.first);
    }
    return ret;
  }
 private:
  inline int RandInt16() { x_ = 214013u * x_ + 2531011u; return static_cast<int>((x_ >> 16) & 0x7FFF); }
  inline uint32_t RandInt32() { x_ = 214013u * x_ + 2531011u; return x_ & 0x7FFFFFFF; }
  uint32_t x_;
};

// ------------------------------------------------------------ Philox4x32 ----
// Counter-based generator: the same (key, counter) gives the same 4 words on the
// host and on the device, so stochastic rounding and bagging are reproducible at
// any GPU count and after a resume.
struct Philox4 { uint32_t v[4]; };

FB_HD inline void PhiloxMulHiLo(uint32_t a, uint32_t b, uint32_t* hi, uint32_t* lo) {
  uint64_t p = static_cast<uint64_t>(a) * static_cast<uint64_t>(b);
  *hi = static_cast<uint32_t>(p >> 32); *lo = static_cast<uint32_t>(p);
}

FB_HD inline Philox4 Philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    PhiloxMulHiLo(0xD2511F53u, c0, &hi0, &lo0);
    PhiloxMulHiLo(0xCD9E8D57u, c2, &hi1, &lo1);
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  Philox4 out; out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// Uniform in [0,1) from the top 24 bits: exactly representable in fp32.
FB_HD inline float U01From24(uint32_t w) { return static_cast<float>(w >> 8) * (1.0f / 16777216.0f); }

}  // namespace fb
