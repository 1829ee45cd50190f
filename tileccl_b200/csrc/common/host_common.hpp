// Host plumbing shared by the stand-alone benchmark programs: error checks,
// size / list / shape parsing, wall-clock-budgeted iteration counts, summary
// statistics, CSV append files, peer enabling, device description.
//
// Reference parity: comm_comp/common.cuh:28-223 (which the reference copies ad
// hoc into every other program).  One header here, included by all.
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace tcl {
namespace host {

#define TCL_CUDA_CHECK(expr)                                                                   \
  do {                                                                                         \
    cudaError_t err__ = (expr);                                                                \
    if (err__ != cudaSuccess) {                                                                \
      std::fprintf(stderr, "CUDA error %s at %s:%d: %s\n", cudaGetErrorName(err__), __FILE__,  \
                   __LINE__, cudaGetErrorString(err__));                                       \
      std::exit(2);                                                                            \
    }                                                                                          \
  } while (0)

// Soft check: reports and returns false; the caller decides (sticky faults are
// not retried: a failed context is reported once and the program exits).
inline bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  std::fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(e));
  return false;
}

// "4096", "4K", "16M", "1G" (powers of 1024), fractional values allowed ("1.5M").
inline bool parse_bytes(const std::string& s, size_t* out) {
  if (s.empty()) return false;
  char* end = nullptr;
  double v = std::strtod(s.c_str(), &end);
  if (end == s.c_str() || v < 0) return false;
  size_t mult = 1;
  if (*end) {
    switch (*end) {
      case 'k': case 'K': mult = size_t(1) << 10; break;
      case 'm': case 'M': mult = size_t(1) << 20; break;
      case 'g': case 'G': mult = size_t(1) << 30; break;
      default: return false;
    }
    if (end[1] && !((end[1] == 'B' || end[1] == 'b') && !end[2])) return false;
  }
  *out = static_cast<size_t>(v * static_cast<double>(mult));
  return true;
}

inline std::vector<std::string> split_csv(const std::string& s) {
  std::vector<std::string> out;
  size_t pos = 0;
  while (pos <= s.size()) {
    size_t c = s.find(',', pos);
    if (c == std::string::npos) c = s.size();
    if (c > pos) out.push_back(s.substr(pos, c - pos));
    pos = c + 1;
  }
  return out;
}

inline bool parse_size_list(const std::string& s, std::vector<size_t>* out) {
  out->clear();
  for (const auto& t : split_csv(s)) {
    size_t v;
    if (!parse_bytes(t, &v)) return false;
    out->push_back(v);
  }
  return !out->empty();
}

inline bool parse_int_list(const std::string& s, std::vector<int>* out) {
  out->clear();
  for (const auto& t : split_csv(s)) out->push_back(std::atoi(t.c_str()));
  return !out->empty();
}

struct Shape3 {
  int m, n, k;
};
// "8192" -> cube; "MxNxK".
inline bool parse_shape(const std::string& s, Shape3* out) {
  int a = 0, b = 0, c = 0;
  if (std::sscanf(s.c_str(), "%dx%dx%d", &a, &b, &c) == 3) {
    *out = {a, b, c};
    return a > 0 && b > 0 && c > 0;
  }
  size_t v;
  if (!parse_bytes(s, &v) || v == 0) return false;
  *out = {static_cast<int>(v), static_cast<int>(v), static_cast<int>(v)};
  return true;
}

// Iterations that fill `window_ms` given the time of one iteration.
inline int iters_for_ms(double one_iter_us, double window_ms, int lo = 5, int hi = 100000) {
  if (one_iter_us <= 0) return lo;
  double n = window_ms * 1000.0 / one_iter_us;
  return std::max(lo, std::min(hi, static_cast<int>(n)));
}

struct Stats {
  int n = 0;
  double mean = 0, p50 = 0, p95 = 0, p99 = 0, min = 0, max = 0;
};
inline Stats make_stats(std::vector<double> v) {
  Stats s;
  if (v.empty()) return s;
  std::sort(v.begin(), v.end());
  s.n = static_cast<int>(v.size());
  double sum = 0;
  for (double x : v) sum += x;
  s.mean = sum / v.size();
  auto pct = [&](double q) { return v[std::min(v.size() - 1, static_cast<size_t>(q * v.size()))]; };
  s.p50 = pct(0.50);
  s.p95 = pct(0.95);
  s.p99 = pct(0.99);
  s.min = v.front();
  s.max = v.back();
  return s;
}

inline double now_ms() {
  using namespace std::chrono;
  return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

// Append-mode CSV: the header is written again on every open (a file may hold
// several headers; readers skip them).
struct Csv {
  std::FILE* f = nullptr;
  bool open(const std::string& path, const char* header) {
    if (path.empty()) return true;
    f = std::fopen(path.c_str(), "a");
    if (!f) {
      std::fprintf(stderr, "cannot open %s for append\n", path.c_str());
      return false;
    }
    std::fprintf(f, "%s\n", header);
    return true;
  }
  void row(const char* fmt, ...) {
    if (!f) return;
    va_list ap;
    va_start(ap, fmt);
    std::vfprintf(f, fmt, ap);
    va_end(ap);
    std::fputc('\n', f);
    std::fflush(f);
  }
  ~Csv() {
    if (f) std::fclose(f);
  }
};

inline int device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

// Enables peer access between every ordered pair of the first `ndev` devices.
// Returns false (and says which pair) if some pair has no P2P path.
inline bool enable_peer_all(int ndev) {
  for (int a = 0; a < ndev; ++a) {
    TCL_CUDA_CHECK(cudaSetDevice(a));
    for (int b = 0; b < ndev; ++b) {
      if (a == b) continue;
      int ok = 0;
      TCL_CUDA_CHECK(cudaDeviceCanAccessPeer(&ok, a, b));
      if (!ok) {
        std::fprintf(stderr, "no peer access from device %d to %d\n", a, b);
        return false;
      }
      cudaError_t e = cudaDeviceEnablePeerAccess(b, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (e != cudaSuccess) TCL_CUDA_CHECK(e);
    }
  }
  return true;
}

inline void print_device_line(int dev) {
  cudaDeviceProp p;
  TCL_CUDA_CHECK(cudaGetDeviceProperties(&p, dev));
  int clk = 0, l2 = 0;
  cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, dev);
  cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
  std::printf("# device %d: %s, %d SMs, cc %d.%d, %.0f GiB, L2 %.0f MiB, max SM clock %d MHz\n", dev, p.name,
              p.multiProcessorCount, p.major, p.minor, p.totalGlobalMem / 1073741824.0, l2 / 1048576.0,
              clk / 1000);
}

// Minimal flag reader: --name value / --flag.  Unknown flags are an error.
struct Args {
  int argc;
  char** argv;
  int i = 1;
  Args(int c, char** v) : argc(c), argv(v) {}
  bool more() const { return i < argc; }
  std::string flag() { return argv[i++]; }
  bool value(std::string* out) {
    if (i >= argc) return false;
    *out = argv[i++];
    return true;
  }
};

inline double elapsed_us(cudaEvent_t a, cudaEvent_t b) {
  float ms = 0;
  TCL_CUDA_CHECK(cudaEventElapsedTime(&ms, a, b));
  return ms * 1000.0;
}

}  // namespace host
}  // namespace tcl
