// host_selftest: checks of the host plumbing shared by the C++ programs (no GPU needed):
// size / list / shape parsing, iteration budgeting, statistics, append-mode CSV.
#include <cmath>
#include <cstdio>
#include <string>

#include "../common/host_common.hpp"

using namespace tcl::host;

static int failures = 0;
#define EXPECT(cond) do { if (!(cond)) { std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); ++failures; } } while (0)

int main(int argc, char** argv) {
  size_t v = 0;
  EXPECT(parse_bytes("4096", &v) && v == 4096);
  EXPECT(parse_bytes("4K", &v) && v == 4096);
  EXPECT(parse_bytes("1.5M", &v) && v == 1572864);
  EXPECT(parse_bytes("1G", &v) && v == (size_t(1) << 30));
  EXPECT(parse_bytes("64KB", &v) && v == 65536);
  EXPECT(!parse_bytes("", &v) && !parse_bytes("12Q", &v) && !parse_bytes("abc", &v) && !parse_bytes("-5", &v));
  auto parts = split_csv("a,b,,c");
  EXPECT(parts.size() == 3 && parts[2] == "c");
  std::vector<size_t> sizes;
  EXPECT(parse_size_list("128,2K,1M", &sizes) && sizes.size() == 3 && sizes[1] == 2048);
  EXPECT(!parse_size_list("128,zz", &sizes));
  Shape3 s;
  EXPECT(parse_shape("8192", &s) && s.m == 8192 && s.n == 8192 && s.k == 8192);
  EXPECT(parse_shape("32768x8192x1024", &s) && s.m == 32768 && s.n == 8192 && s.k == 1024);
  EXPECT(!parse_shape("0x1x2", &s));
  EXPECT(iters_for_ms(100.0, 10.0) == 100 && iters_for_ms(0.0, 10.0) == 5 && iters_for_ms(1.0, 1e9, 5, 1000) == 1000);
  Stats st = make_stats({5, 1, 4, 2, 3});
  EXPECT(st.n == 5 && st.min == 1 && st.max == 5 && st.p50 == 3 && std::fabs(st.mean - 3.0) < 1e-12);
  std::vector<double> hundred;
  for (int i = 0; i < 100; ++i) hundred.push_back(i);
  st = make_stats(hundred);
  EXPECT(st.p95 == 95 && st.p99 == 99);
  EXPECT(make_stats({}).n == 0);
  if (argc > 1) {
    // append mode: two opens leave two headers
    for (int k = 0; k < 2; ++k) { Csv c; EXPECT(c.open(argv[1], "a,b")); c.row("%d,%d", k, k + 1); }
    std::FILE* f = std::fopen(argv[1], "r");
    int headers = 0, lines = 0;
    char line[64];
    while (f && std::fgets(line, sizeof(line), f)) { ++lines; headers += std::string(line) == "a,b\n"; }
    if (f) std::fclose(f);
    EXPECT(headers == 2 && lines == 4);
  }
  std::printf("host_selftest: %s\n", failures ? "FAIL" : "PASS");
  return failures ? 1 : 0;
}
