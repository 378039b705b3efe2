// TEST INFRASTRUCTURE ONLY - never linked into, imported by or executed from the
// product library. This translation unit pulls in the reference project's own CPU
// implementation of the affine quantized path (the file is included from the
// reference checkout at compile time; nothing of it is copied here) and exposes its
// entry points as a small file-driven command line tool.  The tool is used to
//   * pin the C restatement in qref.c (bit-exact comparisons),
//   * generate the golden vectors under tests/golden/,
//   * time the reference CPU path as the reported CPU baseline.
//
// Reference entry points driven (paths relative to the reference project root):
//   quantize<T,U>                 mlx/backend/cpu/quantized.cpp:1148-1211
//   _qmm_dispatch_typed<T>        mlx/backend/cpu/quantized.cpp:340-381
//   gather loop (restated here)   mlx/backend/cpu/quantized.cpp:727-746
//
// Build: see oracle/Makefile (target _ref/ref_oracle).  It must be an executable:
// the unresolved runtime symbols of the reference (array, allocator, scheduler) are
// never reached by the calls below, and are ignored at link time.
//
// Usage (all arrays are raw little-endian files):
//   ref_oracle quantize <f32|f16|bf16> <rows> <K> <group> <bits> w.bin wq.bin s.bin b.bin
//   ref_oracle qmm <dtype> <M> <N> <K> <group> <bits> <transpose> x.bin wq.bin s.bin b.bin y.bin [reps]
//   ref_oracle gather <dtype> <M> <N> <K> <group> <bits> <transpose> <n_idx> x.bin wq.bin s.bin b.bin lhs.bin rhs.bin y.bin
// `qmm` prints "seconds_per_call <t>" on stdout (best of reps).

#include "mlx/backend/cpu/quantized.cpp"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

std::vector<char> slurp(const char* path) {
  FILE* f = std::fopen(path, "rb");
  if (!f) {
    std::fprintf(stderr, "ref_oracle: cannot open %s\n", path);
    std::exit(2);
  }
  std::fseek(f, 0, SEEK_END);
  long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<char> buf(n);
  if (n && std::fread(buf.data(), 1, n, f) != (size_t)n) {
    std::fprintf(stderr, "ref_oracle: short read %s\n", path);
    std::exit(2);
  }
  std::fclose(f);
  return buf;
}

void spill(const char* path, const void* p, size_t n) {
  FILE* f = std::fopen(path, "wb");
  if (!f || (n && std::fwrite(p, 1, n, f) != n)) {
    std::fprintf(stderr, "ref_oracle: cannot write %s\n", path);
    std::exit(2);
  }
  std::fclose(f);
}

template <typename T>
int run_quantize(char** a) {
  size_t rows = std::strtoull(a[0], nullptr, 10);
  size_t K = std::strtoull(a[1], nullptr, 10);
  int group = std::atoi(a[2]);
  int bits = std::atoi(a[3]);
  auto w = slurp(a[4]);
  size_t n = rows * K;
  if (w.size() != n * sizeof(T)) {
    std::fprintf(stderr, "ref_oracle: w size mismatch\n");
    return 2;
  }
  std::vector<uint32_t> wq(n * bits / 32 + 2, 0);
  std::vector<T> s(n / group), b(n / group);
  bool pow2 = (bits & (bits - 1)) == 0;
  // Same U selection as fast::Quantize::eval_cpu (quantized.cpp:1253-1274).
  if (pow2) {
    mlx::core::quantize<T, uint32_t>(
        (const T*)w.data(), wq.data(), s.data(), b.data(), bits, group, n);
  } else {
    mlx::core::quantize<T, uint8_t>(
        (const T*)w.data(), (uint8_t*)wq.data(), s.data(), b.data(), bits, group, n);
  }
  spill(a[5], wq.data(), n * bits / 8);
  spill(a[6], s.data(), s.size() * sizeof(T));
  spill(a[7], b.data(), b.size() * sizeof(T));
  return 0;
}

template <typename T>
int run_qmm(char** a, int extra) {
  int M = std::atoi(a[0]), N = std::atoi(a[1]), K = std::atoi(a[2]);
  int group = std::atoi(a[3]), bits = std::atoi(a[4]);
  bool transpose = std::atoi(a[5]) != 0;
  auto x = slurp(a[6]);
  auto wq = slurp(a[7]);
  auto s = slurp(a[8]);
  auto b = slurp(a[9]);
  int reps = extra > 0 ? std::atoi(a[11]) : 1;
  std::vector<T> y((size_t)M * N);
  double best = 1e30;
  for (int r = 0; r < reps; ++r) {
    auto t0 = std::chrono::steady_clock::now();
    // Pointer-level signature: (..., M, N, K, group_size, bits, transposed).
    mlx::core::_qmm_dispatch_typed<T>(
        y.data(),
        (const T*)x.data(),
        (const uint32_t*)wq.data(),
        (const T*)s.data(),
        (const T*)b.data(),
        M, N, K, group, bits, transpose);
    auto t1 = std::chrono::steady_clock::now();
    best = std::min(best, std::chrono::duration<double>(t1 - t0).count());
  }
  spill(a[10], y.data(), y.size() * sizeof(T));
  std::printf("seconds_per_call %.9f\n", best);
  return 0;
}

template <typename T>
int run_gather(char** a) {
  int M = std::atoi(a[0]), N = std::atoi(a[1]), K = std::atoi(a[2]);
  int group = std::atoi(a[3]), bits = std::atoi(a[4]);
  bool transpose = std::atoi(a[5]) != 0;
  size_t n_idx = std::strtoull(a[6], nullptr, 10);
  auto x = slurp(a[7]);
  auto wq = slurp(a[8]);
  auto s = slurp(a[9]);
  auto b = slurp(a[10]);
  auto lhs = slurp(a[11]);
  auto rhs = slurp(a[12]);
  // Element counts per matrix, as _bs_qmm_dispatch_typed computes them
  // (quantized.cpp:715-716): packed words and groups of one weight matrix.
  size_t w_els = (size_t)N * K * bits / 32;
  size_t g_els = (size_t)N * K / group;
  std::vector<T> y(n_idx * M * N);
  const uint32_t* li = (const uint32_t*)lhs.data();
  const uint32_t* ri = (const uint32_t*)rhs.data();
  for (size_t i = 0; i < n_idx; ++i) {
    mlx::core::_qmm_dispatch_typed<T>(
        y.data() + i * M * N,
        (const T*)x.data() + (size_t)li[i] * M * K,
        (const uint32_t*)wq.data() + (size_t)ri[i] * w_els,
        (const T*)s.data() + (size_t)ri[i] * g_els,
        (const T*)b.data() + (size_t)ri[i] * g_els,
        M, N, K, group, bits, transpose);
  }
  spill(a[13], y.data(), y.size() * sizeof(T));
  return 0;
}

template <typename T>
int dispatch(const std::string& op, char** a, int n) {
  if (op == "quantize" && n == 8) return run_quantize<T>(a);
  if (op == "qmm" && (n == 11 || n == 12)) return run_qmm<T>(a, n - 11);
  if (op == "gather" && n == 14) return run_gather<T>(a);
  std::fprintf(stderr, "ref_oracle: bad arguments for %s (%d)\n", op.c_str(), n);
  return 2;
}

} // namespace

int main(int argc, char** argv) {
  if (argc < 3) {
    std::fprintf(stderr, "usage: ref_oracle <quantize|qmm|gather> <f32|f16|bf16> ...\n");
    return 2;
  }
  std::string op = argv[1], dt = argv[2];
  if (dt == "f32") return dispatch<float>(op, argv + 3, argc - 3);
  if (dt == "f16") return dispatch<mlx::core::float16_t>(op, argv + 3, argc - 3);
  if (dt == "bf16") return dispatch<mlx::core::bfloat16_t>(op, argv + 3, argc - 3);
  std::fprintf(stderr, "ref_oracle: unknown dtype %s\n", dt.c_str());
  return 2;
}
