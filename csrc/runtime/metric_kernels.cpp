// Host reductions behind the streaming regression metrics: sum of squared / absolute differences of
// two float arrays in one pass, vectorised (AVX2 clone chosen at load time) and spread over the
// OpenMP team; the running sums of a metric stay in double precision on the Python side.
// (The reference evaluates its metrics with fused native CPU kernels: README "Metrics" benchmarks.)
#include <cmath>
#include <cstddef>

namespace {

__attribute__((target_clones("avx2,fma", "default")))
double block_sq(const float* a, const float* b, long long n) {
  // eight independent float lanes per accumulator keep the adds pipelined; blocks of 4096 bound
  // the float accumulation error before the sum moves to double
  double total = 0.0;
  for (long long i0 = 0; i0 < n; i0 += 4096) {
    const long long m = n - i0 < 4096 ? n - i0 : 4096;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long i = 0;
    for (; i + 8 <= m; i += 8)
      for (int j = 0; j < 8; ++j) {
        const float d = a[i0 + i + j] - b[i0 + i + j];
        acc[j] += d * d;
      }
    float s = 0.f;
    for (int j = 0; j < 8; ++j) s += acc[j];
    for (; i < m; ++i) {
      const float d = a[i0 + i] - b[i0 + i];
      s += d * d;
    }
    total += s;
  }
  return total;
}

__attribute__((target_clones("avx2,fma", "default")))
double block_abs(const float* a, const float* b, long long n) {
  double total = 0.0;
  for (long long i0 = 0; i0 < n; i0 += 4096) {
    const long long m = n - i0 < 4096 ? n - i0 : 4096;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long i = 0;
    for (; i + 8 <= m; i += 8)
      for (int j = 0; j < 8; ++j) acc[j] += std::fabs(a[i0 + i + j] - b[i0 + i + j]);
    float s = 0.f;
    for (int j = 0; j < 8; ++j) s += acc[j];
    for (; i < m; ++i) s += std::fabs(a[i0 + i] - b[i0 + i]);
    total += s;
  }
  return total;
}

template <typename F>
double reduce(const float* a, const float* b, long long n, F fn) {
  const long long chunk = 1 << 16;
  const long long n_chunks = (n + chunk - 1) / chunk;
  double total = 0.0;
#pragma omp parallel for reduction(+ : total) schedule(static) if (n_chunks > 1)
  for (long long c = 0; c < n_chunks; ++c) {
    const long long lo = c * chunk, len = n - lo < chunk ? n - lo : chunk;
    total += fn(a + lo, b + lo, len);
  }
  return total;
}

}  // namespace

extern "C" {

double tpb_sum_sq_diff_f32(const float* a, const float* b, long long n) { return reduce(a, b, n, block_sq); }
double tpb_sum_abs_diff_f32(const float* a, const float* b, long long n) { return reduce(a, b, n, block_abs); }

}  // extern "C"
