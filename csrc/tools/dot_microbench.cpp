// CPU dot-product microbenchmark: how fast one core (and all cores) stream a weight row against an activation vector
// for the formats the CPU expert path uses (fp32, bf16 weights, int8 weights with an fp32 scale, FP4 E2M1 nibbles with an
// E8M0 scale per 32). Prints one `key=value` line per case. Same purpose as the reference's src/csrc/dot_microbench.cpp:
// pick thread counts and see which weight format the host can keep up with.
//   dot_microbench [--k 4096] [--rows 2048] [--iters 20] [--threads N]
#include <immintrin.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

namespace {

const float kE2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

__attribute__((target("avx2,fma"))) float dot_f32(const float* w, const float* x, int K) {
  __m256 acc = _mm256_setzero_ps();
  for (int k = 0; k < K; k += 8) acc = _mm256_fmadd_ps(_mm256_loadu_ps(w + k), _mm256_loadu_ps(x + k), acc);
  float t[8];
  _mm256_storeu_ps(t, acc);
  return ((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7]));
}

__attribute__((target("avx2,fma"))) float dot_bf16(const uint16_t* w, const float* x, int K) {
  __m256 acc = _mm256_setzero_ps();
  for (int k = 0; k < K; k += 8) {
    const __m128i raw = _mm_loadu_si128((const __m128i*)(w + k));
    const __m256 wf = _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(raw), 16));
    acc = _mm256_fmadd_ps(wf, _mm256_loadu_ps(x + k), acc);
  }
  float t[8];
  _mm256_storeu_ps(t, acc);
  return ((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7]));
}

__attribute__((target("avx2,fma"))) float dot_i8(const int8_t* w, float scale, const float* x, int K) {
  __m256 acc = _mm256_setzero_ps();
  for (int k = 0; k < K; k += 8) {
    const __m128i raw = _mm_loadl_epi64((const __m128i*)(w + k));
    acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(raw)), _mm256_loadu_ps(x + k), acc);
  }
  float t[8];
  _mm256_storeu_ps(t, acc);
  return scale * (((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7])));
}

// two codes per byte (low nibble first), one E8M0 scale byte per 32 weights
float dot_fp4(const uint8_t* q, const uint8_t* s, const float* x, int K) {
  float total = 0.f;
  for (int g = 0; g < K / 32; ++g) {
    float acc = 0.f;
    for (int j = 0; j < 16; ++j) {
      const uint8_t b = q[g * 16 + j];
      acc += kE2M1[b & 15] * x[g * 32 + 2 * j] + kE2M1[b >> 4] * x[g * 32 + 2 * j + 1];
    }
    total += acc * std::ldexp(1.f, (int)s[g] - 127);
  }
  return total;
}

template <class F>
double run(int threads, int rows, int iters, F&& row_fn) {
  // every thread owns a contiguous range of rows; returns seconds per pass over all rows
  std::vector<float> sink(threads, 0.f);
  auto pass = [&]() {
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
      pool.emplace_back([&, t]() {
        const int lo = (int)((long long)rows * t / threads), hi = (int)((long long)rows * (t + 1) / threads);
        float acc = 0.f;
        for (int r = lo; r < hi; ++r) acc += row_fn(r);
        sink[t] += acc;
      });
    for (auto& th : pool) th.join();
  };
  pass();   // warm-up
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < iters; ++i) pass();
  const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() / iters;
  volatile float keep = 0.f;
  for (float v : sink) keep = keep + v;
  (void)keep;
  return s;
}

}  // namespace

int main(int argc, char** argv) {
  int K = 4096, rows = 2048, iters = 20, threads = (int)std::thread::hardware_concurrency();
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string f = argv[i];
    const int v = std::atoi(argv[i + 1]);
    if (f == "--k") K = v;
    else if (f == "--rows") rows = v;
    else if (f == "--iters") iters = v;
    else if (f == "--threads") threads = v;
    else {
      std::fprintf(stderr, "usage: dot_microbench [--k K] [--rows R] [--iters N] [--threads T]\n");
      return 2;
    }
  }
  if (K < 32 || K % 32 != 0 || rows < 1 || iters < 1 || threads < 1) {
    std::fprintf(stderr, "k must be a positive multiple of 32; rows, iters and threads positive\n");
    return 2;
  }
  std::mt19937 rng(1);
  std::normal_distribution<float> nd(0.f, 1.f);
  std::vector<float> x(K), wf((size_t)rows * K);
  for (auto& v : x) v = nd(rng);
  for (auto& v : wf) v = nd(rng) * 0.05f;
  std::vector<uint16_t> wb(wf.size());
  std::vector<int8_t> wi(wf.size());
  std::vector<uint8_t> wq(wf.size() / 2), ws(wf.size() / 32, 127);
  for (size_t i = 0; i < wf.size(); ++i) {
    uint32_t u;
    std::memcpy(&u, &wf[i], 4);
    wb[i] = (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
    wi[i] = (int8_t)std::lrint(std::fmax(-127.f, std::fmin(127.f, wf[i] * 400.f)));
  }
  for (auto& b : wq) b = (uint8_t)(rng() & 0xff);

  // agreement of the vector kernels with a plain loop on one row
  double ref = 0.0;
  for (int k = 0; k < K; ++k) ref += (double)wf[k] * x[k];
  const double err = std::fabs(dot_f32(wf.data(), x.data(), K) - ref) / (std::fabs(ref) + 1e-9);
  std::printf("check=dot_f32 rel_err=%.3e ok=%d\n", err, err < 1e-4 ? 1 : 0);

  struct Case { const char* name; double bytes_per_weight; };
  for (int t : {1, threads}) {
    const double sf = run(t, rows, iters, [&](int r) { return dot_f32(wf.data() + (size_t)r * K, x.data(), K); });
    const double sb = run(t, rows, iters, [&](int r) { return dot_bf16(wb.data() + (size_t)r * K, x.data(), K); });
    const double si = run(t, rows, iters, [&](int r) { return dot_i8(wi.data() + (size_t)r * K, 0.0025f, x.data(), K); });
    const double s4 = run(t, rows, iters, [&](int r) { return dot_fp4(wq.data() + (size_t)r * K / 2, ws.data() + (size_t)r * K / 32, x.data(), K); });
    const double n = (double)rows * K;
    std::printf("threads=%d k=%d rows=%d format=f32 gflops=%.2f gbytes_per_s=%.2f\n", t, K, rows, 2 * n / sf / 1e9, 4 * n / sf / 1e9);
    std::printf("threads=%d k=%d rows=%d format=bf16 gflops=%.2f gbytes_per_s=%.2f\n", t, K, rows, 2 * n / sb / 1e9, 2 * n / sb / 1e9);
    std::printf("threads=%d k=%d rows=%d format=int8 gflops=%.2f gbytes_per_s=%.2f\n", t, K, rows, 2 * n / si / 1e9, 1 * n / si / 1e9);
    std::printf("threads=%d k=%d rows=%d format=fp4_e2m1 gflops=%.2f gbytes_per_s=%.2f\n", t, K, rows, 2 * n / s4 / 1e9, (0.5 + 1.0 / 32) * n / s4 / 1e9);
    if (threads == 1) break;
  }
  return 0;
}
