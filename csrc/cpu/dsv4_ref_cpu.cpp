// Host fp32 reference math of the DeepSeek-V4 block glue, used for parity checks of the device kernels without
// PyTorch: hyper-connection mixes (pre / post / head, with the Sinkhorn-normalised combination matrix), RMSNorm and a
// bf16-weight matvec. Counterpart of the reference's CPU reference math (cpp_engine/src/dsv4_engine.cpp:560-697);
// the Python definitions are in pocketllm_b200/models/deepseek_v4.py (hc_split, hc_pre, hc_post, hc_head).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#define PK_CAPI extern "C" __attribute__((visibility("default")))

namespace {

inline float sigmoid(float v) { return 1.f / (1.f + std::exp(-v)); }

inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// mix [(2 + hc) * hc] of one token -> pre [hc], post [hc], comb [hc, hc]
void hc_split(const float* mix, const float* scale, const float* base, int hc, int iters, float eps, float* pre, float* post, float* comb) {
  for (int i = 0; i < hc; ++i) {
    pre[i] = sigmoid(mix[i] * scale[0] + base[i]) + eps;
    post[i] = 2.f * sigmoid(mix[hc + i] * scale[1] + base[hc + i]);
  }
  for (int i = 0; i < hc; ++i) {   // softmax over the last axis
    float mx = -INFINITY, sum = 0.f;
    for (int j = 0; j < hc; ++j) {
      comb[i * hc + j] = mix[2 * hc + i * hc + j] * scale[2] + base[2 * hc + i * hc + j];
      mx = std::fmax(mx, comb[i * hc + j]);
    }
    for (int j = 0; j < hc; ++j) {
      comb[i * hc + j] = std::exp(comb[i * hc + j] - mx);
      sum += comb[i * hc + j];
    }
    for (int j = 0; j < hc; ++j) comb[i * hc + j] = comb[i * hc + j] / sum + eps;
  }
  auto norm_cols = [&]() {
    for (int j = 0; j < hc; ++j) {
      float sum = 0.f;
      for (int i = 0; i < hc; ++i) sum += comb[i * hc + j];
      for (int i = 0; i < hc; ++i) comb[i * hc + j] /= sum + eps;
    }
  };
  auto norm_rows = [&]() {
    for (int i = 0; i < hc; ++i) {
      float sum = 0.f;
      for (int j = 0; j < hc; ++j) sum += comb[i * hc + j];
      for (int j = 0; j < hc; ++j) comb[i * hc + j] /= sum + eps;
    }
  };
  norm_cols();
  for (int it = 1; it < iters; ++it) {
    norm_rows();
    norm_cols();
  }
}

// mix = (flat(h) @ fn^T) * rsqrt(mean(flat(h)^2) + norm_eps), fn [n_mix, hc * dim]
void hc_mix(const float* h, const float* fn, int hc, int dim, int n_mix, float norm_eps, float* mix) {
  const int F = hc * dim;
  double ss = 0.0;
  for (int i = 0; i < F; ++i) ss += (double)h[i] * h[i];
  const float r = 1.f / std::sqrt((float)(ss / F) + norm_eps);
  for (int m = 0; m < n_mix; ++m) {
    double acc = 0.0;
    for (int i = 0; i < F; ++i) acc += (double)h[i] * fn[(size_t)m * F + i];
    mix[m] = (float)acc * r;
  }
}

}  // namespace

// h [T, hc, dim], fn [(2 + hc) * hc, hc * dim], scale [3], base [(2 + hc) * hc] -> x [T, dim], post [T, hc], comb [T, hc, hc]
PK_CAPI int pk_cpu_hc_pre(const float* h, int T, int hc, int dim, const float* fn, const float* scale, const float* base, int iters, float hc_eps,
                          float norm_eps, float* x, float* post, float* comb) {
  if (T < 0 || hc < 1 || hc > 16 || dim < 1) return 1;
  const int n_mix = (2 + hc) * hc;
  std::vector<float> mix(n_mix), pre(hc);
  for (int t = 0; t < T; ++t) {
    const float* ht = h + (size_t)t * hc * dim;
    hc_mix(ht, fn, hc, dim, n_mix, norm_eps, mix.data());
    hc_split(mix.data(), scale, base, hc, iters, hc_eps, pre.data(), post + (size_t)t * hc, comb + (size_t)t * hc * hc);
    for (int d = 0; d < dim; ++d) {
      float acc = 0.f;
      for (int i = 0; i < hc; ++i) acc += pre[i] * ht[(size_t)i * dim + d];
      x[(size_t)t * dim + d] = acc;
    }
  }
  return 0;
}

// out[t, j, :] = post[t, j] * y[t, :] + sum_i comb[t, i, j] * h[t, i, :]
PK_CAPI int pk_cpu_hc_post(const float* y, const float* h, const float* post, const float* comb, int T, int hc, int dim, float* out) {
  if (T < 0 || hc < 1 || dim < 1) return 1;
  for (int t = 0; t < T; ++t)
    for (int j = 0; j < hc; ++j)
      for (int d = 0; d < dim; ++d) {
        float acc = post[(size_t)t * hc + j] * y[(size_t)t * dim + d];
        for (int i = 0; i < hc; ++i) acc += comb[((size_t)t * hc + i) * hc + j] * h[((size_t)t * hc + i) * dim + d];
        out[((size_t)t * hc + j) * dim + d] = acc;
      }
  return 0;
}

// fn [hc, hc * dim], scale [1], base [hc] -> x [T, dim]
PK_CAPI int pk_cpu_hc_head(const float* h, int T, int hc, int dim, const float* fn, const float* scale, const float* base, float hc_eps,
                           float norm_eps, float* x) {
  if (T < 0 || hc < 1 || hc > 16 || dim < 1) return 1;
  std::vector<float> mix(hc);
  for (int t = 0; t < T; ++t) {
    const float* ht = h + (size_t)t * hc * dim;
    hc_mix(ht, fn, hc, dim, hc, norm_eps, mix.data());
    for (int d = 0; d < dim; ++d) {
      float acc = 0.f;
      for (int i = 0; i < hc; ++i) acc += (sigmoid(mix[i] * scale[0] + base[i]) + hc_eps) * ht[(size_t)i * dim + d];
      x[(size_t)t * dim + d] = acc;
    }
  }
  return 0;
}

// y = x * rsqrt(mean(x^2) + eps) * gamma (gamma may be null)
PK_CAPI int pk_cpu_rmsnorm(const float* x, int T, int dim, const float* gamma, float eps, float* y) {
  if (T < 0 || dim < 1) return 1;
  for (int t = 0; t < T; ++t) {
    double ss = 0.0;
    for (int d = 0; d < dim; ++d) ss += (double)x[(size_t)t * dim + d] * x[(size_t)t * dim + d];
    const float r = 1.f / std::sqrt((float)(ss / dim) + eps);
    for (int d = 0; d < dim; ++d) y[(size_t)t * dim + d] = x[(size_t)t * dim + d] * r * (gamma ? gamma[d] : 1.f);
  }
  return 0;
}

// y[t, n] = sum_k x[t, k] * w[n, k] with bf16 weights (raw 16-bit patterns) and fp32 accumulation
PK_CAPI int pk_cpu_bf16_matvec(const float* x, int T, int K, const uint16_t* w, int N, float* y) {
  if (T < 0 || K < 1 || N < 1) return 1;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int t = 0; t < T; ++t) {
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)x[(size_t)t * K + k] * bf16_to_f32(w[(size_t)n * K + k]);
      y[(size_t)t * N + n] = (float)acc;
    }
  return 0;
}
