// CPU oracle for routed mixture-of-experts blocks with FP4 E2M1 expert weights (two codes
// per byte, low nibble first, one E8M0 scale per 32 values along the input dimension).
//
// y_t = sum_{e in topk(t)} p_te * W2_e ( silu(W1_e x_t) * W3_e x_t )  [+ shared expert]
//
// Role of the reference's AVX2/OpenMP extension (src/csrc/deepseek_cpu_moe_ext.cpp:1778-1999,
// routed_fp4_moe_forward(_raw)): there it is a serving path for CPU-resident experts; here
// it is the numerical oracle for the GPU MoE kernels and the timed CPU baseline of the
// small FP4 MoE block. Plain C++ with OpenMP over experts' output rows, fp32 accumulation.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#define PK_CAPI extern "C" __attribute__((visibility("default")))

namespace {

const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

inline float e8m0(uint8_t c) { return std::ldexp(1.0f, (int)c - 127); }

// One FP4 row (K values = K/2 bytes, K/32 scales) dot an fp32 vector.
float dot_fp4_row(const uint8_t* q, const uint8_t* s, const float* x, int K) {
  float acc = 0.f;
  for (int b = 0; b < K / 32; ++b) {
    float part = 0.f;
    const uint8_t* qb = q + b * 16;
    const float* xb = x + b * 32;
    for (int i = 0; i < 16; ++i) {
      part += kE2M1[qb[i] & 15] * xb[2 * i];
      part += kE2M1[qb[i] >> 4] * xb[2 * i + 1];
    }
    acc += part * e8m0(s[b]);
  }
  return acc;
}

inline float silu(float v) { return v / (1.f + std::exp(-v)); }

struct Fp4Expert {
  const uint8_t *w1, *s1, *w3, *s3, *w2, *s2;
};

void expert_forward(const Fp4Expert& e, const float* x, int H, int I, float limit, float* hidden, float* y, float weight) {
#pragma omp parallel for schedule(static)
  for (int j = 0; j < I; ++j) {
    float g = dot_fp4_row(e.w1 + (size_t)j * H / 2, e.s1 + (size_t)j * H / 32, x, H);
    float u = dot_fp4_row(e.w3 + (size_t)j * H / 2, e.s3 + (size_t)j * H / 32, x, H);
    if (limit > 0.f) {
      g = std::min(g, limit);
      u = std::max(-limit, std::min(u, limit));
    }
    hidden[j] = silu(g) * u;
  }
#pragma omp parallel for schedule(static)
  for (int n = 0; n < H; ++n)
    y[n] += weight * dot_fp4_row(e.w2 + (size_t)n * I / 2, e.s2 + (size_t)n * I / 32, hidden, I);
}

}  // namespace

// score_func: 0 softmax, 1 sigmoid, 2 sqrt(softplus). Selection uses score + bias (bias may
// be null); the weights are the scores of the selected experts, optionally renormalised,
// times route_scale. Ties go to the lower expert id.
PK_CAPI int pk_cpu_route(const float* x, int T, int H, const float* router_w, const float* bias, int E, int topk,
                         int score_func, int norm_topk, float route_scale, int* out_ids, float* out_w) {
  if (topk < 1 || topk > E) return 1;
  std::vector<float> sc(E);
  for (int t = 0; t < T; ++t) {
    const float* xt = x + (size_t)t * H;
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) {
      float a = 0.f;
      for (int k = 0; k < H; ++k) a += router_w[(size_t)e * H + k] * xt[k];
      sc[e] = a;
      mx = std::max(mx, a);
    }
    if (score_func == 0) {
      float sum = 0.f;
      for (int e = 0; e < E; ++e) { sc[e] = std::exp(sc[e] - mx); sum += sc[e]; }
      for (int e = 0; e < E; ++e) sc[e] /= sum;
    } else if (score_func == 1) {
      for (int e = 0; e < E; ++e) sc[e] = 1.f / (1.f + std::exp(-sc[e]));
    } else {
      for (int e = 0; e < E; ++e) sc[e] = std::sqrt(sc[e] > 20.f ? sc[e] : std::log1p(std::exp(sc[e])));
    }
    std::vector<char> used(E, 0);
    float wsum = 0.f;
    for (int j = 0; j < topk; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e) {
        if (used[e]) continue;
        const float v = sc[e] + (bias ? bias[e] : 0.f);
        if (v > bv) { bv = v; best = e; }
      }
      used[best] = 1;
      out_ids[(size_t)t * topk + j] = best;
      out_w[(size_t)t * topk + j] = sc[best];
      wsum += sc[best];
    }
    for (int j = 0; j < topk; ++j) {
      float w = out_w[(size_t)t * topk + j];
      if (norm_topk) w /= (wsum > 0.f ? wsum : 1.f);
      out_w[(size_t)t * topk + j] = w * route_scale;
    }
  }
  return 0;
}

// Expert tensors are contiguous over experts: w13 [E, 2I, H/2] (gate rows then up rows),
// s13 [E, 2I, H/32], w2 [E, H, I/2], s2 [E, H, I/32]. The shared expert (may be null) uses
// the same layout with E = 1 and weight 1. counts[E] receives the tokens routed to each
// expert. y is fp32 [T, H] and is overwritten.
PK_CAPI int pk_cpu_moe_fp4_forward(const float* x, int T, int H, int I, int E, int topk, const int* ids,
                                   const float* weights, const uint8_t* w13, const uint8_t* s13, const uint8_t* w2,
                                   const uint8_t* s2, const uint8_t* sh_w13, const uint8_t* sh_s13,
                                   const uint8_t* sh_w2, const uint8_t* sh_s2, int shared_I, float swiglu_limit,
                                   float* y, int* counts) {
  if (H % 32 || I % 32 || (sh_w13 && shared_I % 32)) return 1;
  std::memset(y, 0, sizeof(float) * (size_t)T * H);
  if (counts) std::memset(counts, 0, sizeof(int) * E);
  std::vector<float> hidden(std::max(I, shared_I));
  for (int t = 0; t < T; ++t) {
    const float* xt = x + (size_t)t * H;
    float* yt = y + (size_t)t * H;
    for (int j = 0; j < topk; ++j) {
      const int e = ids[(size_t)t * topk + j];
      if (e < 0 || e >= E) return 2;
      if (counts) counts[e] += 1;
      Fp4Expert ex{w13 + (size_t)e * 2 * I * H / 2, s13 + (size_t)e * 2 * I * H / 32,
                   w13 + (size_t)e * 2 * I * H / 2 + (size_t)I * H / 2, s13 + (size_t)e * 2 * I * H / 32 + (size_t)I * H / 32,
                   w2 + (size_t)e * H * I / 2, s2 + (size_t)e * H * I / 32};
      expert_forward(ex, xt, H, I, swiglu_limit, hidden.data(), yt, weights[(size_t)t * topk + j]);
    }
    if (sh_w13) {
      Fp4Expert ex{sh_w13, sh_s13, sh_w13 + (size_t)shared_I * H / 2, sh_s13 + (size_t)shared_I * H / 32, sh_w2, sh_s2};
      expert_forward(ex, xt, H, shared_I, swiglu_limit, hidden.data(), yt, 1.f);
    }
  }
  return 0;
}

PK_CAPI void pk_cpu_fp4_dequant(const uint8_t* q, const uint8_t* s, long rows, int K, float* out) {
  for (long r = 0; r < rows; ++r)
    for (int b = 0; b < K / 32; ++b) {
      const float sc = e8m0(s[r * (K / 32) + b]);
      for (int i = 0; i < 16; ++i) {
        const uint8_t v = q[r * (K / 2) + b * 16 + i];
        out[r * K + b * 32 + 2 * i] = kE2M1[v & 15] * sc;
        out[r * K + b * 32 + 2 * i + 1] = kE2M1[v >> 4] * sc;
      }
    }
}

// ---- INT8 routed experts (one fp32 scale per weight row) ------------------------------------------------------------------
// Same layout rules as the FP4 entry: w13 int8 [E, 2I, H] (gate rows then up rows) with s13 fp32 [E, 2I],
// w2 int8 [E, H, I] with s2 fp32 [E, H]. Counterpart of the reference's routed_int8_moe_forward
// (src/csrc/deepseek_cpu_moe_ext.cpp:2000-2115).
namespace {
inline float dot_i8_row(const int8_t* w, float scale, const float* x, int K) {
  float acc = 0.f;
#pragma omp simd reduction(+ : acc)
  for (int k = 0; k < K; ++k) acc += (float)w[k] * x[k];
  return acc * scale;
}
}  // namespace

PK_CAPI int pk_cpu_moe_int8_forward(const float* x, int T, int H, int I, int E, int topk, const int* ids, const float* weights,
                                    const int8_t* w13, const float* s13, const int8_t* w2, const float* s2, float swiglu_limit, float* y,
                                    int* counts) {
  if (T < 0 || H < 1 || I < 1 || topk < 1) return 1;
  std::memset(y, 0, sizeof(float) * (size_t)T * H);
  if (counts) std::memset(counts, 0, sizeof(int) * E);
  std::vector<float> hidden(I);
  for (int t = 0; t < T; ++t) {
    const float* xt = x + (size_t)t * H;
    float* yt = y + (size_t)t * H;
    for (int j = 0; j < topk; ++j) {
      const int e = ids[(size_t)t * topk + j];
      if (e < 0 || e >= E) return 2;
      if (counts) counts[e] += 1;
      const int8_t* g_rows = w13 + (size_t)e * 2 * I * H;
      const int8_t* u_rows = g_rows + (size_t)I * H;
      const float* g_sc = s13 + (size_t)e * 2 * I;
      const float* u_sc = g_sc + I;
      const float rw = weights[(size_t)t * topk + j];
#pragma omp parallel for schedule(static)
      for (int r = 0; r < I; ++r) {
        float g = dot_i8_row(g_rows + (size_t)r * H, g_sc[r], xt, H);
        float u = dot_i8_row(u_rows + (size_t)r * H, u_sc[r], xt, H);
        if (swiglu_limit > 0.f) {
          g = std::min(g, swiglu_limit);
          u = std::max(-swiglu_limit, std::min(u, swiglu_limit));
        }
        hidden[r] = silu(g) * u;
      }
      const int8_t* d_rows = w2 + (size_t)e * H * I;
      const float* d_sc = s2 + (size_t)e * H;
#pragma omp parallel for schedule(static)
      for (int n = 0; n < H; ++n) yt[n] += rw * dot_i8_row(d_rows + (size_t)n * I, d_sc[n], hidden.data(), I);
    }
  }
  return 0;
}

// fp32 [rows, K] -> int8 codes and one scale per row (absmax / 127, round to nearest)
PK_CAPI void pk_cpu_quantize_int8_rows(const float* w, long rows, int K, int8_t* q, float* scale) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r) {
    float amax = 0.f;
    for (int k = 0; k < K; ++k) amax = std::max(amax, std::fabs(w[r * K + k]));
    const float s = amax > 0.f ? amax / 127.f : 1.f;
    scale[r] = s;
    for (int k = 0; k < K; ++k) q[r * K + k] = (int8_t)std::lrint(w[r * K + k] / s);
  }
}
