#include "sampler.hpp"

#include <algorithm>
#include <cmath>
#include <numeric>
#include <vector>

namespace pk {

double next_uniform(uint64_t& s) {
  s ^= s >> 12;
  s ^= s << 25;
  s ^= s >> 27;
  return (double)((s * 0x2545F4914F6CDD1DULL) >> 11) / (double)(1ULL << 53);
}

void apply_penalties(float* logits, int n, const std::vector<int>& generated, const SamplerConfig& cfg) {
  if (!cfg.has_penalties() || generated.empty()) return;
  std::vector<int> ids(generated);
  std::sort(ids.begin(), ids.end());
  for (size_t i = 0; i < ids.size();) {
    size_t j = i;
    while (j < ids.size() && ids[j] == ids[i]) ++j;
    const int t = ids[i];
    if (t >= 0 && t < n) {
      float v = logits[t];
      if (cfg.repetition_penalty != 1.f) v = v > 0.f ? v / cfg.repetition_penalty : v * cfg.repetition_penalty;
      logits[t] = v - cfg.frequency_penalty * (float)(j - i) - cfg.presence_penalty;
    }
    i = j;
  }
}

void token_logprobs(const float* logits, int n, int token, int k, TokenLogprobs* out) {
  out->top.clear();
  out->chosen = 0.f;
  if (n <= 0 || token < 0 || token >= n) return;
  float mx = logits[0];
  for (int i = 1; i < n; ++i) mx = std::max(mx, logits[i]);
  double sum = 0.0;
  for (int i = 0; i < n; ++i) sum += std::exp((double)(logits[i] - mx));
  const double lse = (double)mx + std::log(sum);
  out->chosen = (float)((double)logits[token] - lse);
  k = std::min(k, n);
  if (k <= 0) return;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::partial_sort(order.begin(), order.begin() + k, order.end(),
                    [&](int a, int b) { return logits[a] > logits[b] || (logits[a] == logits[b] && a < b); });
  for (int i = 0; i < k; ++i) out->top.emplace_back(order[i], (float)((double)logits[order[i]] - lse));
}

int sample_token(const float* logits, int n, const SamplerConfig& cfg, uint64_t& rng) {
  if (n <= 0) return -1;
  int best = 0;
  for (int i = 1; i < n; ++i)
    if (logits[i] > logits[best]) best = i;
  if (cfg.temperature <= 0.f) return best;
  // Candidates sorted by logit; top-k / top-p cut the tail before the draw.
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  int keep = n;
  if (cfg.top_k > 0 && cfg.top_k < n) keep = cfg.top_k;
  if (keep < n || cfg.top_p < 1.f || cfg.min_p > 0.f) {
    const int limit = ((cfg.top_p < 1.f || cfg.min_p > 0.f) && keep == n) ? std::min(n, 4096) : keep;   // the head of the distribution is enough
    std::partial_sort(order.begin(), order.begin() + limit, order.end(),
                      [&](int a, int b) { return logits[a] > logits[b] || (logits[a] == logits[b] && a < b); });
    keep = limit;
  }
  const double inv_t = 1.0 / cfg.temperature, mx = logits[best];
  std::vector<double> p(keep);
  double total = 0.0;
  for (int i = 0; i < keep; ++i) {
    p[i] = std::exp((logits[order[i]] - mx) * inv_t);
    total += p[i];
  }
  if (cfg.min_p > 0.f) {
    // candidates are sorted: p[0] is the largest (1 after the shift by the maximum)
    int cut = keep;
    for (int i = 1; i < keep; ++i)
      if (p[i] < (double)cfg.min_p * p[0]) {
        cut = i;
        break;
      }
    keep = cut;
    total = 0.0;
    for (int i = 0; i < keep; ++i) total += p[i];
  }
  if (cfg.top_p < 1.f) {
    // `total` covers only the kept candidates; the tail beyond 4096 sorted entries is negligible.
    double run = 0.0;
    int cut = keep;
    for (int i = 0; i < keep; ++i) {
      run += p[i];
      if (run >= cfg.top_p * total) {
        cut = i + 1;
        break;
      }
    }
    keep = cut;
    total = 0.0;
    for (int i = 0; i < keep; ++i) total += p[i];
  }
  double r = next_uniform(rng) * total;
  for (int i = 0; i < keep; ++i) {
    r -= p[i];
    if (r <= 0.0) return order[i];
  }
  return order[keep - 1];
}

}  // namespace pk
