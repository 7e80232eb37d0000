// Host sampler: greedy, temperature and nucleus (top-p) sampling over one row of fp32 logits.
// Role of the reference's cpp_engine/src/sampler.cpp:11-68.
#pragma once

#include <cstdint>

namespace pk {

struct SamplerConfig {
  float temperature = 0.f;   // <= 0: greedy
  float top_p = 1.f;
  int top_k = 0;             // 0: no limit
};

// xorshift64*; `state` must be non-zero
double next_uniform(uint64_t& state);

// Index of the sampled token. Ties in greedy mode go to the lowest index.
int sample_token(const float* logits, int n, const SamplerConfig& cfg, uint64_t& rng_state);

}  // namespace pk
