// Host sampler: greedy, temperature, top-k, nucleus (top-p) and min-p sampling over one row of fp32 logits, with the
// frequency / presence / repetition penalties of the OpenAI request applied to the logits first.
// Role of the reference's cpp_engine/src/sampler.cpp:11-68 (greedy, temperature, top-p) and of the penalty and min-p
// handling of src/server/openai.py:559-606.
#pragma once

#include <cstdint>
#include <utility>
#include <vector>

namespace pk {

struct SamplerConfig {
  float temperature = 0.f;   // <= 0: greedy
  float top_p = 1.f;
  int top_k = 0;             // 0: no limit
  float min_p = 0.f;         // drop candidates whose probability is below min_p times the largest one
  float frequency_penalty = 0.f, presence_penalty = 0.f;
  float repetition_penalty = 1.f;
  int logprobs = -1;         // -1: off; k >= 0: the engine reports the log-probability of every token and of the k most likely ones
  // The request's limits, for engines that generate ahead of the server or run on several ranks (every rank must leave a
  // request at the same step): 0 / empty when unknown. The server itself enforces both.
  int max_tokens = 0;
  std::vector<int> stop_token_ids;
  bool has_penalties() const { return frequency_penalty != 0.f || presence_penalty != 0.f || repetition_penalty != 1.f; }
};

// xorshift64*; `state` must be non-zero
double next_uniform(uint64_t& state);

// logits[t] of every token t generated so far: divided (positive) or multiplied (negative) by the repetition penalty,
// then lowered by frequency_penalty * count(t) + presence_penalty. Ids outside [0, n) are ignored.
void apply_penalties(float* logits, int n, const std::vector<int>& generated, const SamplerConfig& cfg);

struct TokenLogprobs {
  float chosen = 0.f;                           // log-probability of the generated token
  std::vector<std::pair<int, float>> top;       // the k most likely tokens, most likely first
};

// log-softmax over `logits`: the entry of `token` and the k largest (ties to the lower id).
void token_logprobs(const float* logits, int n, int token, int k, TokenLogprobs* out);

// Index of the sampled token. Ties in greedy mode go to the lowest index.
int sample_token(const float* logits, int n, const SamplerConfig& cfg, uint64_t& rng_state);

}  // namespace pk
